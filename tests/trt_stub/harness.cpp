// TEST INFRASTRUCTURE ONLY.  Compiles the TensorRT plugin shells against tests/trt_stub/NvInfer.h and exposes them to
// the Python tests through a small C interface: the registered creators, and for a plugin deserialised from a data_s
// blob its output count / dims / dtypes, format acceptance, serialisation, clone, workspace size and
// configurePlugin + enqueue (the order TensorRT calls them in).
#include "../../deploy3d_b200/csrc/trt/deploy3d_trt_plugins.cpp"

#ifndef D3D_HAVE_TENSORRT
#error "the stub NvInfer.h must be on the include path"
#endif

#include <cstring>

using namespace nvinfer1;

struct t_desc {  // same fields as d3d_tensor_desc
  int32_t dtype;
  int32_t nb_dims;
  int64_t dims[8];
};

static PluginTensorDesc to_trt(const t_desc& d) {
  PluginTensorDesc t;
  std::memset(&t, 0, sizeof(t));
  t.type = static_cast<DataType>(d.dtype);
  t.format = TensorFormat::kLINEAR;
  t.scale = 1.f;
  t.dims.nbDims = d.nb_dims;
  for (int i = 0; i < d.nb_dims && i < 8; ++i) t.dims.d[i] = static_cast<int32_t>(d.dims[i]);
  return t;
}

extern "C" {
int t_num_creators() { return static_cast<int>(stub_plugin_registry().size()); }
const char* t_creator_name(int i) { return stub_plugin_registry()[i]->getPluginName(); }
const char* t_creator_version(int i) { return stub_plugin_registry()[i]->getPluginVersion(); }
const char* t_creator_namespace(int i) { return stub_plugin_registry()[i]->getPluginNamespace(); }
int t_creator_refuses_fields(int i) {
  IPluginCreator* c = stub_plugin_registry()[i];
  return c->getFieldNames() == nullptr && c->createPlugin("x", nullptr) == nullptr;
}

void* t_deserialize(const char* name, const void* data, size_t len) {
  for (IPluginCreator* c : stub_plugin_registry())
    if (std::strcmp(c->getPluginName(), name) == 0)
      return static_cast<IPluginV2DynamicExt*>(c->deserializePlugin(name, data, len));
  return nullptr;
}
void t_destroy(void* plugin) { static_cast<IPluginV2DynamicExt*>(plugin)->destroy(); }
void* t_clone(void* plugin) { return static_cast<IPluginV2DynamicExt*>(plugin)->clone(); }
const char* t_type(void* plugin) { return static_cast<IPluginV2DynamicExt*>(plugin)->getPluginType(); }
const char* t_version(void* plugin) { return static_cast<IPluginV2DynamicExt*>(plugin)->getPluginVersion(); }
int t_nb_outputs(void* plugin) { return static_cast<IPluginV2DynamicExt*>(plugin)->getNbOutputs(); }
size_t t_serialization_size(void* plugin) { return static_cast<IPluginV2DynamicExt*>(plugin)->getSerializationSize(); }
void t_serialize(void* plugin, void* buffer) { static_cast<IPluginV2DynamicExt*>(plugin)->serialize(buffer); }

// getOutputDimensions with every input dimension a constant; writes nb_dims and dims.
int t_output_dims(void* plugin, int index, const t_desc* in, int n_in, t_desc* out) {
  IExprBuilder eb;
  std::vector<DimsExprs> ins(n_in);
  for (int i = 0; i < n_in; ++i) {
    ins[i].nbDims = in[i].nb_dims;
    for (int d = 0; d < in[i].nb_dims; ++d) ins[i].d[d] = eb.constant(static_cast<int32_t>(in[i].dims[d]));
  }
  DimsExprs r = static_cast<IPluginV2DynamicExt*>(plugin)->getOutputDimensions(index, ins.data(), n_in, eb);
  out->nb_dims = r.nbDims;
  for (int d = 0; d < r.nbDims; ++d) out->dims[d] = r.d[d]->value;
  std::vector<DataType> types(n_in);
  for (int i = 0; i < n_in; ++i) types[i] = static_cast<DataType>(in[i].dtype);
  out->dtype = static_cast<int32_t>(
      static_cast<IPluginV2DynamicExt*>(plugin)->getOutputDataType(index, types.data(), n_in));
  return 0;
}
int t_supports(void* plugin, int pos, const t_desc* inout, int n_in, int n_out, int non_linear) {
  std::vector<PluginTensorDesc> d(n_in + n_out);
  for (int i = 0; i < n_in + n_out; ++i) d[i] = to_trt(inout[i]);
  if (non_linear) d[pos].format = TensorFormat::kCHW32;
  return static_cast<IPluginV2DynamicExt*>(plugin)->supportsFormatCombination(pos, d.data(), n_in, n_out) ? 1 : 0;
}
size_t t_workspace(void* plugin, const t_desc* in, int n_in, const t_desc* out, int n_out) {
  std::vector<PluginTensorDesc> di(n_in), dout(n_out);
  for (int i = 0; i < n_in; ++i) di[i] = to_trt(in[i]);
  for (int i = 0; i < n_out; ++i) dout[i] = to_trt(out[i]);
  return static_cast<IPluginV2DynamicExt*>(plugin)->getWorkspaceSize(di.data(), n_in, dout.data(), n_out);
}
// configurePlugin (static shapes: min = max = the shape) then enqueue, as TensorRT orders them.
int t_configure_and_enqueue(void* plugin, const t_desc* in, int n_in, const t_desc* out, int n_out,
                            const void* const* inputs, void* const* outputs, void* workspace, void* stream) {
  std::vector<PluginTensorDesc> di(n_in), dout(n_out);
  std::vector<DynamicPluginTensorDesc> ci(n_in), co(n_out);
  for (int i = 0; i < n_in; ++i) di[i] = to_trt(in[i]), ci[i].desc = di[i], ci[i].min = di[i].dims, ci[i].max = di[i].dims;
  for (int i = 0; i < n_out; ++i)
    dout[i] = to_trt(out[i]), co[i].desc = dout[i], co[i].min = dout[i].dims, co[i].max = dout[i].dims;
  auto* p = static_cast<IPluginV2DynamicExt*>(plugin);
  p->configurePlugin(ci.data(), n_in, co.data(), n_out);
  return p->enqueue(di.data(), dout.data(), inputs, outputs, workspace, static_cast<cudaStream_t>(stream));
}
}
