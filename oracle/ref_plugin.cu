// TEST INFRASTRUCTURE ONLY.  Runs ONE of the reference's TensorRT plugins without TensorRT: the reference source file
// named by REF_PLUGIN_FILE is compiled as it lies (nothing is copied) against oracle/shim/NvInfer.h, the plugin class
// REF_PLUGIN_CLASS is built from its serialised parameters the way IPluginCreator::deserializePlugin does, and its own
// configurePlugin / getWorkspaceSize / enqueue are called, in TensorRT's order, with plain descriptors.  One shared object per plugin
// (oracle/_ref/libref_<name>.so, see the Makefile), because the reference's files reuse kernel names across files.
// `override` is defined away so that the empty base classes of the shim suffice.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cmath>
#include <cstdio>
#include <string>
#define override
#include REF_PLUGIN_FILE
#undef override

struct ref_tensor_desc {  // same fields as the product ABI's d3d_tensor_desc
  int32_t dtype;          // nvinfer1::DataType value
  int32_t nb_dims;
  int64_t dims[8];
};

static nvinfer1::PluginTensorDesc to_trt(const ref_tensor_desc& d) {
  nvinfer1::PluginTensorDesc t{};
  t.type = static_cast<nvinfer1::DataType>(d.dtype);
  t.format = nvinfer1::TensorFormat::kLINEAR;
  t.scale = 1.f;
  t.dims.nbDims = d.nb_dims;
  for (int i = 0; i < d.nb_dims && i < 8; ++i) t.dims.d[i] = (int32_t)d.dims[i];
  return t;
}

extern "C" int ref_plugin_num_outputs(const void* data_s, size_t len) {
  REF_PLUGIN_CLASS plugin(data_s, len);
  return plugin.getNbOutputs();
}

// Returns the plugin's enqueue status, or 1000 + the CUDA error code.  The workspace the plugin asks for is
// allocated and freed here; the stream is synchronised before returning.
extern "C" int ref_plugin_run(const void* data_s, size_t len, const ref_tensor_desc* in, int n_in,
                              const ref_tensor_desc* out, int n_out, const void* const* inputs, void* const* outputs,
                              cudaStream_t stream) {
  REF_PLUGIN_CLASS plugin(data_s, len);
  nvinfer1::PluginTensorDesc din[16], dout[16];
  if (n_in > 16 || n_out > 16) return -100;
  for (int i = 0; i < n_in; ++i) din[i] = to_trt(in[i]);
  for (int i = 0; i < n_out; ++i) dout[i] = to_trt(out[i]);
  nvinfer1::DynamicPluginTensorDesc cin[16], cout[16];  // static shapes: min = max = the shape itself
  for (int i = 0; i < n_in; ++i) cin[i].desc = din[i], cin[i].min = din[i].dims, cin[i].max = din[i].dims;
  for (int i = 0; i < n_out; ++i) cout[i].desc = dout[i], cout[i].min = dout[i].dims, cout[i].max = dout[i].dims;
  plugin.configurePlugin(cin, n_in, cout, n_out);
  size_t ws_bytes = plugin.getWorkspaceSize(din, n_in, dout, n_out);
  void* ws = nullptr;
  if (ws_bytes && cudaMalloc(&ws, ws_bytes) != cudaSuccess) return 1000 + (int)cudaGetLastError();
  int rc = plugin.enqueue(din, dout, inputs, outputs, ws, stream);
  cudaError_t e = cudaStreamSynchronize(stream);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();  // two reference plugins launch on the default stream
  if (e == cudaSuccess) e = cudaGetLastError();
  if (ws) cudaFree(ws);
  if (e != cudaSuccess) return 1000 + (int)e;
  return rc;
}
