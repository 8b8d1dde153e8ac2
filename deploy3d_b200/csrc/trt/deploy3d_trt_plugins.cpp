// TensorRT plugin shells over the C ABI of libdeploy3d_b200.so.
//
// One IPluginV2DynamicExt class and one IPluginCreator per plugin of the reference, under the reference's names
// ("SPConvIdx1d".."SPConvIdx4d", "SPConvMM", "BEVDensify", "SimpleMeanEncoder", "CylinderEncoder", "ScatterTo",
// "GatherBack", "NMS3d", "YoloX3dDecode"), version "2.0", namespace "", registered with REGISTER_TENSORRT_PLUGIN
// exactly as the reference registers its own (trt/spconv/index_trt.cu:287-290, trt/spconv/mm_trt.cu:239,
// trt/spconv/bev_densify_trt.cu:209, trt/voxel_encoder/simple_mean_trt.cu:346, trt/voxel_encoder/cylinder_trt.cu:366,
// trt/point_voxel_mapping/scatter_to.cu:247, gather_back.cu:216, trt/decoder/nms3d.cu:269, yolox3d_decode.cu:443).
// An engine built from the reference's ONNX export (TRT_PluginV2 nodes carrying name_s / data_s) finds these creators
// after this library has been loaded, in place of libdeploy3d.so.
//
// A shell owns nothing but the serialised parameters: the deserialising constructor keeps the data_s bytes and parses
// them with d3d_<op>_parse, serialize() writes the same bytes back, getOutputDimensions states the rule of
// d3d_<op>_output_desc as IExprBuilder expressions (the reference's own expressions), getWorkspaceSize and enqueue
// forward to the C ABI with the descriptors converted field by field.  SPConvMM keeps the library handle that owns the
// weights; clones share it, as the reference's clones share the device weights (mm_trt.cu:75-79), and
// configurePlugin uploads them (mm_trt.cu:127-142).  Unlike the reference's, this SPConvMM asks TensorRT for workspace
// (the output-stationary neighbour table).
//
// Build where TensorRT is installed (it is compiled only when <NvInfer.h> can be included):
//   g++ -std=c++14 -O2 -fPIC -shared deploy3d_trt_plugins.cpp -I<repo>/include -I$TENSORRT/include -I$CUDA/include
//       -L<repo>/deploy3d_b200/libs -ldeploy3d_b200 -lnvinfer -o libdeploy3d.so
#if defined(__has_include)
#if __has_include(<NvInfer.h>)
#define D3D_HAVE_TENSORRT 1
#endif
#endif

#ifdef D3D_HAVE_TENSORRT
#include <NvInfer.h>

#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "deploy3d_b200.h"

namespace d3d_trt {
using namespace nvinfer1;

constexpr const char* kVersion = "2.0";

inline d3d_tensor_desc to_d3d(const PluginTensorDesc& t) {
  d3d_tensor_desc d;
  std::memset(&d, 0, sizeof(d));
  d.dtype = static_cast<int32_t>(t.type);
  d.nb_dims = t.dims.nbDims;
  for (int i = 0; i < t.dims.nbDims && i < D3D_MAX_DIMS; ++i) d.dims[i] = t.dims.d[i];
  return d;
}

struct Descs {
  d3d_tensor_desc in[16], out[32];
  int n_in, n_out;
  Descs(const PluginTensorDesc* i, int ni, const PluginTensorDesc* o, int no) : n_in(ni), n_out(no) {
    for (int k = 0; k < ni && k < 16; ++k) in[k] = to_d3d(i[k]);
    for (int k = 0; k < no && k < 32; ++k) out[k] = to_d3d(o[k]);
  }
};

inline bool linear(const PluginTensorDesc& t, DataType type) {
  return t.format == TensorFormat::kLINEAR && t.type == type;
}

// Everything that is the same in every shell: the kept blob, name / namespace plumbing, trivial life-cycle calls.
class ShellBase : public IPluginV2DynamicExt {
 protected:
  std::vector<uint8_t> blob_;  // data_s as received: serialize() returns it byte for byte
  std::string name_;
  std::string namespace_;

 public:
  ShellBase(const char* name, const void* data, size_t length)
      : blob_(static_cast<const uint8_t*>(data), static_cast<const uint8_t*>(data) + length), name_(name) {}
  size_t getSerializationSize() const noexcept override { return blob_.size(); }
  void serialize(void* buffer) const noexcept override {
    if (!blob_.empty()) std::memcpy(buffer, blob_.data(), blob_.size());
  }
  int32_t initialize() noexcept override { return 0; }
  void terminate() noexcept override {}
  void destroy() noexcept override { delete this; }
  AsciiChar const* getPluginType() const noexcept override { return name_.c_str(); }
  AsciiChar const* getPluginVersion() const noexcept override { return kVersion; }
  void setPluginNamespace(AsciiChar const* ns) noexcept override { namespace_ = ns ? ns : ""; }
  AsciiChar const* getPluginNamespace() const noexcept override { return namespace_.c_str(); }
  void configurePlugin(const DynamicPluginTensorDesc*, int32_t, const DynamicPluginTensorDesc*,
                       int32_t) noexcept override {}
  size_t getWorkspaceSize(const PluginTensorDesc*, int32_t, const PluginTensorDesc*, int32_t) const noexcept override {
    return 0;
  }
};

// ---- SPConvIdx{1..4}d (trt/spconv/index_trt.cu:52-249) --------------------------------------------------------------
class SPConvIdxShell : public ShellBase {
  d3d_spconv_index_params p_;
  bool ok_;

 public:
  SPConvIdxShell(const char* name, const void* data, size_t length) : ShellBase(name, data, length) {
    const int ndim = name[9] - '0';  // "SPConvIdx<N>d"
    ok_ = d3d_spconv_index_parse(ndim, data, length, &p_) == D3D_OK;
  }
  IPluginV2DynamicExt* clone() const noexcept override {
    auto* c = new SPConvIdxShell(name_.c_str(), blob_.data(), blob_.size());
    c->setPluginNamespace(namespace_.c_str());
    return c;
  }
  int32_t getNbOutputs() const noexcept override { return d3d_spconv_index_num_outputs(&p_); }
  DimsExprs getOutputDimensions(int32_t index, const DimsExprs* in, int32_t, IExprBuilder& eb) noexcept override {
    const int nd = p_.ndim;
    DimsExprs r;
    switch (index) {
      case 0: {  // index [3, kVol * (maxNumActIn + 128)]
        int32_t kvol = 1;
        for (int i = 0; i < nd; ++i) kvol *= p_.kernel_size[i];
        r.nbDims = 2;
        r.d[0] = eb.constant(3);
        r.d[1] = eb.operation(DimensionOperation::kPROD,
                              *eb.operation(DimensionOperation::kSUM, *in[0].d[0], *eb.constant(128)),
                              *eb.constant(kvol));
        return r;
      }
      case 1:
      case 3: r.nbDims = 1, r.d[0] = eb.constant(1); return r;
      case 2: r.nbDims = 2, r.d[0] = eb.constant(p_.max_num_act_out), r.d[1] = eb.constant(nd + 1); return r;
      default: {  // outSpatialShape [B, 0, D0', ...]
        r = in[2];
        for (int i = 0; i < nd; ++i) {
          if (p_.transpose) {
            r.d[i + 2] = eb.operation(
                DimensionOperation::kSUM,
                *eb.operation(DimensionOperation::kPROD, *r.d[i + 2], *eb.constant(p_.stride[i])),
                *eb.constant(-p_.stride[i] - 2 * p_.padding[i] + (p_.kernel_size[i] - 1) * p_.dilation[i] +
                             p_.out_padding[i] + 1));
          } else {
            // floor((D + 2p - d(k-1) - 1) / s) + 1 == ceil((D + 2p - d(k-1)) / s) for positive operands
            r.d[i + 2] = eb.operation(
                DimensionOperation::kCEIL_DIV,
                *eb.operation(DimensionOperation::kSUM, *r.d[i + 2],
                              *eb.constant(2 * p_.padding[i] - p_.dilation[i] * (p_.kernel_size[i] - 1))),
                *eb.constant(p_.stride[i]));
          }
        }
        return r;
      }
    }
  }
  DataType getOutputDataType(int32_t, DataType const*, int32_t) const noexcept override { return DataType::kINT32; }
  bool supportsFormatCombination(int32_t pos, const PluginTensorDesc* io, int32_t, int32_t) noexcept override {
    return linear(io[pos], DataType::kINT32);
  }
  size_t getWorkspaceSize(const PluginTensorDesc* in, int32_t n_in, const PluginTensorDesc* out,
                          int32_t n_out) const noexcept override {
    Descs d(in, n_in, out, n_out);
    size_t bytes = 0;
    return d3d_spconv_index_workspace(&p_, d.in, d.n_in, &bytes) == D3D_OK ? bytes : 0;
  }
  int32_t enqueue(const PluginTensorDesc* in_desc, const PluginTensorDesc* out_desc, const void* const* inputs,
                  void* const* outputs, void* workspace, cudaStream_t stream) noexcept override {
    if (!ok_) return -1;
    const int n_out = getNbOutputs();
    Descs d(in_desc, 3, out_desc, n_out);
    size_t bytes = 0;
    if (d3d_spconv_index_workspace(&p_, d.in, d.n_in, &bytes) != D3D_OK) return -1;
    return d3d_spconv_index_enqueue(&p_, d.in, d.n_in, d.out, d.n_out, inputs, outputs, workspace, bytes, stream);
  }
};

// ---- SPConvMM (trt/spconv/mm_trt.cu:39-206) ---------------------------------------------------------------------------
class SPConvMMShell : public IPluginV2DynamicExt {
  std::shared_ptr<d3d_spconv_mm_s> handle_;  // clones share the weights (mm_trt.cu:75-79)
  d3d_spconv_mm_params p_;
  std::string namespace_;

  explicit SPConvMMShell(const std::shared_ptr<d3d_spconv_mm_s>& h) : handle_(h) {
    std::memset(&p_, 0, sizeof(p_));
    if (handle_) d3d_spconv_mm_get_params(handle_.get(), &p_);
  }

 public:
  SPConvMMShell(const void* data, size_t length) {
    std::memset(&p_, 0, sizeof(p_));
    d3d_spconv_mm_t h = nullptr;
    if (d3d_spconv_mm_create(data, length, &h) == D3D_OK) {
      handle_ = std::shared_ptr<d3d_spconv_mm_s>(h, [](d3d_spconv_mm_s* x) { d3d_spconv_mm_destroy(x); });
      d3d_spconv_mm_get_params(h, &p_);
    }
  }
  size_t getSerializationSize() const noexcept override {
    size_t n = 0;
    return handle_ && d3d_spconv_mm_serialize(handle_.get(), nullptr, &n) == D3D_OK ? n : 0;
  }
  void serialize(void* buffer) const noexcept override {
    size_t n = getSerializationSize();
    if (handle_ && n) d3d_spconv_mm_serialize(handle_.get(), buffer, &n);
  }
  IPluginV2DynamicExt* clone() const noexcept override {
    auto* c = new SPConvMMShell(handle_);
    c->setPluginNamespace(namespace_.c_str());
    return c;
  }
  int32_t initialize() noexcept override { return 0; }
  void terminate() noexcept override {}
  void destroy() noexcept override { delete this; }
  int32_t getNbOutputs() const noexcept override { return 1; }
  DimsExprs getOutputDimensions(int32_t, const DimsExprs*, int32_t, IExprBuilder& eb) noexcept override {
    DimsExprs r;
    r.nbDims = 2, r.d[0] = eb.constant(p_.max_num_act_out), r.d[1] = eb.constant(p_.out_channels);
    return r;
  }
  DataType getOutputDataType(int32_t, DataType const* in, int32_t) const noexcept override { return in[0]; }
  bool supportsFormatCombination(int32_t pos, const PluginTensorDesc* io, int32_t, int32_t) noexcept override {
    switch (pos) {
      // the reference takes half only (mm_trt.cu:111); float is accepted as well (its docstring allows it, :87)
      case 0: return linear(io[pos], DataType::kHALF) || linear(io[pos], DataType::kFLOAT);
      case 5: return linear(io[pos], io[0].type);
      default: return linear(io[pos], DataType::kINT32);
    }
  }
  AsciiChar const* getPluginType() const noexcept override { return "SPConvMM"; }
  AsciiChar const* getPluginVersion() const noexcept override { return kVersion; }
  void setPluginNamespace(AsciiChar const* ns) noexcept override { namespace_ = ns ? ns : ""; }
  AsciiChar const* getPluginNamespace() const noexcept override { return namespace_.c_str(); }
  void configurePlugin(const DynamicPluginTensorDesc* in, int32_t, const DynamicPluginTensorDesc*,
                       int32_t) noexcept override {
    // weights to the compute dtype and onto the device, once per dtype (mm_trt.cu:127-142); enqueue allocates nothing
    if (handle_) d3d_spconv_mm_configure(handle_.get(), static_cast<int>(in[0].desc.type));
  }
  size_t getWorkspaceSize(const PluginTensorDesc* in, int32_t n_in, const PluginTensorDesc* out,
                          int32_t n_out) const noexcept override {
    if (!handle_) return 0;
    Descs d(in, n_in, out, n_out);
    size_t bytes = 0;
    return d3d_spconv_mm_workspace(handle_.get(), d.in, d.n_in, &bytes) == D3D_OK ? bytes : 0;
  }
  int32_t enqueue(const PluginTensorDesc* in_desc, const PluginTensorDesc* out_desc, const void* const* inputs,
                  void* const* outputs, void* workspace, cudaStream_t stream) noexcept override {
    if (!handle_) return -1;
    Descs d(in_desc, 5, out_desc, 1);
    size_t bytes = 0;
    if (d3d_spconv_mm_workspace(handle_.get(), d.in, d.n_in, &bytes) != D3D_OK) return -1;
    return d3d_spconv_mm_enqueue(handle_.get(), d.in, d.n_in, d.out, d.n_out, inputs, outputs, workspace, bytes,
                                 stream);
  }
};

// ---- the plugins whose parameters are plain structs ---------------------------------------------------------------
// Traits: parameter struct, C-ABI entry points, input / output counts.
template <class Params> struct PodOps {
  int (*parse)(const void*, size_t, Params*);
  int (*workspace)(const Params*, const d3d_tensor_desc*, int, size_t*);  // may be null: no workspace
  int (*enqueue)(const Params*, const d3d_tensor_desc*, int, const d3d_tensor_desc*, int, const void* const*,
                 void* const*, void*, size_t, void*);
};

template <class Derived, class Params> class PodShell : public ShellBase {
 protected:
  Params p_;
  bool ok_;

 public:
  PodShell(const char* name, const void* data, size_t length) : ShellBase(name, data, length) {
    std::memset(&p_, 0, sizeof(p_));
    ok_ = Derived::ops().parse(data, length, &p_) == D3D_OK;
  }
  IPluginV2DynamicExt* clone() const noexcept override {
    auto* c = new Derived(blob_.data(), blob_.size());
    c->setPluginNamespace(namespace_.c_str());
    return c;
  }
  size_t getWorkspaceSize(const PluginTensorDesc* in, int32_t n_in, const PluginTensorDesc* out,
                          int32_t n_out) const noexcept override {
    if (!Derived::ops().workspace) return 0;
    Descs d(in, n_in, out, n_out);
    size_t bytes = 0;
    return Derived::ops().workspace(&p_, d.in, d.n_in, &bytes) == D3D_OK ? bytes : 0;
  }
  int32_t enqueue(const PluginTensorDesc* in_desc, const PluginTensorDesc* out_desc, const void* const* inputs,
                  void* const* outputs, void* workspace, cudaStream_t stream) noexcept override {
    if (!ok_) return -1;
    Descs d(in_desc, Derived::kInputs, out_desc, this->getNbOutputs());
    size_t bytes = 0;
    if (Derived::ops().workspace && Derived::ops().workspace(&p_, d.in, d.n_in, &bytes) != D3D_OK) return -1;
    return Derived::ops().enqueue(&p_, d.in, d.n_in, d.out, d.n_out, inputs, outputs, workspace, bytes, stream);
  }
};

// BEVDensify (trt/spconv/bev_densify_trt.cu:52-178)
class BEVDensifyShell : public PodShell<BEVDensifyShell, d3d_bev_densify_params> {
 public:
  static constexpr int kInputs = 4;
  static const PodOps<d3d_bev_densify_params>& ops() {
    static const PodOps<d3d_bev_densify_params> o = {d3d_bev_densify_parse, d3d_bev_densify_workspace,
                                                     d3d_bev_densify_enqueue};
    return o;
  }
  BEVDensifyShell(const void* data, size_t length) : PodShell("BEVDensify", data, length) {}
  int32_t getNbOutputs() const noexcept override { return 1; }
  DimsExprs getOutputDimensions(int32_t, const DimsExprs* in, int32_t, IExprBuilder& eb) noexcept override {
    DimsExprs r;
    r.nbDims = 4, r.d[0] = in[3].d[0], r.d[1] = eb.constant(p_.out_channels), r.d[2] = in[3].d[3], r.d[3] = in[3].d[4];
    return r;
  }
  DataType getOutputDataType(int32_t, DataType const* in, int32_t) const noexcept override { return in[0]; }
  bool supportsFormatCombination(int32_t pos, const PluginTensorDesc* io, int32_t, int32_t) noexcept override {
    switch (pos) {
      case 0: return linear(io[pos], DataType::kFLOAT) || linear(io[pos], DataType::kHALF);
      case 1:
      case 2:
      case 3: return linear(io[pos], DataType::kINT32);
      default: return linear(io[pos], io[0].type);
    }
  }
};

// SimpleMeanEncoder (trt/voxel_encoder/simple_mean_trt.cu:181-314)
class SimpleMeanEncoderShell : public PodShell<SimpleMeanEncoderShell, d3d_voxel_encoder_params> {
 public:
  static constexpr int kInputs = 4;
  static const PodOps<d3d_voxel_encoder_params>& ops() {
    static const PodOps<d3d_voxel_encoder_params> o = {d3d_simple_mean_encoder_parse,
                                                       d3d_simple_mean_encoder_workspace,
                                                       d3d_simple_mean_encoder_enqueue};
    return o;
  }
  SimpleMeanEncoderShell(const void* data, size_t length) : PodShell("SimpleMeanEncoder", data, length) {}
  int32_t getNbOutputs() const noexcept override { return 3; }
  DimsExprs getOutputDimensions(int32_t index, const DimsExprs* in, int32_t, IExprBuilder& eb) noexcept override {
    DimsExprs r;
    switch (index) {
      case 0: r = in[0], r.d[0] = eb.constant(p_.max_num_act_out); return r;
      case 1: r.nbDims = 2, r.d[0] = eb.constant(p_.max_num_act_out), r.d[1] = eb.constant(4); return r;
      default: r.nbDims = 1, r.d[0] = eb.constant(1); return r;
    }
  }
  DataType getOutputDataType(int32_t index, DataType const* in, int32_t) const noexcept override {
    return index == 0 ? in[0] : DataType::kINT32;
  }
  bool supportsFormatCombination(int32_t pos, const PluginTensorDesc* io, int32_t, int32_t) noexcept override {
    switch (pos) {
      case 0: return linear(io[pos], DataType::kFLOAT);
      case 1:
      case 3:
      case 5:
      case 6: return linear(io[pos], DataType::kINT32);
      default: return linear(io[pos], io[0].type);  // voxelConfig, outFeats
    }
  }
};

// CylinderEncoder (trt/voxel_encoder/cylinder_trt.cu:187-333)
class CylinderEncoderShell : public PodShell<CylinderEncoderShell, d3d_voxel_encoder_params> {
 public:
  static constexpr int kInputs = 4;
  static const PodOps<d3d_voxel_encoder_params>& ops() {
    static const PodOps<d3d_voxel_encoder_params> o = {d3d_cylinder_encoder_parse, d3d_cylinder_encoder_workspace,
                                                       d3d_cylinder_encoder_enqueue};
    return o;
  }
  CylinderEncoderShell(const void* data, size_t length) : PodShell("CylinderEncoder", data, length) {}
  int32_t getNbOutputs() const noexcept override { return 5; }
  DimsExprs getOutputDimensions(int32_t index, const DimsExprs* in, int32_t, IExprBuilder& eb) noexcept override {
    DimsExprs r;
    switch (index) {
      case 0:
        r.nbDims = 2, r.d[0] = in[0].d[0];
        r.d[1] = eb.operation(DimensionOperation::kSUM, *in[0].d[1], *eb.constant(5));
        return r;
      case 1: r.nbDims = 1, r.d[0] = in[0].d[0]; return r;
      case 2: r.nbDims = 1, r.d[0] = eb.constant(p_.max_num_act_out); return r;
      case 3: r.nbDims = 2, r.d[0] = eb.constant(p_.max_num_act_out), r.d[1] = eb.constant(4); return r;
      default: r.nbDims = 1, r.d[0] = eb.constant(1); return r;
    }
  }
  DataType getOutputDataType(int32_t index, DataType const* in, int32_t) const noexcept override {
    return index == 0 ? in[0] : DataType::kINT32;
  }
  bool supportsFormatCombination(int32_t pos, const PluginTensorDesc* io, int32_t, int32_t) noexcept override {
    switch (pos) {
      case 0: return linear(io[pos], DataType::kFLOAT);
      case 1:
      case 3:
      case 5:
      case 6:
      case 7:
      case 8: return linear(io[pos], DataType::kINT32);
      default: return linear(io[pos], io[0].type);  // cylinderConfig, outFeats
    }
  }
};

// ScatterTo (trt/point_voxel_mapping/scatter_to.cu:120-214)
class ScatterToShell : public PodShell<ScatterToShell, d3d_scatter_to_params> {
 public:
  static constexpr int kInputs = 3;
  static const PodOps<d3d_scatter_to_params>& ops() {
    static const PodOps<d3d_scatter_to_params> o = {d3d_scatter_to_parse, nullptr, d3d_scatter_to_enqueue};
    return o;
  }
  ScatterToShell(const void* data, size_t length) : PodShell("ScatterTo", data, length) {}
  int32_t getNbOutputs() const noexcept override { return 1; }
  DimsExprs getOutputDimensions(int32_t, const DimsExprs* in, int32_t, IExprBuilder&) noexcept override {
    DimsExprs r;
    r.nbDims = 2, r.d[0] = in[2].d[0], r.d[1] = in[0].d[1];
    return r;
  }
  DataType getOutputDataType(int32_t, DataType const* in, int32_t) const noexcept override { return in[0]; }
  bool supportsFormatCombination(int32_t pos, const PluginTensorDesc* io, int32_t, int32_t) noexcept override {
    switch (pos) {
      case 0: return linear(io[pos], DataType::kFLOAT);
      case 3: return linear(io[pos], io[0].type);
      default: return linear(io[pos], DataType::kINT32);
    }
  }
};

// GatherBack (trt/point_voxel_mapping/gather_back.cu:77-184)
class GatherBackShell : public PodShell<GatherBackShell, d3d_gather_back_params> {
 public:
  static constexpr int kInputs = 2;
  static const PodOps<d3d_gather_back_params>& ops() {
    static const PodOps<d3d_gather_back_params> o = {d3d_gather_back_parse, nullptr, d3d_gather_back_enqueue};
    return o;
  }
  GatherBackShell(const void* data, size_t length) : PodShell("GatherBack", data, length) {}
  int32_t getNbOutputs() const noexcept override { return 1; }
  DimsExprs getOutputDimensions(int32_t, const DimsExprs* in, int32_t, IExprBuilder&) noexcept override {
    DimsExprs r = in[0];
    r.d[0] = in[1].d[0];
    return r;
  }
  DataType getOutputDataType(int32_t, DataType const* in, int32_t) const noexcept override { return in[0]; }
  bool supportsFormatCombination(int32_t pos, const PluginTensorDesc* io, int32_t, int32_t) noexcept override {
    switch (pos) {
      case 0: return linear(io[pos], DataType::kFLOAT);
      case 2: return linear(io[pos], io[0].type);
      default: return linear(io[pos], DataType::kINT32);
    }
  }
};

// NMS3d (trt/decoder/nms3d.cu:135-236): no data_s; the IoU threshold is the reference's constant 0.1 (:138)
class NMS3dShell : public PodShell<NMS3dShell, d3d_nms3d_params> {
 public:
  static constexpr int kInputs = 2;
  static const PodOps<d3d_nms3d_params>& ops() {
    static const PodOps<d3d_nms3d_params> o = {d3d_nms3d_parse, d3d_nms3d_workspace, d3d_nms3d_enqueue};
    return o;
  }
  NMS3dShell(const void* data, size_t length) : PodShell("NMS3d", data, length) {}
  int32_t getNbOutputs() const noexcept override { return 1; }
  DimsExprs getOutputDimensions(int32_t, const DimsExprs* in, int32_t, IExprBuilder&) noexcept override {
    return in[0];
  }
  DataType getOutputDataType(int32_t, DataType const*, int32_t) const noexcept override { return DataType::kFLOAT; }
  bool supportsFormatCombination(int32_t pos, const PluginTensorDesc* io, int32_t, int32_t) noexcept override {
    return linear(io[pos], DataType::kFLOAT);
  }
};

// YoloX3dDecode (trt/decoder/yolox3d_decode.cu:147-412)
class YoloX3dDecodeShell : public PodShell<YoloX3dDecodeShell, d3d_yolox3d_decode_params> {
 public:
  static constexpr int kInputs = 3;
  static const PodOps<d3d_yolox3d_decode_params>& ops() {
    static const PodOps<d3d_yolox3d_decode_params> o = {d3d_yolox3d_decode_parse, d3d_yolox3d_decode_workspace,
                                                        d3d_yolox3d_decode_enqueue};
    return o;
  }
  YoloX3dDecodeShell(const void* data, size_t length) : PodShell("YoloX3dDecode", data, length) {}
  int32_t getNbOutputs() const noexcept override { return d3d_yolox3d_decode_num_outputs(&p_); }
  DimsExprs getOutputDimensions(int32_t index, const DimsExprs* in, int32_t, IExprBuilder& eb) noexcept override {
    const IDimensionExpr* cells = eb.operation(DimensionOperation::kPROD, *in[0].d[2], *in[0].d[3]);
    const IDimensionExpr* k = eb.operation(DimensionOperation::kMIN, *cells, *eb.constant(p_.topk));
    DimsExprs r;
    r.nbDims = 2, r.d[0] = in[0].d[0], r.d[1] = k;
    if (index % 3 == 2) {  // boxes: the two direction channels are folded into the yaw
      r.nbDims = 3;
      r.d[2] = eb.operation(DimensionOperation::kSUB, *in[1].d[1], *eb.constant(2));
    }
    return r;
  }
  DataType getOutputDataType(int32_t index, DataType const*, int32_t) const noexcept override {
    return index % 3 == 0 ? DataType::kINT32 : DataType::kFLOAT;
  }
  bool supportsFormatCombination(int32_t pos, const PluginTensorDesc* io, int32_t, int32_t) noexcept override {
    switch (pos) {
      case 0: return linear(io[pos], DataType::kFLOAT) || linear(io[pos], DataType::kHALF);
      case 1: return linear(io[pos], io[0].type);
      case 2: return linear(io[pos], DataType::kFLOAT);
      default: return linear(io[pos], (pos - 3) % 3 == 0 ? DataType::kINT32 : DataType::kFLOAT);
    }
  }
};

// ---- creators -----------------------------------------------------------------------------------------------------
// Only deserializePlugin is ever used: the ONNX parser creates TRT_PluginV2 nodes from (name_s, data_s); the
// reference's creators return null from createPlugin / getFieldNames as well (index_trt.cu:262-269).
template <class Make> class Creator : public IPluginCreator {
  std::string namespace_;

 public:
  const char* getPluginName() const noexcept override { return Make::name(); }
  const char* getPluginVersion() const noexcept override { return kVersion; }
  const PluginFieldCollection* getFieldNames() noexcept override { return nullptr; }
  IPluginV2DynamicExt* createPlugin(const char*, const PluginFieldCollection*) noexcept override { return nullptr; }
  IPluginV2DynamicExt* deserializePlugin(const char*, const void* data, size_t length) noexcept override {
    IPluginV2DynamicExt* obj = Make::make(data, length);
    obj->setPluginNamespace(namespace_.c_str());
    return obj;
  }
  void setPluginNamespace(const char* ns) noexcept override { namespace_ = ns ? ns : ""; }
  const char* getPluginNamespace() const noexcept override { return namespace_.c_str(); }
};

#define D3D_TRT_CREATOR(Tag, Name, Expr)                                                          \
  struct Tag##Make {                                                                              \
    static const char* name() { return Name; }                                                    \
    static IPluginV2DynamicExt* make(const void* data, size_t length) { return Expr; }            \
  };                                                                                              \
  using Tag##PluginCreator = Creator<Tag##Make>;                                                  \
  REGISTER_TENSORRT_PLUGIN(Tag##PluginCreator)

D3D_TRT_CREATOR(SPConvIdx1d, "SPConvIdx1d", new SPConvIdxShell("SPConvIdx1d", data, length));
D3D_TRT_CREATOR(SPConvIdx2d, "SPConvIdx2d", new SPConvIdxShell("SPConvIdx2d", data, length));
D3D_TRT_CREATOR(SPConvIdx3d, "SPConvIdx3d", new SPConvIdxShell("SPConvIdx3d", data, length));
D3D_TRT_CREATOR(SPConvIdx4d, "SPConvIdx4d", new SPConvIdxShell("SPConvIdx4d", data, length));
D3D_TRT_CREATOR(SPConvMM, "SPConvMM", new SPConvMMShell(data, length));
D3D_TRT_CREATOR(BEVDensify, "BEVDensify", new BEVDensifyShell(data, length));
D3D_TRT_CREATOR(SimpleMeanEncoder, "SimpleMeanEncoder", new SimpleMeanEncoderShell(data, length));
D3D_TRT_CREATOR(CylinderEncoder, "CylinderEncoder", new CylinderEncoderShell(data, length));
D3D_TRT_CREATOR(ScatterTo, "ScatterTo", new ScatterToShell(data, length));
D3D_TRT_CREATOR(GatherBack, "GatherBack", new GatherBackShell(data, length));
D3D_TRT_CREATOR(NMS3d, "NMS3d", new NMS3dShell(data, length));
D3D_TRT_CREATOR(YoloX3dDecode, "YoloX3dDecode", new YoloX3dDecodeShell(data, length));

}  // namespace d3d_trt
#endif  // D3D_HAVE_TENSORRT
