// TEST INFRASTRUCTURE ONLY.  TensorRT is not installed where this repository is built and tested, so the plugin
// shells (deploy3d_b200/csrc/trt/deploy3d_trt_plugins.cpp) are compile-checked and exercised against this stand-in:
// it declares, with the signatures of the TensorRT 8 headers, exactly the types and virtual functions the reference's
// plugin classes use (trt/spconv/index_trt.cu:52-290 is the model): a shell that overrides one of them with a wrong
// signature does not compile.  IExprBuilder evaluates eagerly (every input dimension is a constant in the tests) and
// REGISTER_TENSORRT_PLUGIN appends the creator to a list the test harness walks, in place of TensorRT's registry.
#pragma once
#include <cstddef>
#include <cstdint>
#include <deque>
#include <vector>

struct CUstream_st;
typedef CUstream_st* cudaStream_t;

#define NV_TENSORRT_MAJOR 8

namespace nvinfer1 {
using AsciiChar = char;
enum class DataType : int32_t { kFLOAT = 0, kHALF = 1, kINT8 = 2, kINT32 = 3, kBOOL = 4 };
enum class TensorFormat : int32_t { kLINEAR = 0, kCHW2 = 1, kHWC8 = 2, kCHW4 = 3, kCHW16 = 4, kCHW32 = 5 };
enum class DimensionOperation : int32_t {
  kSUM = 0, kPROD = 1, kMAX = 2, kMIN = 3, kSUB = 4, kEQUAL = 5, kLESS = 6, kFLOOR_DIV = 7, kCEIL_DIV = 8
};
class Dims32 {
 public:
  static constexpr int32_t MAX_DIMS{8};
  int32_t nbDims;
  int32_t d[MAX_DIMS];
};
using Dims = Dims32;
struct PluginTensorDesc {
  Dims dims;
  DataType type;
  TensorFormat format;
  float scale;
};
struct DynamicPluginTensorDesc {
  PluginTensorDesc desc;
  Dims min;
  Dims max;
};

class IDimensionExpr {
 public:
  bool isConstant() const noexcept { return true; }
  int32_t getConstantValue() const noexcept { return static_cast<int32_t>(value); }
  int64_t value;
};
class DimsExprs {
 public:
  int32_t nbDims;
  const IDimensionExpr* d[Dims::MAX_DIMS];
};
class IExprBuilder {
  std::deque<IDimensionExpr> nodes_;  // stable addresses

 public:
  const IDimensionExpr* constant(int32_t value) noexcept {
    nodes_.push_back(IDimensionExpr{value});
    return &nodes_.back();
  }
  const IDimensionExpr* operation(DimensionOperation op, const IDimensionExpr& a, const IDimensionExpr& b) noexcept {
    const int64_t x = a.value, y = b.value;
    int64_t r = 0;
    switch (op) {
      case DimensionOperation::kSUM: r = x + y; break;
      case DimensionOperation::kPROD: r = x * y; break;
      case DimensionOperation::kMAX: r = x > y ? x : y; break;
      case DimensionOperation::kMIN: r = x < y ? x : y; break;
      case DimensionOperation::kSUB: r = x - y; break;
      case DimensionOperation::kEQUAL: r = x == y; break;
      case DimensionOperation::kLESS: r = x < y; break;
      case DimensionOperation::kFLOOR_DIV: r = x / y; break;          // positive operands
      case DimensionOperation::kCEIL_DIV: r = (x + y - 1) / y; break;  // positive operands
    }
    nodes_.push_back(IDimensionExpr{r});
    return &nodes_.back();
  }
};

struct PluginField {};
struct PluginFieldCollection {
  int32_t nbFields;
  const PluginField* fields;
};

class IPluginV2 {
 public:
  virtual AsciiChar const* getPluginType() const noexcept = 0;
  virtual AsciiChar const* getPluginVersion() const noexcept = 0;
  virtual int32_t getNbOutputs() const noexcept = 0;
  virtual int32_t initialize() noexcept = 0;
  virtual void terminate() noexcept = 0;
  virtual size_t getSerializationSize() const noexcept = 0;
  virtual void serialize(void* buffer) const noexcept = 0;
  virtual void destroy() noexcept = 0;
  virtual void setPluginNamespace(AsciiChar const* pluginNamespace) noexcept = 0;
  virtual AsciiChar const* getPluginNamespace() const noexcept = 0;

 protected:
  virtual ~IPluginV2() noexcept = default;
};
class IPluginV2Ext : public IPluginV2 {
 public:
  virtual DataType getOutputDataType(int32_t index, DataType const* inputTypes, int32_t nbInputs) const noexcept = 0;
};
class IPluginV2DynamicExt : public IPluginV2Ext {
 public:
  virtual IPluginV2DynamicExt* clone() const noexcept = 0;
  virtual DimsExprs getOutputDimensions(int32_t outputIndex, const DimsExprs* inputs, int32_t nbInputs,
                                        IExprBuilder& exprBuilder) noexcept = 0;
  virtual bool supportsFormatCombination(int32_t pos, const PluginTensorDesc* inOut, int32_t nbInputs,
                                         int32_t nbOutputs) noexcept = 0;
  virtual void configurePlugin(const DynamicPluginTensorDesc* in, int32_t nbInputs, const DynamicPluginTensorDesc* out,
                               int32_t nbOutputs) noexcept = 0;
  virtual size_t getWorkspaceSize(const PluginTensorDesc* inputs, int32_t nbInputs, const PluginTensorDesc* outputs,
                                  int32_t nbOutputs) const noexcept = 0;
  virtual int32_t enqueue(const PluginTensorDesc* inputDesc, const PluginTensorDesc* outputDesc,
                          const void* const* inputs, void* const* outputs, void* workspace,
                          cudaStream_t stream) noexcept = 0;
};
class IPluginCreator {
 public:
  virtual AsciiChar const* getPluginName() const noexcept = 0;
  virtual AsciiChar const* getPluginVersion() const noexcept = 0;
  virtual const PluginFieldCollection* getFieldNames() noexcept = 0;
  virtual IPluginV2* createPlugin(AsciiChar const* name, const PluginFieldCollection* fc) noexcept = 0;
  virtual IPluginV2* deserializePlugin(AsciiChar const* name, const void* serialData,
                                       size_t serialLength) noexcept = 0;
  virtual void setPluginNamespace(AsciiChar const* pluginNamespace) noexcept = 0;
  virtual AsciiChar const* getPluginNamespace() const noexcept = 0;
  virtual ~IPluginCreator() = default;
};

// what getPluginRegistry()->registerCreator collects in TensorRT
inline std::vector<IPluginCreator*>& stub_plugin_registry() {
  static std::vector<IPluginCreator*> creators;
  return creators;
}
template <class T> class PluginRegistrar {
 public:
  PluginRegistrar() { stub_plugin_registry().push_back(&instance); }

 private:
  T instance{};
};
}  // namespace nvinfer1

#define REGISTER_TENSORRT_PLUGIN(name) static nvinfer1::PluginRegistrar<name> pluginRegistrar##name {}
