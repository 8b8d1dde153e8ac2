// TEST INFRASTRUCTURE ONLY.  Stand-in for the TensorRT header the reference's sources include: TensorRT is not
// installed where those sources are compiled into oracle/_ref.  Only the names the reference's files mention are
// declared, with just enough shape for its plugin classes to compile: tensor descriptors (common/refnd.h:201-243),
// empty plugin base classes (the wrappers compile the reference's files with `override` defined away, so nothing
// virtual is needed), and the shape-expression types getOutputDimensions mentions, which are never called here.
#pragma once
#include <cstddef>
#include <cstdint>
#define NV_TENSORRT_MAJOR 8
#define REGISTER_TENSORRT_PLUGIN(name)
namespace nvinfer1 {
using AsciiChar = char;
enum class DataType : int32_t { kFLOAT = 0, kHALF = 1, kINT8 = 2, kINT32 = 3, kBOOL = 4 };
enum class TensorFormat : int32_t { kLINEAR = 0 };
enum class DimensionOperation : int32_t { kSUM, kPROD, kMAX, kMIN, kSUB, kEQUAL, kLESS, kFLOOR_DIV, kCEIL_DIV };
struct Dims {
  int32_t nbDims;
  int32_t d[8];
};
struct PluginTensorDesc {
  Dims dims;
  DataType type;
  TensorFormat format;
  float scale;
};
struct DynamicPluginTensorDesc {
  PluginTensorDesc desc;
  Dims min, max;
};
class IDimensionExpr {};
struct DimsExprs {
  int32_t nbDims;
  const IDimensionExpr* d[8];
};
class IExprBuilder {
 public:
  const IDimensionExpr* constant(int32_t value);
  const IDimensionExpr* operation(DimensionOperation op, const IDimensionExpr& first, const IDimensionExpr& second);
};
struct PluginField {};
struct PluginFieldCollection {
  int32_t nbFields;
  const PluginField* fields;
};
class IPluginV2 {};
class IPluginV2Ext : public IPluginV2 {};
class IPluginV2DynamicExt : public IPluginV2Ext {};
class IPluginCreator {};
}  // namespace nvinfer1
