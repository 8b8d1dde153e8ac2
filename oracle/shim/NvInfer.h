// TEST INFRASTRUCTURE ONLY.  Stand-in for the TensorRT header the reference's common/refnd.h includes: TensorRT is
// not installed where the reference rulebook / convolution sources are compiled into oracle/_ref, and those sources
// use nothing of it beyond the tensor-descriptor types named in refnd.h:201-243.  Only those names are declared.
#pragma once
#include <cstdint>
#define NV_TENSORRT_MAJOR 8
namespace nvinfer1 {
using AsciiChar = char;
enum class DataType : int32_t { kFLOAT = 0, kHALF = 1, kINT8 = 2, kINT32 = 3, kBOOL = 4 };
enum class TensorFormat : int32_t { kLINEAR = 0 };
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
}  // namespace nvinfer1
