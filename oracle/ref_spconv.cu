// TEST INFRASTRUCTURE ONLY.  C wrappers around the reference's own GPU rulebook builders
// (spconv::func::createSparse{SubM,Conv}Index<3, int32_t>, trt/spconv/index.cu:253-476) and its indexed
// convolution (spconv::func::indexedSpConv<Config>, trt/spconv/mm.h:35-71 with the three configurations of
// trt/spconv/mm_trt.cu:47-49), compiled for sm_100a from the sources where they lie (nothing is copied) into
// oracle/_ref/libref_spconv.so.  The calls below repeat what SPConvIdxPlugin::enqueue (index_trt.cu:189-248) and
// SPConvMMPlugin::enqueue (mm_trt.cu:146-205) do with their tensors.  Used by the GPU parity tests to pin the CPU
// oracle and the product kernels to the reference's results; never linked into the product library.
#include <cuda_fp16.h>
#include <cmath>
#include "spconv/index.h"
#ifdef REF_WITH_MM
#include "spconv/mm.h"
#endif

using utils::nd::Ref1D;
using utils::nd::Ref2D;
using utils::nd::Ref3D;
using utils::nd::Size;
using utils::nd::Vec;

namespace {
Vec<3, int32_t> vec3(const int32_t* v) {
  Vec<3, int32_t> r;
  for (int i = 0; i < 3; ++i) r[i] = v[i];
  return r;
}
}  // namespace

// Workspace bytes for num_act_in live inputs (index_trt.cu:228-229, 239-240).
extern "C" size_t ref_spconv_index_workspace(int subm, int32_t num_act_in, const int32_t* ksize) {
  if (num_act_in <= 0) return 0;
  if (subm) return spconv::func::createSparseSubMIndexMalloc<3, int32_t>(utils::GPU(), num_act_in, vec3(ksize));
  return spconv::func::createSparseConvIndexMalloc<3, int32_t>(utils::GPU(), num_act_in, vec3(ksize));
}

// coors: device [num_act_in, 4]; index: device [3, row_len]; out_coors: device [max_num_act_out, 4];
// out_shape: {B, Z, Y, X} of the output grid.  Returns the CUDA error code (after synchronising the stream when sync != 0).
extern "C" int ref_spconv_index_run(int subm, int transpose, const int32_t* coors, int32_t num_act_in,
                                    const int32_t* ksize, const int32_t* stride, const int32_t* padding,
                                    const int32_t* dilation, const int64_t* out_shape, int32_t max_num_act_out,
                                    int64_t row_len, int32_t* index, int32_t* num_index, int32_t* out_coors,
                                    int32_t* num_act_out, void* workspace, size_t ws_bytes, int sync,
                                    cudaStream_t stream) {
  Ref2D<int32_t> in_coors(const_cast<int32_t*>(coors), {num_act_in, 4});
  Ref1D<int32_t> gather(index, {row_len}), scatter(index + row_len, {row_len}), offset(index + 2 * row_len, {row_len});
  Size<4>::index_vec_t shape_vec;
  for (int i = 0; i < 4; ++i) shape_vec[i] = out_shape[i];
  Size<4> shape(shape_vec);
  utils::GPU gpu(stream);
  Ref1D<uint8_t> ws(reinterpret_cast<uint8_t*>(workspace), {(ssize_t)ws_bytes});
  if (subm) {
    spconv::func::createSparseSubMIndex<3, int32_t>(gpu, ws, gather, scatter, offset, num_index, in_coors, vec3(ksize),
                                                    vec3(stride), vec3(padding), vec3(dilation), shape);
  } else {
    Ref2D<int32_t> coors_out(out_coors, {max_num_act_out, 4});
    spconv::func::createSparseConvIndex<3, int32_t>(gpu, ws, gather, scatter, offset, coors_out, num_index,
                                                    num_act_out, in_coors, vec3(ksize), vec3(stride), vec3(padding),
                                                    vec3(dilation), shape, transpose != 0, max_num_act_out);
  }
  cudaError_t e = sync ? cudaStreamSynchronize(stream) : cudaSuccess;
  if (e == cudaSuccess) e = cudaGetLastError();
  return (int)e;
}

#ifdef REF_WITH_MM
namespace {
using MMOp1 = spconv::mm::TensorOp<cutlass::half_t, 64, 64, 16, 32, 32, 16, cutlass::arch::Sm75>;
using MMOp2 = spconv::mm::TensorOp<cutlass::half_t, 64, 64, 32, 16, 32, 32, cutlass::arch::Sm75>;
using MMOp3 = spconv::mm::Simt<cutlass::half_t, 32, 64, 8, 16, 32, 8, cutlass::arch::Sm80>;
}  // namespace

// fp16 features [n_in_rows, cin], filters [kvol, cin, cout], bias [cout] or null, index [3, row_len], out
// [max_num_act_out, cout]; the same configuration choice as mm_trt.cu:188-200.  Returns 0, -1 when no configuration
// accepts the shapes, or 1000 + the CUDA error code.
extern "C" int ref_spconv_mm_run(const void* in_feats, int64_t n_in_rows, int32_t cin, int32_t cout, int32_t kvol,
                                 const void* filters, const void* bias, const int32_t* index, int64_t row_len,
                                 int inverse, const int32_t* num_index, void* out_feats, int64_t max_num_act_out,
                                 int sync, cudaStream_t stream) {
  using dtype = cutlass::half_t;
  const int32_t* g = index;
  const int32_t* s = index + row_len;
  if (inverse) g = s, s = index;
  Ref1D<const int32_t> gather(g, {row_len}), scatter(s, {row_len}), offset(index + 2 * row_len, {row_len});
  Ref2D<dtype> out(reinterpret_cast<dtype*>(out_feats), {max_num_act_out, cout});
  Ref2D<const dtype> in(reinterpret_cast<const dtype*>(in_feats), {n_in_rows, cin});
  Ref3D<const dtype> w(reinterpret_cast<const dtype*>(filters), {kvol, cin, cout});
  Ref1D<const dtype> b(reinterpret_cast<const dtype*>(bias), {cout});
  utils::GPU gpu(stream);
  bool done;
  if (cin <= 16)
    done = spconv::func::indexedSpConv<MMOp1>(gpu, out, in, w, b, gather, scatter, offset, num_index);
  else
    done = spconv::func::indexedSpConv<MMOp2>(gpu, out, in, w, b, gather, scatter, offset, num_index);
  if (!done) done = spconv::func::indexedSpConv<MMOp3>(gpu, out, in, w, b, gather, scatter, offset, num_index);
  if (!done) return -1;
  cudaError_t e = sync ? cudaStreamSynchronize(stream) : cudaSuccess;
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}
#endif
