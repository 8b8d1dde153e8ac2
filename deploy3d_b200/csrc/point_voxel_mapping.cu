// ScatterTo (point -> voxel max / mean reduction) and GatherBack (voxel -> point gather).
//
// Replace point_voxel_mapping::func::scatterTo (trt/point_voxel_mapping/scatter_to.cu:83-103, kernels :45-79) and
// point_voxel_mapping::func::gatherBack (trt/point_voxel_mapping/gather_back.cu:51-62, kernel :28-47).
// Both run on the stream they are given.  Rows are moved with 16-byte accesses when the channel count allows it;
// the max reduction uses the order-preserving integer view of IEEE floats (one native atomic instead of a
// compare-and-swap loop), so it is deterministic; the mean reduction adds x / count with 16-byte vector atomics.
#include <float.h>

#include "common.cuh"

namespace d3d {
namespace {

__global__ void fill_kernel(float* out, int64_t n, float v) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = v;
}

// max over floats through integer atomics: non-negative values order like signed ints, negative values
// order inversely as unsigned ints.  The destination starts at -FLT_MAX.
__device__ __forceinline__ void atomic_max_float(float* addr, float v) {
  if (v >= 0.f) atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v + 0.f));  // -0.0 -> +0.0
  else atomicMin(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

// one thread per (point, 4-channel group)
template <bool kMean, bool kVec>
__global__ void scatter_reduce_kernel(const float* __restrict__ in_feats, const int32_t* __restrict__ scatter_to,
                                      const int32_t* __restrict__ scatter_count, int64_t n, int c, int64_t m,
                                      float* __restrict__ out) {
  const int groups = kVec ? c / 4 : c;
  int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n * groups) return;
  int64_t p = t / groups;
  int g = (int)(t % groups);
  int v = __ldg(scatter_to + p);
  if (v < 0 || !D3D_BOUNDS_OK(v, 0, m, kSiteScatterTo) || v >= m) return;
  if (kVec) {
    float4 x = __ldg(reinterpret_cast<const float4*>(in_feats + p * c) + g);
    float* o = out + (int64_t)v * c + 4 * g;
    if (kMean) {
      float cnt = (float)__ldg(scatter_count + v);
      x.x = __fdiv_rn(x.x, cnt), x.y = __fdiv_rn(x.y, cnt), x.z = __fdiv_rn(x.z, cnt), x.w = __fdiv_rn(x.w, cnt);
      atomicAdd(reinterpret_cast<float4*>(o), x);
    } else {
      atomic_max_float(o + 0, x.x), atomic_max_float(o + 1, x.y);
      atomic_max_float(o + 2, x.z), atomic_max_float(o + 3, x.w);
    }
  } else {
    float x = __ldg(in_feats + p * c + g);
    float* o = out + (int64_t)v * c + g;
    if (kMean) atomicAdd(o, __fdiv_rn(x, (float)__ldg(scatter_count + v)));
    else atomic_max_float(o, x);
  }
}

// one thread per (point, element group); rows with a negative index are written only when `fill` is set.
template <class V>
__global__ void gather_rows_kernel(const V* __restrict__ in, const int32_t* __restrict__ scatter_to, int64_t n,
                                   int64_t groups, int64_t m, int fill, V fill_val, V* __restrict__ out) {
  int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n * groups) return;
  int64_t p = t / groups, g = t % groups;
  int v = __ldg(scatter_to + p);
  if (v < 0 || !D3D_BOUNDS_OK(v, 0, m, kSiteGatherBack) || v >= m) {
    if (fill) out[t] = fill_val;
    return;
  }
  out[t] = __ldg(in + (int64_t)v * groups + g);
}

// The same for half-precision features (the output of a convolution) gathered into half or float rows.
template <class TIn, class TOut>
__global__ void gather_rows_convert_kernel(const TIn* __restrict__ in, const int32_t* __restrict__ scatter_to, int64_t n,
                                           int64_t c, int64_t m, int fill, float fill_val, TOut* __restrict__ out) {
  int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n * c) return;
  int64_t p = t / c, g = t % c;
  int v = __ldg(scatter_to + p);
  if (v < 0 || !D3D_BOUNDS_OK(v, 0, m, kSiteGatherBack) || v >= m) {
    if (fill) out[t] = static_cast<TOut>(fill_val);
    return;
  }
  out[t] = static_cast<TOut>(static_cast<float>(in[(int64_t)v * c + g]));
}

}  // namespace
}  // namespace d3d

using namespace d3d;

extern "C" int d3d_scatter_to_parse(const void* data_s, size_t len, d3d_scatter_to_params* p) {
  D3D_REQUIRE(data_s && p, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(len >= 1, D3D_ERR_BAD_BLOB);
  p->reduce_type = *reinterpret_cast<const int8_t*>(data_s);
  return D3D_OK;
}

extern "C" int d3d_scatter_to_enqueue(const d3d_scatter_to_params* p, const d3d_tensor_desc* in, int n_in,
                                      const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                                      void* const* outputs, void* workspace, size_t workspace_bytes, void* stream) {
  D3D_NVTX_RANGE("d3d_scatter_to_enqueue");
  (void)workspace, (void)workspace_bytes;
  D3D_REQUIRE(p && in && out && inputs && outputs && n_in >= 3 && n_out >= 1, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(in[0].dtype == D3D_FLOAT, D3D_ERR_UNSUPPORTED_DTYPE);
  D3D_REQUIRE(in[0].nb_dims == 2 && in[1].nb_dims == 1 && in[2].nb_dims == 1, D3D_ERR_INVALID_ARGUMENT);
  const int64_t n = in[0].dims[0], m = in[2].dims[0];
  const int c = (int)in[0].dims[1];
  D3D_REQUIRE(in[1].dims[0] == n && out[0].dims[0] == m && out[0].dims[1] == c, D3D_ERR_INVALID_ARGUMENT);
  if (m == 0 || c == 0) return D3D_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const float* feats = reinterpret_cast<const float*>(inputs[0]);
  const int32_t* idx = reinterpret_cast<const int32_t*>(inputs[1]);
  const int32_t* cnt = reinterpret_cast<const int32_t*>(inputs[2]);
  float* o = reinterpret_cast<float*>(outputs[0]);
  const bool mean = p->reduce_type != 0;
  // scatter_to.cu:92-94 initialises with numeric_limits<float>::lowest(), :98 with zero
  fill_kernel<<<stream_grid(m * c, 256), 256, 0, st>>>(o, m * c, mean ? 0.f : -FLT_MAX);
  if (n > 0) {
    const bool vec = (c % 4 == 0) && (reinterpret_cast<uintptr_t>(feats) % 16 == 0) &&
                     (reinterpret_cast<uintptr_t>(o) % 16 == 0);
    int64_t work = n * (vec ? c / 4 : c);
    unsigned grid = (unsigned)ceil_div(work, 256);
    if (mean && vec) scatter_reduce_kernel<true, true><<<grid, 256, 0, st>>>(feats, idx, cnt, n, c, m, o);
    else if (mean) scatter_reduce_kernel<true, false><<<grid, 256, 0, st>>>(feats, idx, cnt, n, c, m, o);
    else if (vec) scatter_reduce_kernel<false, true><<<grid, 256, 0, st>>>(feats, idx, cnt, n, c, m, o);
    else scatter_reduce_kernel<false, false><<<grid, 256, 0, st>>>(feats, idx, cnt, n, c, m, o);
  }
  D3D_CHECK_LAUNCH();
  return D3D_OK;
}

extern "C" int d3d_gather_back_parse(const void* data_s, size_t len, d3d_gather_back_params* p) {
  D3D_REQUIRE(data_s && p, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(len >= 5, D3D_ERR_BAD_BLOB);
  const uint8_t* b = reinterpret_cast<const uint8_t*>(data_s);
  p->fill = b[0] != 0;
  memcpy(&p->fill_val, b + 1, 4);
  return D3D_OK;
}

extern "C" int d3d_gather_back_enqueue(const d3d_gather_back_params* p, const d3d_tensor_desc* in, int n_in,
                                       const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                                       void* const* outputs, void* workspace, size_t workspace_bytes, void* stream) {
  D3D_NVTX_RANGE("d3d_gather_back_enqueue");
  (void)workspace, (void)workspace_bytes;
  D3D_REQUIRE(p && in && out && inputs && outputs && n_in >= 2 && n_out >= 1, D3D_ERR_INVALID_ARGUMENT);
  // the reference takes float features (gather_back.cu:146-150); half / bf16 features -- what a half-precision
  // network hands over -- are accepted as well and gathered into rows of the same type or widened to float
  const int tin = in[0].dtype, tout = out[0].dtype;
  D3D_REQUIRE(tin == D3D_FLOAT || tin == D3D_HALF || tin == D3D_BF16, D3D_ERR_UNSUPPORTED_DTYPE);
  D3D_REQUIRE(tout == tin || (tout == D3D_FLOAT && tin != D3D_FLOAT), D3D_ERR_UNSUPPORTED_DTYPE);
  D3D_REQUIRE(in[0].nb_dims >= 1 && in[1].nb_dims == 1, D3D_ERR_INVALID_ARGUMENT);
  const int64_t m = in[0].dims[0], n = in[1].dims[0];
  int64_t c = 1;
  for (int d = 1; d < in[0].nb_dims; ++d) c *= in[0].dims[d];  // gather_back.cu:36: row width = stride(0)
  if (n == 0 || c == 0) return D3D_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (tin != D3D_FLOAT) {
    const unsigned grid = (unsigned)ceil_div(n * c, 256);
    const int32_t* ids = reinterpret_cast<const int32_t*>(inputs[1]);
#define D3D_GATHER_CASE(TI, TO)                                                                             \
  gather_rows_convert_kernel<TI, TO><<<grid, 256, 0, st>>>(reinterpret_cast<const TI*>(inputs[0]), ids, n, c, m, \
                                                         p->fill, p->fill_val, reinterpret_cast<TO*>(outputs[0]))
    if (tin == D3D_HALF && tout == D3D_HALF) D3D_GATHER_CASE(__half, __half);
    else if (tin == D3D_HALF) D3D_GATHER_CASE(__half, float);
    else if (tout == D3D_BF16) D3D_GATHER_CASE(__nv_bfloat16, __nv_bfloat16);
    else D3D_GATHER_CASE(__nv_bfloat16, float);
#undef D3D_GATHER_CASE
    D3D_CHECK_LAUNCH();
    return D3D_OK;
  }
  const float* feats = reinterpret_cast<const float*>(inputs[0]);
  const int32_t* idx = reinterpret_cast<const int32_t*>(inputs[1]);
  float* o = reinterpret_cast<float*>(outputs[0]);
  const bool vec = (c % 4 == 0) && (reinterpret_cast<uintptr_t>(feats) % 16 == 0) &&
                   (reinterpret_cast<uintptr_t>(o) % 16 == 0);
  if (vec) {
    float4 fv = make_float4(p->fill_val, p->fill_val, p->fill_val, p->fill_val);
    gather_rows_kernel<float4><<<(unsigned)ceil_div(n * (c / 4), 256), 256, 0, st>>>(
        reinterpret_cast<const float4*>(feats), idx, n, c / 4, m, p->fill, fv, reinterpret_cast<float4*>(o));
  } else {
    gather_rows_kernel<float><<<(unsigned)ceil_div(n * c, 256), 256, 0, st>>>(feats, idx, n, c, m, p->fill,
                                                                               p->fill_val, o);
  }
  D3D_CHECK_LAUNCH();
  return D3D_OK;
}
