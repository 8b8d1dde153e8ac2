// BEVDensify: sparse voxel features -> dense [B, C*Z, Y, X] feature map.
//
// Replaces spconv::BEVDensifyPlugin (trt/spconv/bev_densify_trt.cu:23-35, :136-177).  The reference memsets the
// whole output and then lets one thread per voxel write C values with a stride of Z*Y*X elements.  Here every
// output element is written exactly once with stores that are contiguous along x: a dense voxel-id map
// [B, Z, Y, X] is built in the workspace, then each CTA produces a (b, z, y, 32-wide x) strip for all channels,
// staging the 32 x C feature tile through shared memory so that both the row gather and the channel-major
// stores are coalesced.  numActIn is read on the device (the reference blocks on a D2H copy, :152-155).
#include "common.cuh"

namespace d3d {
namespace {

__global__ void map_fill_kernel(int32_t* map, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    map[i] = -1;
}

__global__ void map_scatter_kernel(int32_t* __restrict__ map, const int32_t* __restrict__ coors,
                                   const int32_t* num_act_in, int64_t n_max, int b, int z, int y, int x) {
  int n = *num_act_in;
  n = n > n_max ? (int)n_max : n;
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int4 c = __ldg(reinterpret_cast<const int4*>(coors) + i);
  if (!(D3D_BOUNDS_OK(c.x, 0, b, kSiteBevCoord) && D3D_BOUNDS_OK(c.y, 0, z, kSiteBevCoord) &&
        D3D_BOUNDS_OK(c.z, 0, y, kSiteBevCoord) && D3D_BOUNDS_OK(c.w, 0, x, kSiteBevCoord)))
    return;
  if (c.x < 0 || c.x >= b || c.y < 0 || c.y >= z || c.z < 0 || c.z >= y || c.w < 0 || c.w >= x) return;
  map[(((int64_t)c.x * z + c.y) * y + c.z) * x + c.w] = i;
}

constexpr int kStrip = 32;

// grid: (ceil(X/32), Y, B*Z); block: 256 threads.
template <class T>
__global__ void densify_kernel(const int32_t* __restrict__ map, const T* __restrict__ feats, int c, int z, int y,
                               int x, T* __restrict__ out) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* tile = reinterpret_cast<T*>(smem_raw);  // [kStrip][c + pad]
  __shared__ int32_t vid[kStrip];
  const int pitch = c + (sizeof(T) == 2 ? 2 : 1);
  const int x0 = blockIdx.x * kStrip, yy = blockIdx.y, bz = blockIdx.z;
  const int b = bz / z, zz = bz % z;
  if (threadIdx.x < kStrip) {
    int xx = x0 + threadIdx.x;
    vid[threadIdx.x] = xx < x ? map[((int64_t)bz * y + yy) * x + xx] : -1;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < kStrip * c; e += blockDim.x) {
    int r = e / c, ch = e % c;
    int v = vid[r];
    tile[r * pitch + ch] = v >= 0 ? feats[(int64_t)v * c + ch] : T(0);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  int xx = x0 + lane;
  if (xx >= x) return;
  for (int ch = warp; ch < c; ch += nwarp)
    out[((((int64_t)b * c + ch) * z + zz) * y + yy) * x + xx] = tile[lane * pitch + ch];
}

// 16-bit features, c a multiple of 8, even x: a CTA takes 64 cells of a row; the feature rows come in as 16-byte
// loads, and every warp store covers 64 consecutive cells of one channel plane (128 bytes).
constexpr int kWideStrip = 64;
__global__ void __launch_bounds__(256)
densify_wide_kernel(const int32_t* __restrict__ map, const unsigned short* __restrict__ feats, int c, int z, int y,
                    int x, unsigned short* __restrict__ out) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint32_t* tile = reinterpret_cast<uint32_t*>(smem_raw);  // [kWideStrip][c / 2 + 1] words: odd pitch
  __shared__ int32_t vid[kWideStrip];
  const int pitch = c / 2 + 1;
  const int x0 = blockIdx.x * kWideStrip, yy = blockIdx.y, bz = blockIdx.z;
  const int b = bz / z, zz = bz % z;
  if (threadIdx.x < kWideStrip) {
    int xx = x0 + threadIdx.x;
    vid[threadIdx.x] = xx < x ? map[((int64_t)bz * y + yy) * x + xx] : -1;
  }
  __syncthreads();
  const int vec_per_row = c / 8;
  for (int e = threadIdx.x; e < kWideStrip * vec_per_row; e += blockDim.x) {
    const int r = e / vec_per_row, q = e - r * vec_per_row;
    const int v = vid[r];
    uint4 w = make_uint4(0u, 0u, 0u, 0u);
    if (v >= 0) w = __ldg(reinterpret_cast<const uint4*>(feats + (int64_t)v * c) + q);
    uint32_t* d = tile + r * pitch + q * 4;
    d[0] = w.x, d[1] = w.y, d[2] = w.z, d[3] = w.w;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int xx = x0 + 2 * lane;
  if (xx >= x) return;  // x is even: a pair of cells is inside or outside together
  const unsigned short* t16 = reinterpret_cast<const unsigned short*>(tile);
  for (int ch = warp; ch < c; ch += nwarp) {
    const uint32_t lo = t16[(2 * lane) * pitch * 2 + ch], hi = t16[(2 * lane + 1) * pitch * 2 + ch];
    *reinterpret_cast<uint32_t*>(out + ((((int64_t)b * c + ch) * z + zz) * y + yy) * x + xx) = lo | (hi << 16);
  }
}

}  // namespace
}  // namespace d3d

using namespace d3d;

extern "C" int d3d_bev_densify_parse(const void* data_s, size_t len, d3d_bev_densify_params* p) {
  D3D_REQUIRE(data_s && p, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(len >= 4, D3D_ERR_BAD_BLOB);
  memcpy(&p->out_channels, data_s, 4);
  return D3D_OK;
}

static int densify_map_elems(const d3d_tensor_desc* in, int n_in, int64_t* elems) {
  D3D_REQUIRE(in && n_in >= 4 && in[3].nb_dims == 5, D3D_ERR_INVALID_ARGUMENT);
  *elems = in[3].dims[0] * in[3].dims[2] * in[3].dims[3] * in[3].dims[4];
  return D3D_OK;
}

extern "C" int d3d_bev_densify_workspace(const d3d_bev_densify_params* p, const d3d_tensor_desc* in, int n_in,
                                         size_t* bytes) {
  D3D_REQUIRE(p && bytes, D3D_ERR_INVALID_ARGUMENT);
  int64_t elems;
  int rc = densify_map_elems(in, n_in, &elems);
  if (rc != D3D_OK) return rc;
  *bytes = align_up((size_t)elems * 4, 256);
  return D3D_OK;
}

extern "C" int d3d_bev_densify_enqueue(const d3d_bev_densify_params* p, const d3d_tensor_desc* in, int n_in,
                                       const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                                       void* const* outputs, void* workspace, size_t workspace_bytes, void* stream) {
  D3D_NVTX_RANGE("d3d_bev_densify_enqueue");
  D3D_REQUIRE(p && in && out && inputs && outputs && n_in >= 4 && n_out >= 1, D3D_ERR_INVALID_ARGUMENT);
  int64_t elems;
  int rc = densify_map_elems(in, n_in, &elems);
  if (rc != D3D_OK) return rc;
  int dtype = in[0].dtype;
  D3D_REQUIRE(dtype == D3D_FLOAT || dtype == D3D_HALF || dtype == D3D_BF16, D3D_ERR_UNSUPPORTED_DTYPE);
  D3D_REQUIRE(in[0].nb_dims == 2 && in[1].nb_dims == 2 && in[1].dims[1] == 4, D3D_ERR_INVALID_ARGUMENT);
  const int64_t n_max = in[0].dims[0];
  const int c = (int)in[0].dims[1];
  const int b = (int)in[3].dims[0], z = (int)in[3].dims[2], y = (int)in[3].dims[3], x = (int)in[3].dims[4];
  D3D_REQUIRE((int64_t)p->out_channels == (int64_t)c * z, D3D_ERR_INVALID_ARGUMENT);
  if (elems == 0 || c == 0) return D3D_OK;
  D3D_REQUIRE(workspace && workspace_bytes >= (size_t)elems * 4, D3D_ERR_WORKSPACE_TOO_SMALL);
  D3D_REQUIRE((int64_t)b * z <= 65535 && y <= 65535, D3D_ERR_TOO_LARGE);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int32_t* map = reinterpret_cast<int32_t*>(workspace);
  map_fill_kernel<<<stream_grid(elems, 256), 256, 0, st>>>(map, elems);
  if (n_max > 0)
    map_scatter_kernel<<<(unsigned)ceil_div(n_max, 256), 256, 0, st>>>(
        map, reinterpret_cast<const int32_t*>(inputs[1]), reinterpret_cast<const int32_t*>(inputs[2]), n_max, b, z, y,
        x);
  dim3 grid((unsigned)ceil_div(x, kStrip), (unsigned)y, (unsigned)(b * z));
  if (dtype == D3D_FLOAT) {
    size_t smem = (size_t)kStrip * (c + 1) * 4;
    D3D_REQUIRE(smem <= 48 * 1024, D3D_ERR_TOO_LARGE);
    densify_kernel<float><<<grid, 256, smem, st>>>(map, reinterpret_cast<const float*>(inputs[0]), c, z, y, x,
                                                   reinterpret_cast<float*>(outputs[0]));
  } else {
    // half and bf16 are both moved as 16-bit words
    const size_t wide_smem = (size_t)kWideStrip * (c / 2 + 1) * 4;
    if (c % 8 == 0 && x % 2 == 0 && wide_smem <= 48 * 1024 && reinterpret_cast<uintptr_t>(inputs[0]) % 16 == 0 &&
        reinterpret_cast<uintptr_t>(outputs[0]) % 4 == 0) {
      dim3 wide((unsigned)ceil_div(x, kWideStrip), (unsigned)y, (unsigned)(b * z));
      densify_wide_kernel<<<wide, 256, wide_smem, st>>>(map, reinterpret_cast<const unsigned short*>(inputs[0]), c, z,
                                                        y, x, reinterpret_cast<unsigned short*>(outputs[0]));
      D3D_CHECK_LAUNCH();
      return D3D_OK;
    }
    size_t smem = (size_t)kStrip * (c + 2) * 2;
    D3D_REQUIRE(smem <= 48 * 1024, D3D_ERR_TOO_LARGE);
    densify_kernel<unsigned short><<<grid, 256, smem, st>>>(map, reinterpret_cast<const unsigned short*>(inputs[0]),
                                                            c, z, y, x, reinterpret_cast<unsigned short*>(outputs[0]));
  }
  D3D_CHECK_LAUNCH();
  return D3D_OK;
}
