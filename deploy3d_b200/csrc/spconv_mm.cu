// SPConvMM: sparse convolution feature computation over a rulebook.
//
// Replaces spconv::SPConvMMPlugin / spconv::func::indexedSpConv of the reference
// (trt/spconv/mm_trt.cu:39-206, trt/spconv/mm.h:35-71).  The reference walks the rulebook pair by pair
// (input-stationary) and scatters with fp16 atomics after a separate bias-initialisation pass.  Here the
// rulebook is first inverted into an output-stationary neighbour table  nbr[k][o] = input row feeding output o
// through offset k (or -1); every output row is then produced exactly once: fp32 accumulation over all offsets,
// bias (+ optional residual and ReLU) in the epilogue, one coalesced store.  Results are deterministic.
//
// This file holds the host side (blob parsing, weight upload, C ABI) and the SIMT kernel that serves fp32 and
// channel counts the tensor-core kernel cannot take; spconv_mm_tc.cu holds the tcgen05/TMEM kernel.
#include <string.h>

#include <cub/device/device_radix_sort.cuh>
#include <new>

#include "common.cuh"
#include "spconv_mm_internal.h"

namespace d3d {
namespace {

// ---------------------------------------------------------------------------------------------
// Neighbour table
// ---------------------------------------------------------------------------------------------
// Clears the row masks (four 32-bit words per (tile, offset): bit r of word q says that row 32 q + r of the tile has
// an input under that offset) and writes the identity output map (tile row p holds output p; a table whose outputs
// were regrouped holds a permutation instead).  The ids themselves need no initialisation: an id is only ever read
// where its row-mask bit is set.  The scatter kernel sets ids and bits; the per-tile offset masks are derived from
// the row masks afterwards.
__global__ void table_fill_kernel(uint32_t* row_masks, int64_t mask_words, int32_t* perm, int64_t perm_words,
                                  int64_t m_max) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t w = tid; w < perm_words; w += nthreads) perm[w] = w < m_max ? (int32_t)w : -1;
  for (int64_t w = tid; w < mask_words; w += nthreads) row_masks[w] = 0u;
}

// One warp per tile: lane k looks at the four row-mask words of offset k.
__global__ void pack_mask_kernel(const uint4* __restrict__ row_masks, int64_t tiles, int kvol,
                                 uint32_t* __restrict__ tile_mask) {
  const int64_t tile = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (tile >= tiles) return;
  const int k = threadIdx.x & 31;
  uint4 w = make_uint4(0u, 0u, 0u, 0u);
  if (k < kvol) w = __ldg(row_masks + tile * kvol + k);
  const unsigned m = __ballot_sync(0xffffffffu, (w.x | w.y | w.z | w.w) != 0u);
  if (k == 0) tile_mask[tile] = m;
}

// index rows: gatherIn | scatterOut | kernelOffset (trt/spconv/index_trt.cu:211-213); `inverse` swaps the
// first two (trt/spconv/mm_trt.cu:174-177).
// Besides the ids, every (tile of 128 outputs, offset) gets a 128-bit mask of the rows that have an input: the
// convolution kernel copies only those rows and lets the tensor core update only those accumulator lanes.
__global__ void table_scatter_kernel(const int32_t* __restrict__ index, int64_t row_len,
                                     const int32_t* __restrict__ num_index, int inverse, int mirror, int kvol,
                                     int64_t m_max, int32_t* __restrict__ table, uint32_t* __restrict__ row_masks) {
  int64_t n = *num_index;
  n = n > row_len ? row_len : n;
  // grid-stride over the live part of the rulebook only (the rows are sized for the worst case, mostly unused)
  const int64_t n_warp = (n + 31) & ~(int64_t)31;
  constexpr int kUnroll = 4;  // entries in flight per thread
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int32_t* gather_row = index + (inverse ? row_len : 0);
  const int32_t* scatter_row = index + (inverse ? 0 : row_len);
  for (int64_t p0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p0 < n_warp; p0 += kUnroll * stride) {
    int k[kUnroll], g[kUnroll], s[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t p = p0 + u * stride;
      const bool in = p < n;
      k[u] = in ? __ldg(index + 2 * row_len + p) : -1;
      g[u] = in ? __ldg(gather_row + p) : -1;
      s[u] = in ? __ldg(scatter_row + p) : -1;
      // A mirror-symmetric SubM rulebook holds (g, s) under offset k exactly when it holds (s, g) under
      // kvol - 1 - k.  Reading every entry as its mirror image makes the table writes follow the ascending gather
      // index of the segment: neighbouring lanes then hit the same few table rows instead of scattered ones.
      if (mirror && k[u] >= 0 && k[u] < kvol) {
        // checked build: the hint holds only if every row is its own centre neighbour
        if (k[u] * 2 + 1 == kvol) (void)D3D_BOUNDS_OK(g[u], s[u], (long long)s[u] + 1, kSiteMirror);
        const int t = g[u];
        g[u] = s[u], s[u] = t, k[u] = kvol - 1 - k[u];
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (p0 + u * stride >= n_warp) break;  // warp-uniform
      // k outside [0, kvol) marks a padding entry
      const bool live = k[u] >= 0 && k[u] < kvol;
      const bool valid = live && g[u] >= 0 && s[u] >= 0 && s[u] < m_max;
      if (live) (void)(D3D_BOUNDS_OK(g[u], 0, 0x7fffffffll, kSiteTableEntry) &&
                       D3D_BOUNDS_OK(s[u], 0, m_max, kSiteTableEntry));  // checked build: recorded
      // tile-major layout [tile of 128 outputs][k][128]: all offsets of a tile are one contiguous block
      if (valid) table[((int64_t)(s[u] >> 7) * kvol + k[u]) * 128 + (s[u] & 127)] = g[u];
      // one result-less atomic per entry (collecting the bits of a warp per mask word first -- match.any + redux.or
      // -- measured slower in the frame: 479 against 486 frames/s)
      if (valid)
        atomicOr(row_masks + ((unsigned long long)(s[u] >> 7) * kvol + k[u]) * 4ull + (unsigned)((s[u] & 127) >> 5),
                 1u << (s[u] & 31));
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Regrouping: tiles of outputs with like offset masks
// ---------------------------------------------------------------------------------------------
// A (tile, offset) block costs the convolution kernel a stage slot, a weight block and its MMAs whether one row or
// all 128 have an input, and with the outputs in voxel order nearly every offset feeds some row of every tile.  Sorted
// by their own offset mask (which of the kVol offsets have an input), outputs with like masks share a tile and the
// tile's mask shrinks to little more than theirs: LiDAR frames go from 27 to 4-19 blocks per tile.  The regrouped
// table lists for every tile row the output it stands for (`perm`); the convolution writes each row where it belongs,
// so nothing outside the table changes, and each output still accumulates its offsets in ascending order: the
// results are bit-identical to those of the plain table.

// One thread per output: its offset mask (bit k: offset k has an input) as sort key, its index as value.
__global__ void regroup_keys_kernel(const uint32_t* __restrict__ row_masks, int kvol, int64_t m_max,
                                    uint32_t* __restrict__ keys, int32_t* __restrict__ vals) {
  const int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= m_max) return;
  const uint32_t* w = row_masks + (o >> 7) * kvol * 4 + ((o & 127) >> 5);
  const int r = (int)(o & 31);
  uint32_t key = 0;
  for (int k = 0; k < kvol; ++k) key |= ((__ldg(w + k * 4) >> r) & 1u) << k;
  keys[o] = key;
  vals[o] = (int32_t)o;
}

// One CTA of 128 threads per tile of the regrouped table: thread r fetches the ids of its output from the plain table
// (only where the output has an input), and the ballots of the four warps are the row masks.
__global__ void __launch_bounds__(128)
regroup_gather_kernel(const int32_t* __restrict__ ids_in, const uint32_t* __restrict__ keys, const int32_t* __restrict__ vals,
                      int kvol, int64_t m_max, int32_t* __restrict__ ids_out, uint32_t* __restrict__ row_masks,
                      uint32_t* __restrict__ tile_mask, int32_t* __restrict__ perm) {
  __shared__ unsigned tile_bits;
  const int64_t tile = blockIdx.x, p = tile * 128 + threadIdx.x;
  if (threadIdx.x == 0) tile_bits = 0u;
  __syncthreads();
  const bool live = p < m_max;
  const int32_t o = live ? __ldg(vals + p) : -1;
  const uint32_t key = live ? __ldg(keys + p) : 0u;
  perm[p] = o;
  const int32_t* src = ids_in + ((int64_t)(o >> 7) * kvol) * 128 + (o & 127);
  int32_t* dst = ids_out + (tile * kvol) * 128 + threadIdx.x;
  uint32_t* rows = row_masks + (tile * kvol) * 4 + (threadIdx.x >> 5);
  unsigned mine = 0u;
#pragma unroll 3
  for (int k = 0; k < kvol; ++k) {
    const bool has = (key >> k) & 1u;
    if (has) dst[k * 128] = __ldg(src + k * 128);
    const unsigned ballot = __ballot_sync(0xffffffffu, has);
    if ((threadIdx.x & 31) == 0) {
      rows[k * 4] = ballot;
      if (ballot) mine |= 1u << k;
    }
  }
  if ((threadIdx.x & 31) == 0 && mine) atomicOr(&tile_bits, mine);
  __syncthreads();
  if (threadIdx.x == 0) tile_mask[tile] = tile_bits;
}

struct RegroupScratch {
  uint32_t *keys, *keys_sorted;
  int32_t *vals, *vals_sorted;
  void* temp;
  size_t temp_bytes, total;
};
RegroupScratch regroup_scratch(void* scratch, int kernel_vol, int64_t m_max) {
  RegroupScratch r;
  const size_t arr = align_up((size_t)(m_max > 0 ? m_max : 1) * 4, 256);
  unsigned char* b = reinterpret_cast<unsigned char*>(scratch);
  r.keys = reinterpret_cast<uint32_t*>(b), r.keys_sorted = reinterpret_cast<uint32_t*>(b + arr);
  r.vals = reinterpret_cast<int32_t*>(b + 2 * arr), r.vals_sorted = reinterpret_cast<int32_t*>(b + 3 * arr);
  r.temp = b + 4 * arr;
  r.temp_bytes = 0;
  // size query: host only, no launch
  cub::DeviceRadixSort::SortPairs(nullptr, r.temp_bytes, (const uint32_t*)nullptr, (uint32_t*)nullptr,
                                  (const int32_t*)nullptr, (int32_t*)nullptr, (int)m_max, 0, kernel_vol);
  r.total = 4 * arr + align_up(r.temp_bytes, 256);
  return r;
}

// ---------------------------------------------------------------------------------------------
// SIMT kernel: tile of 32 outputs per CTA, 256 threads, thread = (row, 8-strided column group).
// ---------------------------------------------------------------------------------------------
constexpr int kTileM = 32;
constexpr int kChunkK = 32;
constexpr int kSimtThreads = 256;

template <class T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <class T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <class T, int CPT>
__global__ void __launch_bounds__(kSimtThreads)
spconv_mm_simt_kernel(const T* __restrict__ in_feats, int64_t n_in_max, const T* __restrict__ weight,
                      const float* __restrict__ bias, const int32_t* __restrict__ table,
                      const uint32_t* __restrict__ row_masks, const int32_t* __restrict__ perm, int64_t m_max,
                      int kvol, int cin, int cout, T* __restrict__ out_feats, int relu, const T* __restrict__ residual) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* a_s = reinterpret_cast<float*>(smem_raw);                   // [kTileM][kChunkK + 1]
  float* w_s = a_s + kTileM * (kChunkK + 1);                         // [kChunkK][cout]
  int32_t* idx_s = reinterpret_cast<int32_t*>(w_s + kChunkK * cout); // [kvol][kTileM]
  int32_t* kvalid_s = idx_s + kvol * kTileM;                         // [kvol]

  // the CTA's 32 tile rows are one quarter of a 128-row tile of the table: one row-mask word per offset
  const int64_t tile0 = (int64_t)blockIdx.x * kTileM;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = tid >> 3, cg = tid & 7;
  const int64_t blk0 = (tile0 >> 7) * kvol;
  const int quarter = (int)((tile0 & 127) >> 5);

  for (int k = warp; k < kvol; k += kSimtThreads / 32) {
    const unsigned rows = __ldg(row_masks + (blk0 + k) * 4 + quarter);
    int v = ((rows >> lane) & 1u) ? __ldg(table + (blk0 + k) * 128 + quarter * 32 + lane) : -1;
    if (!D3D_BOUNDS_OK(v, -1, n_in_max, kSiteMmSimtId) || v >= n_in_max) v = -1;
    idx_s[k * kTileM + lane] = v;
    unsigned any = __ballot_sync(0xffffffffu, v >= 0);
    if (lane == 0) kvalid_s[k] = any != 0;
  }
  __syncthreads();

  float acc[CPT];
#pragma unroll
  for (int j = 0; j < CPT; ++j) acc[j] = 0.f;

  for (int k = 0; k < kvol; ++k) {
    if (!kvalid_s[k]) continue;
    const T* wk = weight + (int64_t)k * cin * cout;
    for (int c0 = 0; c0 < cin; c0 += kChunkK) {
      int kc = cin - c0 < kChunkK ? cin - c0 : kChunkK;
      __syncthreads();
      for (int e = tid; e < kTileM * kChunkK; e += kSimtThreads) {
        int rr = e / kChunkK, cc = e % kChunkK;
        int src = idx_s[k * kTileM + rr];
        float v = 0.f;
        if (src >= 0 && cc < kc) v = to_f32(in_feats[(int64_t)src * cin + c0 + cc]);
        a_s[rr * (kChunkK + 1) + cc] = v;
      }
      for (int e = tid; e < kc * cout; e += kSimtThreads) w_s[e] = to_f32(wk[(int64_t)c0 * cout + e]);
      __syncthreads();
      for (int cc = 0; cc < kc; ++cc) {
        float a = a_s[r * (kChunkK + 1) + cc];
#pragma unroll
        for (int j = 0; j < CPT; ++j) {
          int col = cg + 8 * j;
          if (col < cout) acc[j] = fmaf(a, w_s[cc * cout + col], acc[j]);
        }
      }
    }
  }

  const int64_t o = __ldg(perm + tile0 + r);  // the output this tile row stands for, -1 = none
  if (o >= 0 && o < m_max) {
#pragma unroll
    for (int j = 0; j < CPT; ++j) {
      int col = cg + 8 * j;
      if (col < cout) {
        float v = acc[j] + bias[col];
        if (relu == 2) v = fmaxf(v, 0.f);
        if (residual) v += to_f32(residual[o * cout + col]);
        if (relu == 1) v = fmaxf(v, 0.f);
        out_feats[o * cout + col] = from_f32<T>(v);
      }
    }
  }
}

template <class T> int launch_simt_typed(const MmLaunch& a) {
  const d3d_spconv_mm_s* h = a.h;
  int cout = h->p.out_channels, cin = h->p.in_channels, kvol = h->p.kernel_vol;
  int64_t m_max = h->p.max_num_act_out;
  if (m_max == 0) return D3D_OK;
  size_t smem = sizeof(float) * (kTileM * (kChunkK + 1) + (size_t)kChunkK * cout) +
                sizeof(int32_t) * ((size_t)kvol * kTileM + kvol);
  D3D_REQUIRE(smem <= 200 * 1024, D3D_ERR_TOO_LARGE);
  dim3 grid((unsigned)ceil_div(m_max, kTileM));
  const TableParts tp = table_parts(const_cast<int32_t*>(a.table), kvol, m_max);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(a.stream);
  int cpt = (cout + 7) / 8;
#define D3D_SIMT_CASE(N)                                                                                           \
  {                                                                                                                \
    auto kern = spconv_mm_simt_kernel<T, N>;                                                                       \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
    kern<<<grid, kSimtThreads, smem, st>>>(reinterpret_cast<const T*>(a.in_feats), a.max_num_act_in,               \
                                           reinterpret_cast<const T*>(h->w_dev), h->b_dev, tp.ids, tp.row_masks,    \
                                           tp.perm, m_max, kvol, cin, cout, reinterpret_cast<T*>(a.out_feats),      \
                                           a.relu, reinterpret_cast<const T*>(a.residual));                        \
  }
  if (cpt <= 2) D3D_SIMT_CASE(2)
  else if (cpt <= 4) D3D_SIMT_CASE(4)
  else if (cpt <= 8) D3D_SIMT_CASE(8)
  else if (cpt <= 16) D3D_SIMT_CASE(16)
  else if (cpt <= 32) D3D_SIMT_CASE(32)
  else return D3D_ERR_TOO_LARGE;
#undef D3D_SIMT_CASE
  D3D_CHECK_LAUNCH();
  return D3D_OK;
}

}  // namespace

int launch_spconv_mm_simt(const MmLaunch& a) {
  switch (a.dtype) {
    case D3D_FLOAT: return launch_simt_typed<float>(a);
    case D3D_HALF: return launch_simt_typed<__half>(a);
    case D3D_BF16: return launch_simt_typed<__nv_bfloat16>(a);
    default: return D3D_ERR_UNSUPPORTED_DTYPE;
  }
}

}  // namespace d3d

using namespace d3d;

// ---------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------
extern "C" int d3d_spconv_mm_create(const void* data_s, size_t len, d3d_spconv_mm_t* handle) {
  D3D_REQUIRE(data_s && handle, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(len >= 19, D3D_ERR_BAD_BLOB);
  const uint8_t* b = reinterpret_cast<const uint8_t*>(data_s);
  d3d_spconv_mm_params p;
  memcpy(&p.kernel_vol, b + 0, 4);
  memcpy(&p.in_channels, b + 4, 4);
  memcpy(&p.out_channels, b + 8, 4);
  memcpy(&p.max_num_act_out, b + 12, 4);
  p.subm = b[16] != 0;
  p.inverse = b[17] != 0;
  p.with_bias = b[18] != 0;
  D3D_REQUIRE(p.kernel_vol >= 1 && p.in_channels >= 1 && p.out_channels >= 1 && p.max_num_act_out >= 0,
              D3D_ERR_BAD_BLOB);
  size_t nw = (size_t)p.kernel_vol * p.in_channels * p.out_channels;
  size_t need = nw + (p.with_bias ? (size_t)p.out_channels : 0);
  D3D_REQUIRE((len - 19) / 4 >= need, D3D_ERR_BAD_BLOB);
  d3d_spconv_mm_s* h = new (std::nothrow) d3d_spconv_mm_s();
  D3D_REQUIRE(h, D3D_ERR_INVALID_ARGUMENT);
  h->p = p;
  h->wb.resize((len - 19) / 4);  // keeps trailing floats for a faithful serialize() (mm_trt.cu:61-74)
  memcpy(h->wb.data(), b + 19, h->wb.size() * 4);
  *handle = h;
  return D3D_OK;
}

extern "C" int d3d_spconv_mm_get_params(d3d_spconv_mm_t h, d3d_spconv_mm_params* p) {
  D3D_REQUIRE(h && p, D3D_ERR_INVALID_ARGUMENT);
  *p = h->p;
  return D3D_OK;
}

extern "C" int d3d_spconv_mm_serialize(d3d_spconv_mm_t h, void* buffer, size_t* len) {
  D3D_REQUIRE(h && len, D3D_ERR_INVALID_ARGUMENT);
  size_t need = 19 + h->wb.size() * 4;
  if (buffer) {
    D3D_REQUIRE(*len >= need, D3D_ERR_INVALID_ARGUMENT);
    uint8_t* b = reinterpret_cast<uint8_t*>(buffer);
    memcpy(b + 0, &h->p.kernel_vol, 4);
    memcpy(b + 4, &h->p.in_channels, 4);
    memcpy(b + 8, &h->p.out_channels, 4);
    memcpy(b + 12, &h->p.max_num_act_out, 4);
    b[16] = h->p.subm != 0, b[17] = h->p.inverse != 0, b[18] = h->p.with_bias != 0;
    memcpy(b + 19, h->wb.data(), h->wb.size() * 4);
  }
  *len = need;
  return D3D_OK;
}

static void release_device(d3d_spconv_mm_s* h) {
  spconv_mm_tc_release(h);
  if (h->w_dev) cudaFree(h->w_dev);
  if (h->wt_dev) cudaFree(h->wt_dev);
  if (h->b_dev) cudaFree(h->b_dev);
  h->w_dev = h->wt_dev = nullptr;
  h->b_dev = nullptr;
  h->dtype = -1;
}

template <class T, class Cvt> static int upload_weights(d3d_spconv_mm_s* h, Cvt cvt) {
  const int kvol = h->p.kernel_vol, cin = h->p.in_channels, cout = h->p.out_channels;
  size_t nw = (size_t)kvol * cin * cout;
  std::vector<T> w(nw), wt(nw);
  for (size_t i = 0; i < nw; ++i) w[i] = cvt(h->wb[i]);
  for (int k = 0; k < kvol; ++k)
    for (int ci = 0; ci < cin; ++ci)
      for (int co = 0; co < cout; ++co)
        wt[((size_t)k * cout + co) * cin + ci] = w[((size_t)k * cin + ci) * cout + co];
  if (cudaMalloc(&h->w_dev, nw * sizeof(T)) != cudaSuccess) return D3D_ERR_CUDA;
  if (cudaMalloc(&h->wt_dev, nw * sizeof(T)) != cudaSuccess) return D3D_ERR_CUDA;
  if (cudaMemcpy(h->w_dev, w.data(), nw * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess) return D3D_ERR_CUDA;
  if (cudaMemcpy(h->wt_dev, wt.data(), nw * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess) return D3D_ERR_CUDA;
  return D3D_OK;
}

extern "C" int d3d_spconv_mm_configure(d3d_spconv_mm_t h, int dtype) {
  D3D_REQUIRE(h, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(dtype == D3D_FLOAT || dtype == D3D_HALF || dtype == D3D_BF16, D3D_ERR_UNSUPPORTED_DTYPE);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return D3D_ERR_CUDA;
  if (h->dtype == dtype && h->device == dev) return D3D_OK;
  release_device(h);
  int rc;
  if (dtype == D3D_FLOAT) rc = upload_weights<float>(h, [](float v) { return v; });
  else if (dtype == D3D_HALF) rc = upload_weights<__half>(h, [](float v) { return __float2half_rn(v); });
  else rc = upload_weights<__nv_bfloat16>(h, [](float v) { return __float2bfloat16_rn(v); });
  if (rc != D3D_OK) {
    release_device(h);
    return rc;
  }
  // Bias is applied in fp32 after rounding it to the compute dtype, matching the half-precision upload of the
  // reference (mm_trt.cu:131-139).
  const int cout = h->p.out_channels;
  std::vector<float> bias(cout, 0.f);
  if (h->p.with_bias) {
    const float* src = h->wb.data() + (size_t)h->p.kernel_vol * h->p.in_channels * cout;
    for (int c = 0; c < cout; ++c) {
      float v = src[c];
      if (dtype == D3D_HALF) v = __half2float(__float2half_rn(v));
      if (dtype == D3D_BF16) v = __bfloat162float(__float2bfloat16_rn(v));
      bias[c] = v;
    }
  }
  if (cudaMalloc(&h->b_dev, cout * sizeof(float)) != cudaSuccess ||
      cudaMemcpy(h->b_dev, bias.data(), cout * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) {
    release_device(h);
    return D3D_ERR_CUDA;
  }
  rc = spconv_mm_tc_prepare(h, dtype);  // tensor map over the transposed weights (nothing for fp32 / odd channels)
  if (rc != D3D_OK) {
    release_device(h);
    return rc;
  }
  h->dtype = dtype;
  h->device = dev;
  return D3D_OK;
}

extern "C" int d3d_spconv_mm_destroy(d3d_spconv_mm_t h) {
  if (!h) return D3D_OK;
  release_device(h);
  delete h;
  return D3D_OK;
}

#ifdef DEPLOY3D_BOUNDS_CHECK
namespace d3d {
__device__ int g_d3d_bounds[4];
}
#endif
// Debug aid without a reference counterpart.  In a checked build (-DDEPLOY3D_BOUNDS_CHECK): synchronises the device,
// copies {violations seen, site / value / limit of the first} to `record` and clears them.  The regular build checks
// nothing and says so with D3D_ERR_INVALID_ARGUMENT.
extern "C" int d3d_debug_take_bounds_violation(int32_t* record) {
#ifdef DEPLOY3D_BOUNDS_CHECK
  if (!record) return D3D_ERR_INVALID_ARGUMENT;
  const int32_t zero[4] = {0, 0, 0, 0};
  if (cudaDeviceSynchronize() != cudaSuccess) return D3D_ERR_CUDA;
  if (cudaMemcpyFromSymbol(record, d3d::g_d3d_bounds, sizeof(zero)) != cudaSuccess) return D3D_ERR_CUDA;
  if (cudaMemcpyToSymbol(d3d::g_d3d_bounds, zero, sizeof(zero)) != cudaSuccess) return D3D_ERR_CUDA;
  return D3D_OK;
#else
  (void)record;
  return D3D_ERR_INVALID_ARGUMENT;
#endif
}

extern "C" int d3d_spconv_mm_set_dependent_launch(d3d_spconv_mm_t h, int enable) {
  D3D_REQUIRE(h, D3D_ERR_INVALID_ARGUMENT);
  h->dependent_launch = enable ? 1 : 0;
  return D3D_OK;
}

extern "C" int d3d_spconv_mm_set_kernel(d3d_spconv_mm_t h, int which) {
  D3D_REQUIRE(h && which >= 0 && which <= 3, D3D_ERR_INVALID_ARGUMENT);
  h->kernel_choice = which;
  return D3D_OK;
}

extern "C" size_t d3d_spconv_mm_table_bytes(int kernel_vol, int64_t max_num_act_out) {
  // rows are padded to a multiple of 128 entries so every 128-output tile can be read as a whole
  // followed by one 32-bit offset mask per tile, four 32-bit row masks per (tile, offset) and the output row of
  // every tile row
  return table_ids_bytes(kernel_vol, max_num_act_out) + table_mask_bytes(max_num_act_out) +
         table_rows_bytes(kernel_vol, max_num_act_out) + table_perm_bytes(max_num_act_out);
}

extern "C" int d3d_spconv_mm_workspace(d3d_spconv_mm_t h, const d3d_tensor_desc* in, int n_in, size_t* bytes) {
  D3D_REQUIRE(h && bytes, D3D_ERR_INVALID_ARGUMENT);
  (void)in, (void)n_in;
  *bytes = d3d_spconv_mm_table_bytes(h->p.kernel_vol, h->p.max_num_act_out);
  return D3D_OK;
}

extern "C" int d3d_spconv_mm_prepare(int kernel_vol, int mode, int64_t max_num_act_out, const int32_t* index,
                                     int64_t index_row_len, const int32_t* num_index, void* table, void* stream) {
  D3D_NVTX_RANGE("d3d_spconv_mm_prepare");
  D3D_REQUIRE(kernel_vol >= 1 && max_num_act_out >= 0 && index_row_len >= 0 && mode >= 0 && mode <= 3,
              D3D_ERR_INVALID_ARGUMENT);
  if (max_num_act_out == 0) return D3D_OK;
  D3D_REQUIRE(index && num_index && table, D3D_ERR_INVALID_ARGUMENT);
  const int inverse = mode & 1;
  const int mirror = (mode & 2) && !inverse;  // a symmetric rulebook is its own inverse
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t pitch = (max_num_act_out + 127) / 128 * 128;
  const TableParts t = table_parts(table, kernel_vol, max_num_act_out);
  table_fill_kernel<<<stream_grid(t.tiles * kernel_vol * 4, 256), 256, 0, st>>>(t.row_masks, t.tiles * kernel_vol * 4,
                                                                               t.perm, t.tiles * 128, max_num_act_out);
  if (index_row_len > 0)
    table_scatter_kernel<<<stream_grid(index_row_len, 256), 256, 0, st>>>(
        index, index_row_len, num_index, inverse, mirror, kernel_vol, pitch, t.ids, t.row_masks);
  pack_mask_kernel<<<(unsigned)ceil_div(t.tiles * 32, 256), 256, 0, st>>>(reinterpret_cast<const uint4*>(t.row_masks),
                                                                          t.tiles, kernel_vol, t.tile_mask);
  D3D_CHECK_LAUNCH();
  return D3D_OK;
}

// No plugin counterpart: see the header.
extern "C" size_t d3d_spconv_mm_regroup_scratch_bytes(int kernel_vol, int64_t max_num_act_out) {
  if (kernel_vol < 1 || kernel_vol > 32 || max_num_act_out < 0 || max_num_act_out >= (1ll << 31)) return 0;
  return regroup_scratch(nullptr, kernel_vol, max_num_act_out).total;
}

extern "C" int d3d_spconv_mm_regroup(int kernel_vol, int64_t max_num_act_out, const void* table_in, void* table_out,
                                     void* scratch, size_t scratch_bytes, void* stream) {
  D3D_NVTX_RANGE("d3d_spconv_mm_regroup");
  D3D_REQUIRE(kernel_vol >= 1 && kernel_vol <= 32 && max_num_act_out >= 0 && max_num_act_out < (1ll << 31),
              D3D_ERR_INVALID_ARGUMENT);
  if (max_num_act_out == 0) return D3D_OK;
  D3D_REQUIRE(table_in && table_out && scratch && table_in != table_out, D3D_ERR_INVALID_ARGUMENT);
  RegroupScratch r = regroup_scratch(scratch, kernel_vol, max_num_act_out);
  D3D_REQUIRE(scratch_bytes >= r.total, D3D_ERR_WORKSPACE_TOO_SMALL);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const TableParts in = table_parts(const_cast<void*>(table_in), kernel_vol, max_num_act_out);
  const TableParts out = table_parts(table_out, kernel_vol, max_num_act_out);
  regroup_keys_kernel<<<(unsigned)ceil_div(max_num_act_out, 256), 256, 0, st>>>(in.row_masks, kernel_vol,
                                                                                max_num_act_out, r.keys, r.vals);
  // stable, so outputs with equal masks keep their order: the table is the same every time
  if (cub::DeviceRadixSort::SortPairs(r.temp, r.temp_bytes, r.keys, r.keys_sorted, r.vals, r.vals_sorted,
                                      (int)max_num_act_out, 0, kernel_vol, st) != cudaSuccess)
    return D3D_ERR_CUDA;
  regroup_gather_kernel<<<(unsigned)out.tiles, 128, 0, st>>>(in.ids, r.keys_sorted, r.vals_sorted, kernel_vol,
                                                              max_num_act_out, out.ids, out.row_masks, out.tile_mask,
                                                              out.perm);
  D3D_CHECK_LAUNCH();
  return D3D_OK;
}

extern "C" int d3d_spconv_mm_run(d3d_spconv_mm_t h, int dtype, const void* in_feats, int64_t max_num_act_in,
                                 const int32_t* num_act_out, const void* table, void* out_feats,
                                 const d3d_spconv_mm_epilogue* epilogue, void* stream) {
  D3D_NVTX_RANGE("d3d_spconv_mm_run");
  D3D_REQUIRE(h, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(dtype == D3D_FLOAT || dtype == D3D_HALF || dtype == D3D_BF16, D3D_ERR_UNSUPPORTED_DTYPE);
  D3D_REQUIRE(h->dtype == dtype, D3D_ERR_INVALID_ARGUMENT);  // configure() must have run for this dtype
  if (h->p.max_num_act_out == 0) return D3D_OK;
  D3D_REQUIRE(in_feats && table && out_feats, D3D_ERR_INVALID_ARGUMENT);
  MmLaunch a;
  a.h = h, a.dtype = dtype, a.in_feats = in_feats, a.max_num_act_in = max_num_act_in, a.num_act_out = num_act_out;
  a.table = reinterpret_cast<const int32_t*>(table), a.out_feats = out_feats;
  a.relu = epilogue ? epilogue->relu : 0;
  a.residual = epilogue ? epilogue->residual : nullptr;
  a.regrouped = epilogue ? epilogue->regrouped : 0;
  a.stream = stream;
  bool tc_ok = spconv_mm_tc_eligible(h, dtype);
  if (h->kernel_choice == 2 || h->kernel_choice == 3) {
    D3D_REQUIRE(tc_ok, D3D_ERR_INVALID_ARGUMENT);
    return launch_spconv_mm_tc(a);
  }
  if (h->kernel_choice == 0 && tc_ok) return launch_spconv_mm_tc(a);
  return launch_spconv_mm_simt(a);
}

extern "C" int d3d_spconv_mm_enqueue(d3d_spconv_mm_t h, const d3d_tensor_desc* in, int n_in,
                                     const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                                     void* const* outputs, void* workspace, size_t workspace_bytes, void* stream) {
  D3D_NVTX_RANGE("d3d_spconv_mm_enqueue");
  D3D_REQUIRE(h && in && out && inputs && outputs && n_in >= 5 && n_out >= 1, D3D_ERR_INVALID_ARGUMENT);
  int dtype = in[0].dtype;
  D3D_REQUIRE(dtype == D3D_FLOAT || dtype == D3D_HALF || dtype == D3D_BF16, D3D_ERR_UNSUPPORTED_DTYPE);
  D3D_REQUIRE(out[0].dtype == dtype, D3D_ERR_UNSUPPORTED_DTYPE);
  D3D_REQUIRE(in[0].nb_dims == 2 && in[0].dims[1] == h->p.in_channels, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(in[3].nb_dims == 2 && in[3].dims[0] == 3, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(out[0].nb_dims == 2 && out[0].dims[0] == h->p.max_num_act_out && out[0].dims[1] == h->p.out_channels,
              D3D_ERR_INVALID_ARGUMENT);
  size_t need = d3d_spconv_mm_table_bytes(h->p.kernel_vol, h->p.max_num_act_out);
  D3D_REQUIRE(h->p.max_num_act_out == 0 || (workspace && workspace_bytes >= need), D3D_ERR_WORKSPACE_TOO_SMALL);
  // configurePlugin (d3d_spconv_mm_configure) uploads the weights; enqueue itself allocates nothing and copies
  // nothing from the host (the reference uploads in configurePlugin too, trt/spconv/mm_trt.cu:127-142)
  int dev = -1;
  D3D_REQUIRE(cudaGetDevice(&dev) == cudaSuccess, D3D_ERR_CUDA);
  D3D_REQUIRE(h->dtype == dtype && h->device == dev, D3D_ERR_INVALID_ARGUMENT);
  int rc = d3d_spconv_mm_prepare(h->p.kernel_vol, h->p.inverse, h->p.max_num_act_out,
                             reinterpret_cast<const int32_t*>(inputs[3]), in[3].dims[1],
                             reinterpret_cast<const int32_t*>(inputs[4]), workspace, stream);
  if (rc != D3D_OK) return rc;
  return d3d_spconv_mm_run(h, dtype, inputs[0], in[0].dims[0], reinterpret_cast<const int32_t*>(inputs[2]),
                           workspace, outputs[0], nullptr, stream);
}
