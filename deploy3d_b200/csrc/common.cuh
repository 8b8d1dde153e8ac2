// Shared helpers for the sm_100a kernels: status handling, launch geometry, warp primitives and
// the 64-bit-slot open-addressing hash table used by the rulebook generator and the voxel encoders.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>
#include <stdint.h>
#include <stdlib.h>

#include "../../include/deploy3d_b200.h"

namespace d3d {

// NVTX range around every C-ABI enqueue, off unless the process was started with D3D_NVTX=1 (the reference has a
// per-layer profiler on the TensorRT side only, deploy3d/symfun/trt_utils/trt_module.py:20-44).
inline bool nvtx_enabled() {
  static const bool on = [] {
    const char* v = getenv("D3D_NVTX");
    return v && v[0] == '1';
  }();
  return on;
}
struct NvtxRange {
  bool on;
  explicit NvtxRange(const char* name) : on(nvtx_enabled()) {
    if (on) nvtxRangePushA(name);
  }
  ~NvtxRange() {
    if (on) nvtxRangePop();
  }
};
#define D3D_NVTX_RANGE(name) ::d3d::NvtxRange d3d_nvtx_range_(name)

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs; grids of streaming kernels are sized in multiples of it

#define D3D_CHECK_LAUNCH()                                  \
  do {                                                      \
    if (cudaGetLastError() != cudaSuccess) return D3D_ERR_CUDA; \
  } while (0)

#define D3D_REQUIRE(cond, code) \
  do {                          \
    if (!(cond)) return (code); \
  } while (0)

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
static inline size_t next_pow2(size_t x) {
  size_t y = 1;
  while (y < x) y <<= 1;
  return y;
}
// Grid for a grid-stride kernel: enough CTAs to cover `work_items`, capped at `waves` full waves of the GPU.
static inline int stream_grid(int64_t work_items, int threads, int ctas_per_sm = 8) {
  int64_t need = ceil_div(work_items > 0 ? work_items : 1, threads);
  int64_t cap = (int64_t)kNumSMs * ctas_per_sm;
  return (int)(need < cap ? need : cap);
}

static inline size_t dtype_size(int dtype) {
  switch (dtype) {
    case D3D_FLOAT: return 4;
    case D3D_HALF: return 2;
    case D3D_BF16: return 2;
    case D3D_INT32: return 4;
    case D3D_INT8: return 1;
    case D3D_BOOL: return 1;
    default: return 0;
  }
}

// Bump allocator over the caller-provided workspace (256-byte granularity).
struct Carver {
  uint8_t* base;
  size_t off;
  explicit Carver(void* p) : base(reinterpret_cast<uint8_t*>(p)), off(0) {}
  template <class T> T* take(size_t count) {
    T* r = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off += align_up(count * sizeof(T), 256);
    return r;
  }
};

// ---------------------------------------------------------------------------------------------
// Device side
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }
__device__ __forceinline__ unsigned lanemask_lt() {
  unsigned m;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}

// Inclusive scan of `v` over the CTA (blockDim.x multiple of 32, <= 1024). `warp_sums` : >= 32 ints of smem.
// Returns the exclusive prefix of this thread; *total receives the CTA sum.
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_sums, int* total) {
  int lane = lane_id(), warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  int inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += t;
  }
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = lane < nwarp ? warp_sums[lane] : 0;
    int winc = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, winc, d);
      if (lane >= d) winc += t;
    }
    warp_sums[lane] = winc - w;  // exclusive warp offsets
    if (lane == 31) warp_sums[32] = winc;
  }
  __syncthreads();
  int excl = warp_sums[warp] + inc - v;
  *total = warp_sums[32];
  __syncthreads();
  return excl;
}

// ---------------------------------------------------------------------------------------------
// Open-addressing hash table on packed voxel keys.
//   slot word  = (key << 32) | value, EMPTY = all ones; one 64-bit CAS claims key and value together,
//                a 64-bit atomicMin on an owned slot keeps the smallest value (first touch).
//   key        = mixed-radix packing of (b, d0, d1, ..) into 31 bits (the linear offset the reference
//                uses as key, trt/include/common/refnd.h:48-54).
//   hash       = Murmur3 finaliser of (key >> 2) selects a 32-byte bucket of four slots, key & 3 selects the
//                slot inside it; probing advances by whole buckets.  Keys that differ only in the two low bits
//                (neighbours along the fastest axis) therefore share one 32-byte sector, so the three probes
//                a thread issues along x usually cost a single L2 sector instead of three.
//   capacity   = power of two chosen on the device from the live input count, >= 2 x the keys inserted.
// Probe loops are bounded by the capacity and report failure instead of spinning.
// ---------------------------------------------------------------------------------------------
constexpr unsigned long long kEmptySlot = ~0ull;

__device__ __forceinline__ uint32_t murmur_mix(uint32_t k) {
  k ^= k >> 16;
  k *= 0x85ebca6bu;
  k ^= k >> 13;
  k *= 0xc2b2ae35u;
  k ^= k >> 16;
  return k;
}

__device__ __forceinline__ uint32_t home_slot(uint32_t key, uint32_t cap_mask) {
  return ((murmur_mix(key >> 2) << 2) | (key & 3u)) & cap_mask;
}

// Insert (key -> min(value)). Returns the slot, or 0xFFFFFFFF when the table is full.
__device__ __forceinline__ uint32_t hash_insert_min(unsigned long long* table, uint32_t cap_mask, uint32_t key,
                                                    uint32_t value) {
  const unsigned long long mine = ((unsigned long long)key << 32) | value;
  uint32_t slot = home_slot(key, cap_mask);
  for (uint32_t probes = 0; probes <= (cap_mask >> 2); ++probes) {
    unsigned long long cur = table[slot];
    if (cur == kEmptySlot) {
      cur = atomicCAS(&table[slot], kEmptySlot, mine);
      if (cur == kEmptySlot) return slot;
    }
    if ((uint32_t)(cur >> 32) == key) {
      if ((uint32_t)cur > value) atomicMin(&table[slot], mine);
      return slot;
    }
    slot = (slot + 4u) & cap_mask;
  }
  return 0xFFFFFFFFu;
}

// The same insertion for key sets with few repeats (one voxel per key, or nearly): the slot is claimed without looking
// first, so the common case -- an empty home slot -- costs one round trip to the table instead of two.
__device__ __forceinline__ uint32_t hash_insert_min_claim_first(unsigned long long* table, uint32_t cap_mask,
                                                                uint32_t key, uint32_t value) {
  const unsigned long long mine = ((unsigned long long)key << 32) | value;
  uint32_t slot = home_slot(key, cap_mask);
  for (uint32_t probes = 0; probes <= (cap_mask >> 2); ++probes) {
    const unsigned long long cur = atomicCAS(&table[slot], kEmptySlot, mine);
    if (cur == kEmptySlot) return slot;
    if ((uint32_t)(cur >> 32) == key) {
      if ((uint32_t)cur > value) atomicMin(&table[slot], mine);
      return slot;
    }
    slot = (slot + 4u) & cap_mask;
  }
  return 0xFFFFFFFFu;
}

// Lookup; returns the value or -1.
__device__ __forceinline__ int32_t hash_lookup(const unsigned long long* __restrict__ table, uint32_t cap_mask,
                                               uint32_t key) {
  uint32_t slot = home_slot(key, cap_mask);
  for (uint32_t probes = 0; probes <= (cap_mask >> 2); ++probes) {
    unsigned long long cur = __ldg(&table[slot]);
    if ((uint32_t)(cur >> 32) == key) return (int32_t)(uint32_t)cur;
    if (cur == kEmptySlot) return -1;
    slot = (slot + 4u) & cap_mask;
  }
  return -1;
}

// Lookup split in two so that a thread can have the first probes of several keys in flight at once: the caller
// loads `first = table[home_slot(key)]` for all its keys, then resolves each; only a collision walks on.
__device__ __forceinline__ int32_t hash_lookup_resolve(const unsigned long long* __restrict__ table, uint32_t cap_mask,
                                                       uint32_t key, unsigned long long first) {
  if ((uint32_t)(first >> 32) == key) return (int32_t)(uint32_t)first;
  if (first == kEmptySlot) return -1;
  uint32_t slot = (home_slot(key, cap_mask) + 4u) & cap_mask;
  for (uint32_t probes = 1; probes <= (cap_mask >> 2); ++probes) {
    unsigned long long cur = __ldg(&table[slot]);
    if ((uint32_t)(cur >> 32) == key) return (int32_t)(uint32_t)cur;
    if (cur == kEmptySlot) return -1;
    slot = (slot + 4u) & cap_mask;
  }
  return -1;
}

// Capacity (slots, power of two >= 16) for `keys` insertions at load factor <= 0.5, clamped to `cap_max`.
__device__ __forceinline__ uint32_t hash_capacity(long long keys, uint32_t cap_max) {
  unsigned long long want = (unsigned long long)(keys > 8 ? keys : 8) * 2ull;
  uint32_t cap = 16;
  while (cap < want && cap < cap_max) cap <<= 1;
  return cap;
}

// Checked build (-DDEPLOY3D_BOUNDS_CHECK, python -m deploy3d_b200.build --checked): every row id, table entry or
// coordinate a kernel is about to index with is range-checked first; the first violation is recorded (site, value,
// limit), every one counted, and the access skipped.  One record for the whole library, so the checked build is
// compiled as relocatable device code.  In the regular build the macro is the constant `true`: the kernels keep only
// the range checks they need for safety and drop out-of-range entries silently, as the reference does.
enum BoundsSite {
  kSiteMmTcId = 1,      // SPConvMM tensor-core kernel: neighbour id outside [-1, rows of the input tensor)
  kSiteMmSimtId = 2,    // SPConvMM SIMT kernel: the same
  kSiteTableEntry = 3,  // neighbour table build: rulebook entry with a negative gather or an out-of-range scatter index
  kSiteBevCoord = 4,    // BEVDensify: voxel coordinate outside the dense grid
  kSiteScatterTo = 5,   // ScatterTo: voxel id >= number of voxels
  kSiteGatherBack = 6,  // GatherBack: voxel id >= number of voxels
  kSiteMirror = 7,      // neighbour table build with the mirror hint: a centre-offset entry that does not map a row to
                        // itself (duplicate input coordinates: the rulebook is not mirror-symmetric)
};
#ifdef DEPLOY3D_BOUNDS_CHECK
extern __device__ int g_d3d_bounds[4];  // violations seen; site, value and limit of the first
__device__ __forceinline__ bool bounds_ok(long long v, long long lo, long long hi, int site) {
  if (v >= lo && v < hi) return true;
  if (atomicAdd(&g_d3d_bounds[0], 1) == 0) g_d3d_bounds[1] = site, g_d3d_bounds[2] = (int)v, g_d3d_bounds[3] = (int)hi;
  return false;
}
#define D3D_BOUNDS_OK(v, lo, hi, site) ::d3d::bounds_ok((long long)(v), (long long)(lo), (long long)(hi), site)
#else
#define D3D_BOUNDS_OK(v, lo, hi, site) true
#endif

// Soft failures a kernel reports in the caller's optional status word (atomicOr; the word is the caller's to
// clear): they drop work instead of faulting, exactly where the reference is silent
// (trt/include/common/hash32.h:70, trt/spconv/index.cu:163-168).
__device__ __forceinline__ void report_status(int32_t* status, int bit) {
  if (status) atomicOr(status, bit);
}

// Single CTA: in-place exclusive scan of `totals[0..n)`; *clamped_total = min(sum, limit).  A sum above the limit
// (more voxels than the output buffers hold: the surplus is dropped) sets D3D_STATUS_OUTPUT_OVERFLOW.
static __global__ void scan_totals_kernel(int32_t* totals, int n, int32_t limit, int32_t* clamped_total,
                                          int32_t* status = nullptr) {
  __shared__ int scratch[40];
  int carry = 0;
  for (int base = 0; base < n; base += blockDim.x) {
    int j = base + threadIdx.x;
    int v = j < n ? totals[j] : 0;
    int total;
    int ex = block_exclusive_scan(v, scratch, &total);
    if (j < n) totals[j] = carry + ex;
    carry += total;
  }
  if (threadIdx.x == 0) {
    *clamped_total = carry < limit ? carry : limit;
    if (carry > limit) report_status(status, D3D_STATUS_OUTPUT_OVERFLOW);
  }
}

}  // namespace d3d
