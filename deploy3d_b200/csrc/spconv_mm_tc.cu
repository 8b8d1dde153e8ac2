// SPConvMM on the 5th-generation tensor cores: output-stationary implicit GEMM.
//
// For a tile of 128 consecutive output voxels and every kernel offset k that feeds at least one of them:
//   A = the 128 input rows named by the neighbour table, gathered by TMA (tile::gather4, four arbitrary rows per
//       instruction, missing neighbours addressed out of bounds so the TMA zero-fills them without touching memory),
//   B = W[k]^T, K-major, loaded by a tiled TMA copy,
//   D += A * B with tcgen05.mma (M = 128, N = Cout, K = 16 per instruction), fp32 accumulator in tensor memory.
// All offsets of a tile accumulate into the same TMEM columns; the epilogue reads them once with tcgen05.ld, adds
// bias (+ residual), applies ReLU, converts and stores the row.  No atomics, no bias-initialisation pass.
// (The reference: gather iterator + mma.sync tiles of 64 pairs of one offset, fp16 accumulate, half2 atomicAdd
// scatter, trt/spconv/mm/kernel.h:84-179, mm/output_iterator.h:189-206.)
//
// CTA = 6 warps, persistent over tiles (tile = blockIdx.x, += gridDim.x):
//   warp 0    producer: scans the tile's offsets, issues the gathers and the weight loads into an smem ring
//   warp 1    MMA issuer (one elected lane); owns the TMEM allocation (two accumulators, double buffered)
//   warps 2-5 epilogue: TMEM -> registers -> global
// Stages and accumulators are handed over through mbarriers; every wait is bounded (about one second) and on
// expiry raises an error word, lets the CTA drain and return instead of spinning.
#include <cuda.h>

#include "common.cuh"
#include "spconv_mm_internal.h"

namespace d3d {
namespace {

constexpr int kTcThreads = 192;
constexpr int kTileRows = 128;
constexpr int kMaxStages = 8;
constexpr int kNumAcc = 2;
constexpr unsigned long long kWaitLimitNs = 1000ull * 1000ull * 1000ull;

__device__ int g_tc_error;  // 0 ok; otherwise the code of the first wait that gave up

enum StageFlags : int { kFirst = 1, kLast = 2, kEmptyTile = 4, kStop = 8 };

struct TcParams {
  const int32_t* table;  // [kvol][pitch]
  int64_t pitch;
  int64_t m_max;
  int32_t n_in_rows;  // rows of the gathered tensor (out-of-range row index = zero fill)
  int kvol, cin, cout;
  int num_tiles;
  int stages;
  uint32_t a_bytes, b_bytes;  // per stage, each a multiple of 1024
  int row_bytes;              // bytes of one smem row = min(cin, 64) * 2
  int kchunk;                 // input channels per stage (cin, or a 64-multiple part of it when cin is large)
  int kparts;                 // cin / kchunk: stages per kernel offset
  int chunks;                 // kchunk / 64 (at least 1): swizzle-span wide column blocks per stage
  uint32_t idesc;
  uint32_t layout_type;  // UMMA smem layout code: 6 = 32B, 4 = 64B, 2 = 128B swizzle
  uint32_t tmem_cols;
  const float* bias;
  void* out;
  const void* residual;
  int relu;
  int is_bf16;
};

// ---- PTX wrappers ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false (and records `code`) when the barrier did not flip within the limit or another role
// already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (global_ns() - t0 > kWaitLimitNs) {
      *abort_flag = code;
      atomicCAS(&g_tc_error, 0, code);
      return false;
    }
  }
}

__device__ __forceinline__ void tma_gather4(const CUtensorMap* map, uint64_t* bar, void* dst, int x, int4 rows) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      :
      : "r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(rows.x), "r"(rows.y), "r"(rows.z),
        "r"(rows.w)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d(const CUtensorMap* map, uint64_t* bar, void* dst, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, "
      "%24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand descriptor: rows of `row_bytes` (the swizzle span), groups of 8 rows `8 * row_bytes` apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t sbo_bytes, uint32_t layout_type) {
  uint64_t d = (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;                         // leading byte offset: unused for swizzled K-major, 1 by convention
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;                         // descriptor version of sm_100
  d |= (uint64_t)layout_type << 61;
  return d;
}

struct __align__(8) Shared {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[kNumAcc];
  uint64_t acc_empty[kNumAcc];
  int stage_k[kMaxStages];
  int stage_flags[kMaxStages];
  int acc_empty_tile[kNumAcc];
  uint32_t tmem_base;
  int abort_flag;
};

template <bool kBf16>
__device__ __forceinline__ void store_chunk(const uint32_t* acc, int n, const float* bias_s, int col0, void* out_row,
                                            const void* res_row, int relu) {
  // n = 16 or 32 accumulator columns starting at col0 of this thread's row
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j)
    if (j < n) v[j] = __uint_as_float(acc[j]) + bias_s[col0 + j];
  if (res_row) {
    const uint4* r4 = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(res_row) + col0);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (q * 8 < n) {
        uint4 raw = __ldg(r4 + q);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float lo, hi;
          if (kBf16) {
            lo = __uint_as_float(w[e] << 16), hi = __uint_as_float(w[e] & 0xFFFF0000u);
          } else {
            __half2 h = *reinterpret_cast<const __half2*>(&w[e]);
            lo = __low2float(h), hi = __high2float(h);
          }
          v[q * 8 + 2 * e] += lo, v[q * 8 + 2 * e + 1] += hi;
        }
      }
    }
  }
  uint4* o4 = reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(out_row) + col0);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    if (q * 8 < n) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float a = v[q * 8 + 2 * e], b = v[q * 8 + 2 * e + 1];
        if (relu) a = fmaxf(a, 0.f), b = fmaxf(b, 0.f);
        if (kBf16) {
          __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
          w[e] = *reinterpret_cast<uint32_t*>(&h);
        } else {
          __half2 h = __floats2half2_rn(a, b);
          w[e] = *reinterpret_cast<uint32_t*>(&h);
        }
      }
      o4[q] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

__global__ void __launch_bounds__(kTcThreads, 1)
spconv_mm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const TcParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // dynamic smem: [stages x (A | B)] aligned to 1024, then the bias, then the control block
  const uint32_t raw_addr = smem_u32(smem_raw);
  unsigned char* tiles = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const uint32_t stage_bytes = p.a_bytes + p.b_bytes;
  float* bias_s = reinterpret_cast<float*>(tiles + (size_t)p.stages * stage_bytes);
  Shared* sh = reinterpret_cast<Shared*>(bias_s + ((p.cout + 1) & ~1));
  volatile int* abort_flag = &sh->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) mbar_init(&sh->full[s], 1), mbar_init(&sh->empty[s], 1);
    for (int a = 0; a < kNumAcc; ++a) mbar_init(&sh->acc_full[a], 1), mbar_init(&sh->acc_empty[a], 4);
    sh->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int c = threadIdx.x; c < p.cout; c += kTcThreads) bias_s[c] = p.bias[c];
  if (warp == 1) tmem_alloc(&sh->tmem_base, p.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    const uint32_t tx_bytes = (uint32_t)kTileRows * p.kchunk * 2 + (uint32_t)p.cout * p.kchunk * 2;
    for (int tile = blockIdx.x; ok; tile += gridDim.x) {
      const bool stop = tile >= p.num_tiles;
      uint32_t mask = 0;
      if (!stop) {
        const int32_t* trow = p.table + (int64_t)tile * kTileRows + 4 * lane;
        for (int k = 0; k < p.kvol; ++k) {
          int4 r = __ldg(reinterpret_cast<const int4*>(trow + (int64_t)k * p.pitch));
          bool any = (r.x >= 0) | (r.y >= 0) | (r.z >= 0) | (r.w >= 0);
          if (__ballot_sync(0xffffffffu, any)) mask |= 1u << k;
        }
      }
      if (stop || mask == 0) {  // a control stage: nothing to load
        ok = mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag, 11);
        if (!ok) break;
        if (lane == 0) {
          sh->stage_k[stage] = 0;
          sh->stage_flags[stage] = stop ? kStop : (kEmptyTile | kFirst | kLast);
          mbar_arrive(&sh->full[stage]);
        }
        __syncwarp();
        if (++stage == p.stages) stage = 0, phase ^= 1;
        if (stop) break;
        continue;
      }
      const int first_k = __ffs(mask) - 1, last_k = 31 - __clz(mask);
      for (uint32_t m = mask; m && ok; m &= m - 1) {
        const int k = __ffs(m) - 1;
        int4 r = __ldg(reinterpret_cast<const int4*>(p.table + (int64_t)k * p.pitch + (int64_t)tile * kTileRows +
                                                     4 * lane));
        // a missing neighbour (or a stale id beyond the gathered tensor) is addressed one row past the end:
        // the TMA fills that row with zeros
        r.x = (r.x < 0 || r.x >= p.n_in_rows) ? p.n_in_rows : r.x;
        r.y = (r.y < 0 || r.y >= p.n_in_rows) ? p.n_in_rows : r.y;
        r.z = (r.z < 0 || r.z >= p.n_in_rows) ? p.n_in_rows : r.z;
        r.w = (r.w < 0 || r.w >= p.n_in_rows) ? p.n_in_rows : r.w;
        for (int part = 0; part < p.kparts; ++part) {
          ok = mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag, 12);
          if (!ok) break;
          unsigned char* a_dst = tiles + (size_t)stage * stage_bytes;
          unsigned char* b_dst = a_dst + p.a_bytes;
          const int x0 = part * p.kchunk;
          if (lane == 0) {
            sh->stage_k[stage] = k;
            sh->stage_flags[stage] = ((k == first_k && part == 0) ? kFirst : 0) |
                                     ((k == last_k && part == p.kparts - 1) ? kLast : 0);
            mbar_arrive_expect_tx(&sh->full[stage], tx_bytes);
            for (int c = 0; c < p.chunks; ++c)
              tma_load_2d(&map_b, &sh->full[stage], b_dst + (size_t)c * p.cout * p.row_bytes, x0 + c * 64,
                          k * p.cout);
          }
          __syncwarp();
          for (int c = 0; c < p.chunks; ++c)
            tma_gather4(&map_a, &sh->full[stage],
                        a_dst + (size_t)c * kTileRows * p.row_bytes + 4 * lane * p.row_bytes, x0 + c * 64, r);
          if (++stage == p.stages) stage = 0, phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    int stage = 0, acc = 0;
    uint32_t phase = 0, acc_phase = 0;
    const uint32_t sbo = 8u * p.row_bytes;
    const int ksteps = p.kchunk / 16;
    bool ok = true;
    while (ok) {
      ok = mbar_wait(&sh->full[stage], phase, abort_flag, 21);
      if (!ok) break;
      tc_fence_after();
      const int flags = sh->stage_flags[stage];
      if (flags & kStop) break;
      if (flags & kFirst) {
        ok = mbar_wait(&sh->acc_empty[acc], acc_phase ^ 1, abort_flag, 22);
        if (!ok) break;
        tc_fence_after();
      }
      if (lane == 0) {
        if (flags & kEmptyTile) {
          sh->acc_empty_tile[acc] = 1;
          mbar_arrive(&sh->empty[stage]);
          mbar_arrive(&sh->acc_full[acc]);
        } else {
          const uint32_t a_addr = smem_u32(tiles + (size_t)stage * stage_bytes);
          const uint32_t b_addr = a_addr + p.a_bytes;
          const uint32_t d_addr = tmem_base + (uint32_t)(acc * p.cout);
          for (int ks = 0; ks < ksteps; ++ks) {
            const int chunk = ks >> 2, within = (ks & 3) * 32;
            uint64_t da = make_desc(a_addr + chunk * kTileRows * p.row_bytes + within, sbo, p.layout_type);
            uint64_t db = make_desc(b_addr + chunk * p.cout * p.row_bytes + within, sbo, p.layout_type);
            umma_f16(d_addr, da, db, p.idesc, ((flags & kFirst) && ks == 0) ? 0u : 1u);
          }
          umma_commit(&sh->empty[stage]);  // the stage may be refilled once these MMAs have read it
          if (flags & kLast) {
            sh->acc_empty_tile[acc] = 0;
            umma_commit(&sh->acc_full[acc]);
          }
        }
      }
      __syncwarp();
      if (flags & kLast) {
        if (++acc == kNumAcc) acc = 0, acc_phase ^= 1;
      }
      if (++stage == p.stages) stage = 0, phase ^= 1;
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) belong to this warp
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
      ok = mbar_wait(&sh->acc_full[acc], acc_phase, abort_flag, 31);
      if (!ok) break;
      tc_fence_after();
      const bool empty_tile = sh->acc_empty_tile[acc] != 0;
      const int64_t row = (int64_t)tile * kTileRows + quad * 32 + lane;
      const bool row_ok = row < p.m_max;
      unsigned short* out_row = reinterpret_cast<unsigned short*>(p.out) + row * p.cout;
      const unsigned short* res_row =
          (p.residual && row_ok) ? reinterpret_cast<const unsigned short*>(p.residual) + row * p.cout : nullptr;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * p.cout);
      for (int c0 = 0; c0 < p.cout; c0 += 32) {
        const int n = p.cout - c0 >= 32 ? 32 : 16;
        uint32_t v[32];
        if (empty_tile) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;
        } else {
          if (n == 32) tmem_ld32(taddr + c0, v);
          else tmem_ld16(taddr + c0, v);
          tmem_ld_wait();
        }
        if (row_ok) {
          if (p.is_bf16) store_chunk<true>(v, n, bias_s, c0, out_row, res_row, p.relu);
          else store_chunk<false>(v, n, bias_s, c0, out_row, res_row, p.relu);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->acc_empty[acc]);
      if (++acc == kNumAcc) acc = 0, acc_phase ^= 1;
    }
  }

  // teardown: everyone meets, then the allocating warp returns the tensor memory
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

// ---- host --------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

bool make_map(CUtensorMap* map, int dtype, const void* base, uint64_t cols, uint64_t rows, uint32_t box_cols,
              uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapSwizzle sw = box_cols * 2 == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                             : box_cols * 2 == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMapDataType dt = dtype == D3D_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct TcState {
  CUtensorMap map_b;
  bool map_b_ok = false;
};

}  // namespace

bool spconv_mm_tc_eligible(const d3d_spconv_mm_s* h, int dtype) {
  if (dtype != D3D_HALF && dtype != D3D_BF16) return false;
  const int cin = h->p.in_channels, cout = h->p.out_channels, kvol = h->p.kernel_vol;
  if (!(cin == 16 || cin == 32 || cin == 64 || cin == 128 || cin == 256)) return false;
  if (cout % 16 != 0 || cout < 16 || cout > 256) return false;
  if (kvol > 32) return false;
  return encode_fn() != nullptr;
}

void spconv_mm_tc_release(d3d_spconv_mm_s* h) {
  delete reinterpret_cast<TcState*>(h->tc_state);
  h->tc_state = nullptr;
}

int launch_spconv_mm_tc(const MmLaunch& a) {
  d3d_spconv_mm_s* h = const_cast<d3d_spconv_mm_s*>(a.h);
  const int cin = h->p.in_channels, cout = h->p.out_channels, kvol = h->p.kernel_vol;
  const int64_t m_max = h->p.max_num_act_out;
  if (m_max == 0) return D3D_OK;
  D3D_REQUIRE(a.max_num_act_in >= 1 && a.max_num_act_in < (1ll << 31), D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(reinterpret_cast<uintptr_t>(a.in_feats) % 16 == 0 && reinterpret_cast<uintptr_t>(a.out_feats) % 16 == 0,
              D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(!a.residual || reinterpret_cast<uintptr_t>(a.residual) % 16 == 0, D3D_ERR_INVALID_ARGUMENT);
  if (!h->tc_state) h->tc_state = new TcState();
  TcState* st = reinterpret_cast<TcState*>(h->tc_state);
  const uint32_t box_cols = cin < 64 ? cin : 64;
  if (!st->map_b_ok) {
    st->map_b_ok = make_map(&st->map_b, a.dtype, h->wt_dev, cin, (uint64_t)kvol * cout, box_cols, cout);
    D3D_REQUIRE(st->map_b_ok, D3D_ERR_CUDA);
  }
  CUtensorMap map_a;
  D3D_REQUIRE(make_map(&map_a, a.dtype, a.in_feats, cin, (uint64_t)a.max_num_act_in, box_cols, 1), D3D_ERR_CUDA);

  TcParams p;
  p.table = a.table;
  p.pitch = (m_max + 127) / 128 * 128;
  p.m_max = m_max;
  p.n_in_rows = (int32_t)a.max_num_act_in;
  p.kvol = kvol, p.cin = cin, p.cout = cout;
  p.num_tiles = (int)(p.pitch / kTileRows);
  p.row_bytes = (int)box_cols * 2;
  // a stage holds `kchunk` input channels of one kernel offset; split large Cin so that at least two stages fit
  const size_t ctrl = 1024 + align_up((size_t)cout * 4 + 8, 16) + sizeof(Shared);
  int kchunk = cin;
  while (kchunk > 64 && 2 * (align_up((size_t)kTileRows * kchunk * 2, 1024) + align_up((size_t)cout * kchunk * 2, 1024)) >
                            200 * 1024 - ctrl)
    kchunk /= 2;
  p.kchunk = kchunk;
  p.kparts = cin / kchunk;
  p.chunks = kchunk <= 64 ? 1 : kchunk / 64;
  p.a_bytes = (uint32_t)align_up((size_t)kTileRows * kchunk * 2, 1024);
  p.b_bytes = (uint32_t)align_up((size_t)cout * kchunk * 2, 1024);
  p.layout_type = p.row_bytes == 32 ? 6u : p.row_bytes == 64 ? 4u : 2u;
  const uint32_t fmt = a.dtype == D3D_BF16 ? 1u : 0u;
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(cout >> 3) << 17) | ((uint32_t)(kTileRows >> 4) << 24);
  uint32_t cols = 32;
  while (cols < (uint32_t)(kNumAcc * cout)) cols <<= 1;
  p.tmem_cols = cols;
  p.bias = h->b_dev;
  p.out = a.out_feats;
  p.residual = a.residual;
  p.relu = a.relu;
  p.is_bf16 = a.dtype == D3D_BF16;
  // shared memory: as many stages as fit in ~200 KB (at least 2, at most kMaxStages); never less than 120 KB so that
  // one CTA owns an SM and its tensor memory
  const size_t stage_bytes = (size_t)p.a_bytes + p.b_bytes;
  int stages = (int)((200 * 1024 - ctrl) / stage_bytes);
  stages = stages > kMaxStages ? kMaxStages : stages;
  D3D_REQUIRE(stages >= 2, D3D_ERR_TOO_LARGE);
  p.stages = stages;
  size_t smem = ctrl + (size_t)stages * stage_bytes;
  if (smem < 120 * 1024) smem = 120 * 1024;
  static bool attr_set[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return D3D_ERR_CUDA;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(spconv_mm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) !=
        cudaSuccess)
      return D3D_ERR_CUDA;
    attr_set[dev] = true;
  }
  int grid = p.num_tiles < kNumSMs ? p.num_tiles : kNumSMs;
  spconv_mm_tc_kernel<<<grid, kTcThreads, smem, reinterpret_cast<cudaStream_t>(a.stream)>>>(map_a, st->map_b, p);
  D3D_CHECK_LAUNCH();
  return D3D_OK;
}

}  // namespace d3d

// Debug aid without a reference counterpart (the reference prints CUDA errors, trt/include/common/macros.h:14-34):
// synchronises the device and returns the error word the tensor-core kernel raises when one of its bounded waits
// expires (0 = none), clearing it.
extern "C" int d3d_debug_take_kernel_error(int* code) {
  if (!code) return D3D_ERR_INVALID_ARGUMENT;
  int zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return D3D_ERR_CUDA;
  if (cudaMemcpyFromSymbol(code, d3d::g_tc_error, sizeof(int)) != cudaSuccess) return D3D_ERR_CUDA;
  if (cudaMemcpyToSymbol(d3d::g_tc_error, &zero, sizeof(int)) != cudaSuccess) return D3D_ERR_CUDA;
  return D3D_OK;
}
