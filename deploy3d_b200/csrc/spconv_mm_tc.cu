// SPConvMM on the 5th-generation tensor cores: output-stationary implicit GEMM.
//
// For a tile of 128 consecutive output voxels and every kernel offset k that feeds at least one of them:
//   A = the 128 input rows named by the neighbour table (zero rows where the neighbour is missing), staged in shared
//       memory in the K-major swizzled layout the tensor core reads,
//   B = W[k]^T, K-major, loaded by a tiled TMA copy,
//   D += A * B with tcgen05.mma (M = 128, N = Cout, K = 16 per instruction), fp32 accumulator in tensor memory.
// All offsets of a tile accumulate into the same TMEM columns; the epilogue reads them once with tcgen05.ld, adds
// bias (+ residual), applies ReLU, converts and stores the row.  No atomics, no bias-initialisation pass.
// (The reference: gather iterator + mma.sync tiles of 64 pairs of one offset, fp16 accumulate, half2 atomicAdd
// scatter, trt/spconv/mm/kernel.h:84-179, mm/output_iterator.h:189-206.)
//
// Two producers exist for the A operand, same consumer side:
//   * TMA gather   tile::gather4, four arbitrary rows per instruction issued by one warp; missing neighbours are
//                  addressed out of bounds so the TMA zero-fills them.  Measured on B200: about 11 ns per gathered
//                  row whatever its width (a request-rate limit of the TMA unit), i.e. ~1.4 us per (tile, offset).
//   * cp.async     four producer warps, 16-byte LDGSTS per thread with zero-fill for missing rows, written straight
//                  into the swizzled layout; an order of magnitude more row requests in flight.  This is the default.
// CTA roles (persistent over tiles: tile = blockIdx.x, += gridDim.x):
//   producer warp(s)  prefetch the tile's neighbour ids into smem (one bulk copy), find the offsets that occur,
//                     fill the smem ring: up to `group` offsets per stage
//   MMA warp          one elected lane issues tcgen05.mma; owns the TMEM allocation (two accumulators)
//   4 epilogue warps  TMEM -> registers -> global
// Stages and accumulators are handed over through mbarriers; every wait is bounded (about one second) and on
// expiry raises an error word, lets the CTA drain and return instead of spinning.
#include <cuda.h>

#include "common.cuh"
#include "spconv_mm_internal.h"

namespace d3d {
namespace {

constexpr int kTileRows = 128;
constexpr int kMaxStages = 8;
constexpr int kNumAcc = 2;
constexpr int kMaxGroup = 8;  // kernel offsets that may share one pipeline stage
constexpr unsigned long long kWaitLimitNs = 1000ull * 1000ull * 1000ull;

__device__ int g_tc_error;  // 0 ok; otherwise the code of the first wait that gave up

enum StageFlags : int { kFirst = 1, kLast = 2, kEmptyTile = 4, kStop = 8 };

struct TcParams {
  const int32_t* table;  // [tiles][kvol][128]
  const void* in_feats;  // [n_in_rows][cin]
  int64_t m_max;
  int32_t n_in_rows;  // rows of the gathered tensor (out-of-range row index = zero fill)
  int kvol, cin, cout;
  int num_tiles;
  int stages;
  int group;                  // kernel offsets per stage (> 1 only when kparts == 1)
  uint32_t a_bytes, b_bytes;  // per (offset, K part) block, each a multiple of 1024
  uint32_t idx_bytes;         // kvol * 512: neighbour ids of one tile
  int row_bytes;              // bytes of one smem row = min(cin, 64) * 2
  int kchunk;                 // input channels per block (cin, or a 64-multiple part of it when cin is large)
  int kparts;                 // cin / kchunk: blocks per kernel offset
  int chunks;                 // kchunk / 64 (at least 1): swizzle-span wide column blocks per block
  uint32_t idesc;
  uint32_t layout_type;  // UMMA smem layout code: 6 = 32B, 4 = 64B, 2 = 128B swizzle
  uint32_t tmem_cols;
  uint32_t full_count;  // arrivals that complete a `full` barrier (1 for the TMA producer, 129 for cp.async)
  int b_resident;       // all kvol weight blocks stay in smem for the whole kernel (small layers)
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
// Contiguous global -> shared copy (both 16-byte aligned, size a multiple of 16) signalled on an mbarrier.
__device__ __forceinline__ void bulk_load_1d(uint64_t* bar, void* dst, const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :
               : "r"(smem_u32(dst)), "l"((uint64_t)src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// 16-byte asynchronous copy; src_bytes = 0 writes 16 zero bytes without reading global memory.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// The barrier receives one arrival (counted in its expected arrivals) once all cp.async issued so far by this
// thread have landed.
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

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
  uint64_t idx_full[2];
  uint64_t idx_free[2];
  uint64_t b_ready;           // resident weights have landed
  int stage_cnt[kMaxStages];  // (offset, K part) blocks in the stage
  int stage_flags[kMaxStages];
  unsigned char stage_k[kMaxStages][kMaxGroup];  // kernel offset of each block
  int acc_empty_tile[kNumAcc];
  uint32_t tmem_base;
  int abort_flag;
};

// Carved dynamic shared memory: [stages x (group A blocks | group B blocks)] aligned to 1024, two neighbour-id
// buffers [kvol][128], the bias, the control block.
struct Smem {
  unsigned char* tiles;
  unsigned char* bres;  // resident weights [kvol][b_bytes] (when p.b_resident)
  int32_t* idx;
  float* bias;
  Shared* sh;
  uint32_t stage_bytes;
};
__device__ __forceinline__ Smem carve_smem(unsigned char* raw, const TcParams& p) {
  Smem s;
  const uint32_t raw_addr = smem_u32(raw);
  s.tiles = raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  s.stage_bytes = (uint32_t)p.group * (p.a_bytes + (p.b_resident ? 0u : p.b_bytes));
  s.bres = s.tiles + (size_t)p.stages * s.stage_bytes;
  s.idx = reinterpret_cast<int32_t*>(s.bres + (p.b_resident ? (size_t)p.kvol * p.b_bytes : 0));
  s.bias = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(s.idx) + 2 * (size_t)p.idx_bytes);
  s.sh = reinterpret_cast<Shared*>(s.bias + ((p.cout + 1) & ~1));
  return s;
}

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

// Barrier initialisation, bias staging and the TMEM allocation (by warp `mma_warp`); returns the TMEM base address.
__device__ __forceinline__ uint32_t cta_setup(const TcParams& p, const Smem& s, int producer_warps, int mma_warp) {
  Shared* sh = s.sh;
  if (threadIdx.x == 0) {
    for (int i = 0; i < p.stages; ++i) mbar_init(&sh->full[i], (int)p.full_count), mbar_init(&sh->empty[i], 1);
    for (int a = 0; a < kNumAcc; ++a) mbar_init(&sh->acc_full[a], 1), mbar_init(&sh->acc_empty[a], 4);
    for (int b = 0; b < 2; ++b) mbar_init(&sh->idx_full[b], 1), mbar_init(&sh->idx_free[b], producer_warps);
    mbar_init(&sh->b_ready, 1);
    sh->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int c = threadIdx.x; c < p.cout; c += blockDim.x) s.bias[c] = p.bias[c];
  if ((int)(threadIdx.x >> 5) == mma_warp) tmem_alloc(&sh->tmem_base, p.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  return sh->tmem_base;
}

// Low word of a K-major operand descriptor: start address in 16-byte units, leading byte offset 1 (unused for the
// swizzled K-major layouts).  Advancing the operand by `d` bytes adds d / 16 to this word.
__device__ __forceinline__ uint32_t desc_lo(uint32_t smem_addr) { return ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16); }

// The kSteps tcgen05.mma instructions (K = 16 each) of one (offset, K part) block.
template <int kSteps>
__device__ __forceinline__ void issue_block(uint32_t d_addr, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                            uint32_t idesc, uint32_t& accumulate, uint32_t cs_a, uint32_t cs_b) {
#pragma unroll
  for (int ks = 0; ks < kSteps; ++ks) {
    const uint32_t within = (uint32_t)(ks & 3) * 2u;  // 32 bytes per K step inside the swizzle span
    const uint64_t da = ((uint64_t)desc_hi << 32) | (a_lo + (uint32_t)(ks >> 2) * cs_a + within);
    const uint64_t db = ((uint64_t)desc_hi << 32) | (b_lo + (uint32_t)(ks >> 2) * cs_b + within);
    umma_f16(d_addr, da, db, idesc, accumulate);
    accumulate = 1u;
  }
}

// MMA issuer warp: consumes the stages in ring order until the stop stage.
__device__ __forceinline__ void mma_role(const TcParams& p, const Smem& s, uint32_t tmem_base) {
  Shared* sh = s.sh;
  volatile int* abort_flag = &sh->abort_flag;
  const int lane = threadIdx.x & 31;
  int stage = 0, acc = 0;
  uint32_t phase = 0, acc_phase = 0;
  const int ksteps = p.kchunk / 16;
  // descriptor pieces that never change: high word (group stride, version, swizzle), and the distance in 16-byte
  // units between the 64-column blocks of the A and the B operand
  const uint32_t desc_hi = ((8u * p.row_bytes) >> 4) | (1u << 14) | (p.layout_type << 29);
  const uint32_t cs_a = (uint32_t)(kTileRows * p.row_bytes) >> 4, cs_b = (uint32_t)(p.cout * p.row_bytes) >> 4;
  bool ok = true;
  if (p.b_resident) ok = mbar_wait(&sh->b_ready, 0, abort_flag, 23);
  const uint32_t bres_addr = smem_u32(s.bres);
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
      fence_proxy_async();  // rows written by cp.async (generic proxy) -> tensor-core reads (async proxy)
      if (flags & kEmptyTile) {
        sh->acc_empty_tile[acc] = 1;
        mbar_arrive(&sh->empty[stage]);
        mbar_arrive(&sh->acc_full[acc]);
      } else {
        const uint32_t a_base = smem_u32(s.tiles + (size_t)stage * s.stage_bytes);
        const uint32_t b_base = a_base + (uint32_t)p.group * p.a_bytes;
        const uint32_t d_addr = tmem_base + (uint32_t)(acc * p.cout);
        const int cnt = sh->stage_cnt[stage];
        uint32_t accumulate = (flags & kFirst) ? 0u : 1u;
        for (int e = 0; e < cnt; ++e) {
          const uint32_t a_addr = a_base + (uint32_t)e * p.a_bytes;
          const uint32_t b_addr = p.b_resident ? bres_addr + (uint32_t)sh->stage_k[stage][e] * p.b_bytes
                                               : b_base + (uint32_t)e * p.b_bytes;
          const uint32_t a_lo = desc_lo(a_addr), b_lo = desc_lo(b_addr);
          switch (ksteps) {
            case 1: issue_block<1>(d_addr, a_lo, b_lo, desc_hi, p.idesc, accumulate, cs_a, cs_b); break;
            case 2: issue_block<2>(d_addr, a_lo, b_lo, desc_hi, p.idesc, accumulate, cs_a, cs_b); break;
            case 4: issue_block<4>(d_addr, a_lo, b_lo, desc_hi, p.idesc, accumulate, cs_a, cs_b); break;
            default: issue_block<8>(d_addr, a_lo, b_lo, desc_hi, p.idesc, accumulate, cs_a, cs_b); break;
          }
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
}

// Epilogue warp `quad` (= warp index mod 4: it may touch TMEM lanes [32*quad, 32*quad + 32)).
__device__ __forceinline__ void epilogue_role(const TcParams& p, const Smem& s, uint32_t tmem_base, int quad) {
  Shared* sh = s.sh;
  volatile int* abort_flag = &sh->abort_flag;
  const int lane = threadIdx.x & 31;
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
        if (p.is_bf16) store_chunk<true>(v, n, s.bias, c0, out_row, res_row, p.relu);
        else store_chunk<false>(v, n, s.bias, c0, out_row, res_row, p.relu);
      }
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(&sh->acc_empty[acc]);
    if (++acc == kNumAcc) acc = 0, acc_phase ^= 1;
  }
}

// All roles meet, then the allocating warp returns the tensor memory.
__device__ __forceinline__ void cta_teardown(const TcParams& p, uint32_t tmem_base, int mma_warp) {
  tc_fence_before();
  __syncthreads();
  if ((int)(threadIdx.x >> 5) == mma_warp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

// Copy the 32 operand rows [row0, row0 + 32) of one (offset, K part) block with 16-byte cp.async pieces.
// kPieces = 16-byte pieces per row (row bytes / 16).  Consecutive lanes take consecutive pieces of a row, so one
// warp instruction reads 32 / kPieces whole rows: few cache lines per instruction on the global side, whole
// 128-byte lines on the shared side.  Piece j of row r lands at the XOR-swizzled position the tensor core expects;
// pieces 8.. belong to the next 64-column block (`blk_stride` bytes further).
template <int kPieces>
__device__ __forceinline__ void copy_rows(uint32_t a_addr, const int32_t* ids_k, const unsigned char* feats,
                                          int row_src_bytes, int n_in_rows, int row0, int lane, int row_bytes,
                                          int swz_shift, int swz_mask, uint32_t blk_stride) {
  constexpr int kRowsPerInstr = 32 / kPieces;
  const int j = lane % kPieces, rsub = lane / kPieces;
  int id[kPieces];
#pragma unroll
  for (int it = 0; it < kPieces; ++it) id[it] = ids_k[row0 + it * kRowsPerInstr + rsub];
  const uint32_t dst0 = a_addr + (uint32_t)(j >> 3) * blk_stride;
#pragma unroll
  for (int it = 0; it < kPieces; ++it) {
    const int row = row0 + it * kRowsPerInstr + rsub;
    const bool valid = id[it] >= 0 && id[it] < n_in_rows;
    const unsigned char* src = feats + (size_t)(valid ? id[it] : 0) * row_src_bytes + j * 16;
    const uint32_t dst = dst0 + row * row_bytes + ((((uint32_t)j & 7u) ^ (uint32_t)((row >> swz_shift) & swz_mask)) << 4);
    cp_async_16(dst, src, valid ? 16u : 0u);
  }
}

// Producer warps (1 for the TMA gather, 4 for cp.async).  Every producer warp walks the same tiles and stages; the
// leader (warp 0, lane 0) additionally prefetches neighbour ids, publishes the stage descriptors and loads B.
template <bool kTma>
__device__ __forceinline__ void producer_role(const TcParams& p, const Smem& s, const CUtensorMap* map_a,
                                              const CUtensorMap* map_b, int pw) {
  Shared* sh = s.sh;
  volatile int* abort_flag = &sh->abort_flag;
  const int lane = threadIdx.x & 31;
  const bool leader = pw == 0 && lane == 0;
  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  const uint32_t a_tx = (uint32_t)kTileRows * p.kchunk * 2, b_tx = (uint32_t)p.cout * p.kchunk * 2;
  const int ids_per_tile = p.kvol * kTileRows;
  const int cpr = p.kchunk / 8;  // 16-byte pieces per gathered row
  const int swz_shift = p.row_bytes == 128 ? 0 : p.row_bytes == 64 ? 1 : 2;
  const int swz_mask = p.row_bytes == 128 ? 7 : p.row_bytes == 64 ? 3 : 1;
  int buf = 0;
  uint32_t idx_phase = 0;   // bit b: parity to wait for on idx_full[b]
  uint32_t free_phase = 0;  // bit b: parity to wait for on idx_free[b] (leader only)
  if (leader && (int)blockIdx.x < p.num_tiles) {
    mbar_arrive_expect_tx(&sh->idx_full[0], p.idx_bytes);
    bulk_load_1d(&sh->idx_full[0], s.idx, p.table + (int64_t)blockIdx.x * ids_per_tile, p.idx_bytes);
    if (p.b_resident) {  // all weight blocks once, in the layout the per-stage loads would have produced
      mbar_arrive_expect_tx(&sh->b_ready, (uint32_t)p.kvol * b_tx);
      for (int k = 0; k < p.kvol; ++k)
        for (int c = 0; c < p.chunks; ++c)
          tma_load_2d(map_b, &sh->b_ready, s.bres + (size_t)k * p.b_bytes + (size_t)c * p.cout * p.row_bytes, c * 64,
                      k * p.cout);
    }
  }
  for (int tile = blockIdx.x; ok; tile += gridDim.x) {
    const bool stop = tile >= p.num_tiles;
    uint32_t mask = 0;
    const int32_t* ids = s.idx + (size_t)buf * ids_per_tile;
    if (!stop) {
      // prefetch the ids of this CTA's next tile into the other buffer once all producer warps have released it
      const int next = tile + gridDim.x;
      if (leader && next < p.num_tiles) {
        bool free_ok = true;
        if (tile != (int)blockIdx.x) {
          free_ok = mbar_wait(&sh->idx_free[buf ^ 1], (free_phase >> (buf ^ 1)) & 1u, abort_flag, 14);
          free_phase ^= 1u << (buf ^ 1);
        }
        if (free_ok) {
          mbar_arrive_expect_tx(&sh->idx_full[buf ^ 1], p.idx_bytes);
          bulk_load_1d(&sh->idx_full[buf ^ 1], s.idx + (size_t)(buf ^ 1) * ids_per_tile,
                       p.table + (int64_t)next * ids_per_tile, p.idx_bytes);
        }
      }
      __syncwarp();
      ok = mbar_wait(&sh->idx_full[buf], (idx_phase >> buf) & 1u, abort_flag, 13);
      if (!ok) break;
      idx_phase ^= 1u << buf;
      for (int k = 0; k < p.kvol; ++k) {
        int4 r = *reinterpret_cast<const int4*>(ids + k * kTileRows + 4 * lane);
        bool any = (r.x >= 0) | (r.y >= 0) | (r.z >= 0) | (r.w >= 0);
        if (__ballot_sync(0xffffffffu, any)) mask |= 1u << k;
      }
    }
    if (stop || mask == 0) {  // a control stage: nothing to load
      ok = mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag, 11);
      if (!ok) break;
      if (leader) {
        sh->stage_cnt[stage] = 0;
        sh->stage_flags[stage] = stop ? kStop : (kEmptyTile | kFirst | kLast);
        mbar_arrive(&sh->full[stage]);
      }
      if (!kTma) mbar_arrive(&sh->full[stage]);
      __syncwarp();
      if (++stage == p.stages) stage = 0, phase ^= 1;
      if (stop) break;
    }
    // data stages: up to `group` offsets per stage (one offset, one K part when Cin is split)
    uint32_t m = mask;
    int part = 0;
    while (m && ok) {
      ok = mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag, 12);
      if (!ok) break;
      const bool first = (m == mask) && part == 0;
      uint32_t take = 0, rest = m;
      int cnt = 0;
      if (p.kparts == 1) {
        for (; cnt < p.group && rest; ++cnt) take |= rest & (0u - rest), rest &= rest - 1;
      } else {
        take = m & (0u - m), cnt = 1;
        if (part == p.kparts - 1) rest &= rest - 1;
      }
      const int x0 = part * p.kchunk;
      unsigned char* a_base = s.tiles + (size_t)stage * s.stage_bytes;
      unsigned char* b_base = a_base + (size_t)p.group * p.a_bytes;
      if (leader) {
        sh->stage_cnt[stage] = cnt;
        sh->stage_flags[stage] = (first ? kFirst : 0) | (rest == 0 ? kLast : 0);
        int e = 0;
        for (uint32_t t = take; t; t &= t - 1, ++e) sh->stage_k[stage][e] = (unsigned char)(__ffs(t) - 1);
        const uint32_t tx = (uint32_t)cnt * ((p.b_resident ? 0u : b_tx) + (kTma ? a_tx : 0u));
        if (tx) mbar_arrive_expect_tx(&sh->full[stage], tx);
        else mbar_arrive(&sh->full[stage]);
        e = 0;
        for (uint32_t t = take; t; t &= t - 1, ++e) {
          const int k = __ffs(t) - 1;
          if (!p.b_resident)
            for (int c = 0; c < p.chunks; ++c)
              tma_load_2d(map_b, &sh->full[stage],
                          b_base + (size_t)e * p.b_bytes + (size_t)c * p.cout * p.row_bytes, x0 + c * 64, k * p.cout);
        }
      }
      __syncwarp();
      int e = 0;
      for (uint32_t t = take; t; t &= t - 1, ++e) {
        const int k = __ffs(t) - 1;
        unsigned char* a_blk = a_base + (size_t)e * p.a_bytes;
        if (kTma) {
          int4 r = *reinterpret_cast<const int4*>(ids + k * kTileRows + 4 * lane);
          // a missing neighbour (or a stale id beyond the gathered tensor) is addressed one row past the end:
          // the TMA fills that row with zeros
          r.x = (r.x < 0 || r.x >= p.n_in_rows) ? p.n_in_rows : r.x;
          r.y = (r.y < 0 || r.y >= p.n_in_rows) ? p.n_in_rows : r.y;
          r.z = (r.z < 0 || r.z >= p.n_in_rows) ? p.n_in_rows : r.z;
          r.w = (r.w < 0 || r.w >= p.n_in_rows) ? p.n_in_rows : r.w;
          for (int c = 0; c < p.chunks; ++c)
            tma_gather4(map_a, &sh->full[stage], a_blk + (size_t)c * kTileRows * p.row_bytes + 4 * lane * p.row_bytes,
                        x0 + c * 64, r);
        } else {
          // this warp copies rows [32 * pw, 32 * pw + 32) of the block
          const unsigned char* feats = reinterpret_cast<const unsigned char*>(p.in_feats) + (size_t)x0 * 2;
          const int32_t* ids_k = ids + k * kTileRows;
          const uint32_t a_addr = smem_u32(a_blk);
          switch (cpr) {
            case 2:
              copy_rows<2>(a_addr, ids_k, feats, p.cin * 2, p.n_in_rows, 32 * pw, lane, 32, swz_shift, swz_mask, 0);
              break;
            case 4:
              copy_rows<4>(a_addr, ids_k, feats, p.cin * 2, p.n_in_rows, 32 * pw, lane, 64, swz_shift, swz_mask, 0);
              break;
            case 8:
              copy_rows<8>(a_addr, ids_k, feats, p.cin * 2, p.n_in_rows, 32 * pw, lane, 128, swz_shift, swz_mask, 0);
              break;
            default:
              copy_rows<16>(a_addr, ids_k, feats, p.cin * 2, p.n_in_rows, 32 * pw, lane, 128, swz_shift, swz_mask,
                            kTileRows * 128);
              break;
          }
        }
      }
      if (!kTma) cp_async_arrive(&sh->full[stage]);  // one arrival per producer thread once its copies land
      if (p.kparts > 1 && ++part == p.kparts) part = 0;
      m = rest;
      if (++stage == p.stages) stage = 0, phase ^= 1;
    }
    if (!stop) {  // this warp is done with the id buffer of the tile
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->idx_free[buf]);
      buf ^= 1;
    }
  }
}

// TMA-gather variant: warp 0 producer, warp 1 MMA, warps 2-5 epilogue.
__global__ void __launch_bounds__(192, 1)
spconv_mm_tc_tma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const TcParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const Smem s = carve_smem(smem_raw, p);
  const int warp = threadIdx.x >> 5;
  const uint32_t tmem_base = cta_setup(p, s, 1, 1);
  if (warp == 0) producer_role<true>(p, s, &map_a, &map_b, 0);
  else if (warp == 1) mma_role(p, s, tmem_base);
  else epilogue_role(p, s, tmem_base, warp & 3);
  cta_teardown(p, tmem_base, 1);
}

// cp.async variant: warps 0-3 producers, warp 4 MMA, warps 5-8 epilogue.
__global__ void __launch_bounds__(288, 1)
spconv_mm_tc_cpasync_kernel(const __grid_constant__ CUtensorMap map_b, const TcParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const Smem s = carve_smem(smem_raw, p);
  const int warp = threadIdx.x >> 5;
  const uint32_t tmem_base = cta_setup(p, s, 4, 4);
  if (warp < 4) producer_role<false>(p, s, nullptr, &map_b, warp);
  else if (warp == 4) mma_role(p, s, tmem_base);
  else epilogue_role(p, s, tmem_base, warp & 3);
  cta_teardown(p, tmem_base, 4);
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
  const bool use_tma_gather = h->kernel_choice == 3;
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

  TcParams p;
  p.table = a.table;
  p.in_feats = a.in_feats;
  p.m_max = m_max;
  p.n_in_rows = (int32_t)a.max_num_act_in;
  p.kvol = kvol, p.cin = cin, p.cout = cout;
  p.num_tiles = (int)((m_max + kTileRows - 1) / kTileRows);
  p.row_bytes = (int)box_cols * 2;
  p.idx_bytes = (uint32_t)kvol * kTileRows * 4;
  p.full_count = use_tma_gather ? 1u : 129u;  // leader + (cp.async) every producer thread
  // shared-memory budget: 227 KB per CTA minus alignment slack, the two neighbour-id buffers, bias and control block
  const size_t ctrl = 1024 + 2 * (size_t)p.idx_bytes + align_up((size_t)cout * 4 + 8, 16) + sizeof(Shared);
  const size_t budget = 227 * 1024 - ctrl;
  // a block holds `kchunk` input channels of one kernel offset; split large Cin so that at least two stages fit
  int kchunk = cin;
  while (kchunk > 64 &&
         2 * (align_up((size_t)kTileRows * kchunk * 2, 1024) + align_up((size_t)cout * kchunk * 2, 1024)) > budget)
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
  // small layers keep all weight blocks in shared memory for the whole kernel instead of reloading one per stage
  const size_t bres_bytes = (size_t)kvol * p.b_bytes;
  p.b_resident = (p.kparts == 1 && bres_bytes <= 64 * 1024) ? 1 : 0;
  const size_t ring_budget = budget - (p.b_resident ? bres_bytes : 0);
  // several offsets share a stage when their blocks are small, so that the per-stage hand-over cost is amortised
  const size_t blk_bytes = (size_t)p.a_bytes + (p.b_resident ? 0 : p.b_bytes);
  int group = 1;
  if (p.kparts == 1) {
    group = (int)(48 * 1024 / blk_bytes);
    group = group < 1 ? 1 : group > kMaxGroup ? kMaxGroup : group;
  }
  p.group = group;
  const size_t stage_bytes = (size_t)group * blk_bytes;
  int stages = (int)(ring_budget / stage_bytes);
  stages = stages > kMaxStages ? kMaxStages : stages;
  D3D_REQUIRE(stages >= 2, D3D_ERR_TOO_LARGE);
  p.stages = stages;
  size_t smem = ctrl + (size_t)stages * stage_bytes + (p.b_resident ? bres_bytes : 0);
  if (smem < 120 * 1024) smem = 120 * 1024;  // one CTA per SM: it owns the SM's tensor memory
  static bool attr_set[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return D3D_ERR_CUDA;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(spconv_mm_tc_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) !=
            cudaSuccess ||
        cudaFuncSetAttribute(spconv_mm_tc_cpasync_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) !=
            cudaSuccess)
      return D3D_ERR_CUDA;
    attr_set[dev] = true;
  }
  const int grid = p.num_tiles < kNumSMs ? p.num_tiles : kNumSMs;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(a.stream);
  if (use_tma_gather) {
    CUtensorMap map_a;
    D3D_REQUIRE(make_map(&map_a, a.dtype, a.in_feats, cin, (uint64_t)a.max_num_act_in, box_cols, 1), D3D_ERR_CUDA);
    spconv_mm_tc_tma_kernel<<<grid, 192, smem, stream>>>(map_a, st->map_b, p);
  } else {
    spconv_mm_tc_cpasync_kernel<<<grid, 288, smem, stream>>>(st->map_b, p);
  }
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
