// SPConvMM on the 5th-generation tensor cores: output-stationary implicit GEMM.
//
// For a tile of 128 consecutive output voxels and every kernel offset k that feeds at least one of them:
//   A = the 128 input rows named by the neighbour table (zero rows where the neighbour is missing), staged in shared
//       memory in the K-major swizzled layout the tensor core reads,
//   B = W[k]^T, K-major, loaded by a tiled TMA copy (once per kernel for small layers, else once per stage),
//   D += A * B with tcgen05.mma (M = 128, N = Cout, K = 16 per instruction), fp32 accumulator in tensor memory.
// All offsets of a tile accumulate into the same TMEM columns; the epilogue reads them once with tcgen05.ld, adds
// bias (+ residual), applies ReLU, converts and stores the row.  No atomics, no bias-initialisation pass.
// (The reference: gather iterator + mma.sync tiles of 64 pairs of one offset, fp16 accumulate, half2 atomicAdd
// scatter, trt/spconv/mm/kernel.h:84-179, mm/output_iterator.h:189-206.)
//
// The A rows are gathered with 16-byte cp.async (zero-fill for missing neighbours) written straight into the
// swizzled layout.  A TMA tile::gather4 producer was measured on B200 at about 11 ns per gathered row whatever the
// row width (a request-rate limit), 2-3x slower than cp.async for these row sizes, and is not used.
//
// What bounds the kernel is shared-memory bandwidth (every A block is written once and read once by the tensor
// core, 128 B/clk per SM) and, for a single issuing thread, the scalar instructions between two tcgen05.mma; the
// roles below therefore keep their inner loops to a handful of instructions per copy / per MMA:
//   8 (4) producer warps  thread t owns piece t % P of rows t / P + i * (threads / P) of every block (P = 16-byte
//                      pieces per row), so its shared-memory offsets are constants; ids come from the tile's id buffer
//   1 MMA warp         one lane issues tcgen05.mma from precomputed descriptor words; owns the TMEM allocation
//   1 control warp     prefetches the neighbour ids of the next tile (one bulk copy) and loads B by TMA
//   4 epilogue warps   TMEM -> registers -> global
// Layers of at most 64 input channels run TWO such CTAs per SM (4 producer warps and half the shared memory each):
// their bound is the serial fill -> issue -> commit chain of a tile, not a hardware unit, and two independent
// chains per SM overlap each other's hand-over time (measured: 18-24 % faster at 16 / 32 / 64 channels).
// Every role derives the stage sequence of a tile from the tile's offset mask (built with the neighbour table), so
// no per-stage metadata is exchanged.  Stages and accumulators are handed over through mbarriers; every wait is
// bounded (about one second) and on expiry raises an error word, lets the CTA drain and return instead of spinning.
#include <cuda.h>

#include "common.cuh"
#include "spconv_mm_internal.h"

namespace d3d {
namespace {

constexpr int kTileRows = 128;
constexpr int kMaxStages = 8;
constexpr int kNumAcc = 2;
constexpr int kMaxGroup = 8;  // kernel offsets that may share one pipeline stage
// Warp roles, for kProd producer threads (256: one CTA per SM; 128: two CTAs per SM, each with half the shared
// memory, which gives small layers two independent producer -> MMA -> epilogue chains per SM): producers first, then
// the MMA warp, the control warp and four epilogue warps (whose index mod 4 covers the four TMEM lane quarters).
__host__ __device__ constexpr int mma_warp_of(int prod) { return prod / 32; }
__host__ __device__ constexpr int threads_of(int prod) { return prod + 6 * 32; }
constexpr unsigned long long kWaitLimitNs = 1000ull * 1000ull * 1000ull;

__device__ int g_tc_error;  // 0 ok; otherwise the code of the first wait that gave up

struct TcParams {
  const int32_t* table;        // [tiles][kvol][128]
  const uint32_t* tile_mask;   // [tiles] bit k set: offset k feeds the tile
  const void* in_feats;        // [n_in_rows][cin]
  int64_t m_max;
  int32_t n_in_rows;  // rows of the gathered tensor (an id outside [0, n_in_rows) = zero row)
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
  int b_resident;  // all kvol weight blocks stay in smem for the whole kernel (small layers)
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
// 16-byte asynchronous copy; src_bytes = 0 writes 16 zero bytes without reading global memory.  No memory clobber:
// it touches only the operand ring, which the issuing thread never accesses with ordinary loads or stores, and the
// compiler may then overlap the id loads of the next block with these copies.
// Predicated on `run` != 0 instead of branched around.
__device__ __forceinline__ void cp_async_16_if(uint32_t run, uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.b32 q, %3, 0;\n\t"
      "@q cp.async.cg.shared.global [%0], [%1], 16, %2;\n\t}" ::"r"(dst),
      "l"(src), "r"(src_bytes), "r"(run));
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
// Programmatic dependent launch.  `pdl_release` lets the next kernel of the stream start its prologue once every CTA
// of this grid has called it (the CTAs of the next grid become resident as this grid's CTAs leave their SMs);
// `pdl_wait` blocks until the preceding grid has completed and its memory is visible.  Both are no-ops when the
// kernels were launched without the programmatic attribute.
__device__ __forceinline__ void pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit_if(uint32_t run, uint64_t* bar) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(smem_u32(bar)),
      "r"(run)
      : "memory");
}
// D (+)= A * B, issued only when `run` != 0 (predicated, not branched around).
__device__ __forceinline__ void umma_f16_if(uint32_t run, uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(run)
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

struct __align__(8) Shared {
  uint64_t full[kMaxStages];   // producers (+ the B load) -> MMA
  uint64_t empty[kMaxStages];  // MMA (tcgen05.commit) -> producers, control
  uint64_t acc_full[kNumAcc];
  uint64_t acc_empty[kNumAcc];
  uint64_t idx_full[2];  // neighbour ids of a tile have landed
  uint64_t idx_free[2];  // all producer warps are done with them
  uint64_t b_ready;      // resident weights have landed
  uint32_t tmem_base;
  int abort_flag;
};

// Carved dynamic shared memory: [stages x (group A blocks | group B blocks)] aligned to 1024, the resident weights,
// two neighbour-id buffers [kvol][128], the bias, the control block.
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

// The stage sequence of a tile is derived identically by every role from the tile's offset mask: the kernel
// offsets are cut into windows of `group` consecutive offsets; a window with at least one offset present is one
// stage per K part (kparts > 1 implies group == 1), and offset `base + e` of the window owns block slot e of the
// stage whether or not its neighbours in the window are present.  All addresses are then plain increments.

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

// Barrier initialisation, bias staging and the TMEM allocation (by the MMA warp); returns the TMEM base address.
template <int kProd>
__device__ __forceinline__ uint32_t cta_setup(const TcParams& p, const Smem& s) {
  Shared* sh = s.sh;
  if (threadIdx.x == 0) {
    // a stage is full once every producer thread's copies have landed and, when B travels with the stage, its
    // TMA bytes too (the control warp's expect_tx arrival)
    const int full_count = kProd + (p.b_resident ? 0 : 1);
    for (int i = 0; i < p.stages; ++i) mbar_init(&sh->full[i], full_count), mbar_init(&sh->empty[i], 1);
    for (int a = 0; a < kNumAcc; ++a) mbar_init(&sh->acc_full[a], 1), mbar_init(&sh->acc_empty[a], 4);
    for (int b = 0; b < 2; ++b) mbar_init(&sh->idx_full[b], 1), mbar_init(&sh->idx_free[b], kProd / 32);
    mbar_init(&sh->b_ready, 1);
    sh->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int c = threadIdx.x; c < p.cout; c += blockDim.x) s.bias[c] = p.bias[c];
  if ((int)(threadIdx.x >> 5) == mma_warp_of(kProd)) tmem_alloc(&sh->tmem_base, p.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  return sh->tmem_base;
}

// All roles meet, then the allocating warp returns the tensor memory.
template <int kProd>
__device__ __forceinline__ void cta_teardown(const TcParams& p, uint32_t tmem_base) {
  tc_fence_before();
  __syncthreads();
  if ((int)(threadIdx.x >> 5) == mma_warp_of(kProd)) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

// ---- producers ---------------------------------------------------------------------------------------------------
// kPieces = 16-byte pieces per block row (kchunk / 8).  The kProd producer threads cover a [128 x kPieces] block in
// 128 * kPieces / kProd passes; thread t copies piece t % kPieces of row t / kPieces + pass * (kProd / kPieces).  Consecutive
// lanes take consecutive pieces of a row (whole rows per warp instruction on the global side, whole 128-byte lines
// on the shared side), and because a pass advances by a multiple of 8 rows the XOR swizzle term of the destination
// is the same in every pass: one per-thread offset, the rest are immediates.
// The body of a stage is branch-free and fully unrolled over the kGroup block slots (absent offsets are predicated
// off): a taken branch costs a lone warp tens of cycles, more than the copies it would skip.
template <int kPieces, int kGroup, int kProd>
__device__ __forceinline__ void producer_role(const TcParams& p, const Smem& s, int t) {
  constexpr int kPasses = kTileRows * kPieces / kProd;
  constexpr uint32_t kBlockBytes = kTileRows * kPieces * 16;  // = p.a_bytes
  constexpr uint32_t gmask = (1u << kGroup) - 1u;
  constexpr int kRowsPerPass = kProd / kPieces;
  static_assert(kRowsPerPass % 8 == 0, "a pass must advance by whole swizzle periods");
  constexpr int kBits = kGroup * kPasses <= 8 ? 8 : 16;  // zero-row flags per stage
  constexpr int kRowBytes = kPieces >= 8 ? 128 : kPieces * 16;
  constexpr int kSwzShift = kRowBytes == 128 ? 0 : kRowBytes == 64 ? 1 : 2;
  constexpr int kSwzMask = kRowBytes == 128 ? 7 : kRowBytes == 64 ? 3 : 1;
  Shared* sh = s.sh;
  volatile int* abort_flag = &sh->abort_flag;
  const int lane = t & 31;
  const int j = t % kPieces, rsub = t / kPieces;
  const uint32_t dst_lane = (uint32_t)(j >> 3) * (kTileRows * 128) + (uint32_t)rsub * kRowBytes +
                            ((((uint32_t)j & 7u) ^ (uint32_t)((rsub >> kSwzShift) & kSwzMask)) << 4);
  const unsigned char* src_j = reinterpret_cast<const unsigned char*>(p.in_feats) + j * 16;
  const uint32_t row_src_bytes = (uint32_t)p.cin * 2;
  const uint32_t n_in_rows = (uint32_t)p.n_in_rows;
  const uint32_t tiles_addr = smem_u32(s.tiles);
  const int ids_per_tile = p.kvol * kTileRows;
  static_assert(kGroup * kPasses <= 16 && kMaxStages <= 8, "zero_rows keeps 8 or 16 bits per stage (then <= 4 stages)");
  uint64_t zero_rows = 0;  // bit kBits * stage + e * kPasses + i: this thread's last copy to that position was a zero fill
  int stage = 0;
  uint32_t phase = 0, idx_phase = 0;  // idx_phase bit b: parity to wait for on idx_full[b]
  int buf = 0;
  bool ok = true;
  pdl_wait();  // masks, ids and features may come from the preceding kernels
  uint32_t mask = (int)blockIdx.x < p.num_tiles ? __ldg(p.tile_mask + blockIdx.x) : 0u;
  for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
    const int next = tile + gridDim.x;
    const uint32_t next_mask = next < p.num_tiles ? __ldg(p.tile_mask + next) : 0u;
    ok = mbar_wait(&sh->idx_full[buf], (idx_phase >> buf) & 1u, abort_flag, 13);
    if (!ok) break;
    idx_phase ^= 1u << buf;
    const int32_t* ids = s.idx + (size_t)buf * ids_per_tile + rsub;
    for (int base = 0; base < p.kvol && ok; base += kGroup) {
      const uint32_t take = (mask >> base) & gmask;
      if (!take) continue;
      for (int part = 0; part < p.kparts; ++part) {
        ok = mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag, 12);
        if (!ok) break;
        const unsigned char* src_part = src_j + (size_t)part * p.kchunk * 2;
        const uint32_t dst = tiles_addr + (uint32_t)stage * s.stage_bytes + dst_lane;
        const int32_t* idp = ids + base * kTileRows;
        int id[kGroup][kPasses];
#pragma unroll
        for (int e = 0; e < kGroup; ++e)
#pragma unroll
          for (int i = 0; i < kPasses; ++i)
            id[e][i] = ((take >> e) & 1u) ? idp[e * kTileRows + i * kRowsPerPass] : -1;
        // Most rows of a block have no neighbour (LiDAR: about 5 of 27 offsets per voxel).  A position this thread
        // zero-filled the last time it wrote the stage is still zero (nobody else writes it), so a zero row over a
        // zero row is skipped: it would only spend shared-memory bandwidth the tensor core needs.
        const uint32_t was_zero = (uint32_t)(zero_rows >> (stage * kBits)) & ((1u << kBits) - 1u);
        uint32_t now_zero = was_zero;
#pragma unroll
        for (int e = 0; e < kGroup; ++e)
#pragma unroll
          for (int i = 0; i < kPasses; ++i) {
            constexpr uint32_t kNone = 0u;
            const uint32_t bit = 1u << (e * kPasses + i);
            const uint32_t run = (take >> e) & 1u;
            const bool valid = (uint32_t)id[e][i] < n_in_rows;  // negative = no neighbour
            const unsigned char* src = src_part + (uint64_t)(valid ? (uint32_t)id[e][i] : 0u) * row_src_bytes;
            const uint32_t redundant = (!valid && (was_zero & bit)) ? 1u : kNone;
            cp_async_16_if(run & (redundant ^ 1u), dst + (uint32_t)(e * kBlockBytes + i * kRowsPerPass * kRowBytes),
                           src, valid ? 16u : 0u);
            if (run) now_zero = valid ? (now_zero & ~bit) : (now_zero | bit);
          }
        zero_rows = (zero_rows & ~((unsigned long long)((1u << kBits) - 1u) << (stage * kBits))) |
                    ((uint64_t)now_zero << (stage * kBits));
        cp_async_arrive(&sh->full[stage]);  // one arrival per producer thread once its copies have landed
        if (++stage == p.stages) stage = 0, phase ^= 1;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&sh->idx_free[buf]);  // this warp has read all the ids it needs
    buf ^= 1;
    mask = next_mask;
  }
}

// ---- control warp (one lane) ---------------------------------------------------------------------------------------
// Keeps the two id buffers filled one tile ahead and brings in the weights: all of them once when they are
// resident, else the blocks of every stage as soon as the stage is free.
__device__ __forceinline__ void control_role(const TcParams& p, const Smem& s, const CUtensorMap* map_b) {
  Shared* sh = s.sh;
  volatile int* abort_flag = &sh->abort_flag;
  const uint32_t b_tx = (uint32_t)p.cout * p.kchunk * 2;
  const int ids_per_tile = p.kvol * kTileRows;
  const uint32_t gmask = (1u << p.group) - 1u;
  if ((int)blockIdx.x >= p.num_tiles) return;
  // the weights are constants of the layer: their load does not wait for the preceding kernel
  if (p.b_resident) {  // in the layout the per-stage loads would have produced
    mbar_arrive_expect_tx(&sh->b_ready, (uint32_t)p.kvol * b_tx);
    for (int k = 0; k < p.kvol; ++k)
      for (int c = 0; c < p.chunks; ++c)
        tma_load_2d(map_b, &sh->b_ready, s.bres + (size_t)k * p.b_bytes + (size_t)c * p.cout * p.row_bytes, c * 64,
                    k * p.cout);
  }
  pdl_wait();
  mbar_arrive_expect_tx(&sh->idx_full[0], p.idx_bytes);
  bulk_load_1d(&sh->idx_full[0], s.idx, p.table + (int64_t)blockIdx.x * ids_per_tile, p.idx_bytes);
  int stage = 0, buf = 0;
  uint32_t phase = 0, free_phase = 0;  // free_phase bit b: parity to wait for on idx_free[b]
  bool first_tile = true;
  uint32_t mask = __ldg(p.tile_mask + blockIdx.x);
  for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
    const int next = tile + gridDim.x;
    uint32_t next_mask = 0;
    if (next < p.num_tiles) {
      next_mask = __ldg(p.tile_mask + next);
      // the other buffer held the previous tile's ids: wait until every producer warp has released it
      if (!first_tile) {
        if (!mbar_wait(&sh->idx_free[buf ^ 1], (free_phase >> (buf ^ 1)) & 1u, abort_flag, 14)) return;
        free_phase ^= 1u << (buf ^ 1);
      }
      mbar_arrive_expect_tx(&sh->idx_full[buf ^ 1], p.idx_bytes);
      bulk_load_1d(&sh->idx_full[buf ^ 1], s.idx + (size_t)(buf ^ 1) * ids_per_tile,
                   p.table + (int64_t)next * ids_per_tile, p.idx_bytes);
    }
    if (!p.b_resident) {
      for (int base = 0; base < p.kvol; base += p.group) {
        const uint32_t take = (mask >> base) & gmask;
        if (!take) continue;
        for (int part = 0; part < p.kparts; ++part) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag, 11)) return;
          mbar_arrive_expect_tx(&sh->full[stage], (uint32_t)__popc(take) * b_tx);
          unsigned char* b_dst = s.tiles + (size_t)stage * s.stage_bytes + (size_t)p.group * p.a_bytes;
          for (int e = 0; e < p.group; ++e, b_dst += p.b_bytes) {
            if (!((take >> e) & 1u)) continue;
            for (int c = 0; c < p.chunks; ++c)
              tma_load_2d(map_b, &sh->full[stage], b_dst + (size_t)c * p.cout * p.row_bytes,
                          part * p.kchunk + c * 64, (base + e) * p.cout);
          }
          if (++stage == p.stages) stage = 0, phase ^= 1;
        }
      }
    }
    first_tile = false;
    buf ^= 1;
    mask = next_mask;
  }
}

// ---- MMA issuer (one lane) ---------------------------------------------------------------------------------------
// Low word of a K-major operand descriptor: start address in 16-byte units, leading byte offset 1 (unused for the
// swizzled K-major layouts).  Advancing the operand by `d` bytes adds d / 16 to this word.
__device__ __forceinline__ uint32_t desc_lo(uint32_t smem_addr) { return ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16); }

// kSteps = tcgen05.mma instructions (K = 16 each) per (offset, K part) block.
// The body of a stage is branch-free: all kGroup block slots are unrolled and absent offsets predicated off, so
// the issuing thread runs a straight line of descriptor adds and MMAs (a taken branch would cost it more than an MMA).
template <int kSteps, int kGroup>
__device__ __forceinline__ void mma_role(const TcParams& p, const Smem& s, uint32_t tmem_base) {
  constexpr uint32_t kRowBytes = kSteps >= 4 ? 128 : kSteps * 32;
  constexpr uint32_t a_step = (kTileRows * kSteps * 32) >> 4;  // = p.a_bytes / 16
  constexpr uint32_t cs_a = (kTileRows * kRowBytes) >> 4;      // between the 64-column blocks of A, 16-byte units
  constexpr uint32_t gmask = (1u << kGroup) - 1u;
  Shared* sh = s.sh;
  volatile int* abort_flag = &sh->abort_flag;
  // descriptor high word: stride between 8-row groups, version, swizzle mode
  const uint64_t desc_hi = (uint64_t)(((8u * kRowBytes) >> 4) | (1u << 14) | (p.layout_type << 29)) << 32;
  const uint32_t cs_b = (uint32_t)(p.cout * kRowBytes) >> 4;
  const uint32_t b_step = p.b_bytes >> 4, stage_step = s.stage_bytes >> 4;
  const uint32_t tiles_lo = desc_lo(smem_u32(s.tiles)), bres_lo = desc_lo(smem_u32(s.bres));
  const uint32_t b_in_stage = (uint32_t)kGroup * a_step;
  const uint32_t idesc = p.idesc;
  const bool resident = p.b_resident != 0;
  if (resident && !mbar_wait(&sh->b_ready, 0, abort_flag, 23)) return;
  int stage = 0, acc = 0;
  uint32_t phase = 0, acc_phase = 0;
  const int num_stages = p.stages, kvol = p.kvol, kparts = p.kparts;
  const uint32_t lane0 = (threadIdx.x & 31) == 0 ? 1u : 0u;  // the lane that issues; the others keep it company
  pdl_wait();
  uint32_t mask = (int)blockIdx.x < p.num_tiles ? __ldg(p.tile_mask + blockIdx.x) : 0u;
  for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
    const int next = tile + gridDim.x;
    const uint32_t next_mask = next < p.num_tiles ? __ldg(p.tile_mask + next) : 0u;
    if (mask) {  // a tile no offset feeds uses no accumulator: the epilogue writes its bias rows on its own
      if (!mbar_wait(&sh->acc_empty[acc], acc_phase ^ 1, abort_flag, 22)) return;
      tc_fence_after();
      const uint32_t d_addr = tmem_base + (uint32_t)(acc * p.cout);
      uint32_t accumulate = 0;
      int part = 0;
      for (int base = 0; base < kvol;) {
        const uint32_t take = (mask >> base) & gmask;
        if (take) {
          // the full barrier guards shared memory only: no tcgen05 fence is needed, but the rows written by
          // cp.async (generic proxy) must be made visible to the tensor core's reads (async proxy)
          if (!mbar_wait(&sh->full[stage], phase, abort_flag, 21)) return;
          fence_proxy_async();
          const uint32_t a_lo = tiles_lo + (uint32_t)stage * stage_step;
          uint32_t b_lo = resident ? bres_lo + (uint32_t)base * b_step : a_lo + b_in_stage;
#pragma unroll
          for (int e = 0; e < kGroup; ++e, b_lo += b_step) {
            const uint32_t present = (take >> e) & 1u, run = present & lane0;
#pragma unroll
            for (int ks = 0; ks < kSteps; ++ks) {
              // 32 bytes per K step inside the swizzle span, the next 64-column block every 4 steps
              const uint32_t adv_a = (uint32_t)e * a_step + (uint32_t)(ks >> 2) * cs_a + (uint32_t)(ks & 3) * 2u;
              const uint32_t adv_b = (uint32_t)(ks >> 2) * cs_b + (uint32_t)(ks & 3) * 2u;
              umma_f16_if(run, d_addr, desc_hi | (a_lo + adv_a), desc_hi | (b_lo + adv_b), idesc, accumulate);
              accumulate |= present;
            }
          }
          umma_commit_if(lane0, &sh->empty[stage]);  // the stage may be refilled once these MMAs have read it
          const bool wrap = stage + 1 == num_stages;
          stage = wrap ? 0 : stage + 1;
          phase ^= wrap ? 1u : 0u;
          ++part;
        }
        // next K part of the same window, or the next window (one loop, one back edge: branches are what costs)
        const bool window_done = !take || part == kparts;
        base += window_done ? kGroup : 0;
        part = window_done ? 0 : part;
      }
      umma_commit_if(lane0, &sh->acc_full[acc]);
      if (++acc == kNumAcc) acc = 0, acc_phase ^= 1;
    }
    mask = next_mask;
  }
}

// ---- epilogue ----------------------------------------------------------------------------------------------------
// Epilogue warp `quad` (= warp index mod 4: it may touch TMEM lanes [32*quad, 32*quad + 32)).
__device__ __forceinline__ void epilogue_role(const TcParams& p, const Smem& s, uint32_t tmem_base, int quad) {
  Shared* sh = s.sh;
  volatile int* abort_flag = &sh->abort_flag;
  const int lane = threadIdx.x & 31;
  int acc = 0;
  uint32_t acc_phase = 0;
  pdl_wait();  // residual rows come from an earlier layer; output rows may still be read by the preceding kernel
  uint32_t mask = (int)blockIdx.x < p.num_tiles ? __ldg(p.tile_mask + blockIdx.x) : 0u;
  for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
    const int next = tile + gridDim.x;
    const uint32_t next_mask = next < p.num_tiles ? __ldg(p.tile_mask + next) : 0u;
    const bool empty_tile = mask == 0;  // bias (+ residual) only, no accumulator involved
    if (!empty_tile) {
      if (!mbar_wait(&sh->acc_full[acc], acc_phase, abort_flag, 31)) return;
      tc_fence_after();
    }
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
    if (!empty_tile) {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->acc_empty[acc]);
      if (++acc == kNumAcc) acc = 0, acc_phase ^= 1;
    }
    mask = next_mask;
  }
}

// kSteps = kchunk / 16 (1, 2, 4, 8), kGroup = offsets per stage (1, 2, 4, 8), kProd = producer threads (256 or 128).
template <int kSteps, int kGroup, int kProd>
__global__ void __launch_bounds__(threads_of(kProd), kProd == 256 ? 1 : 2)
spconv_mm_tc_kernel(const __grid_constant__ CUtensorMap map_b, const TcParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const Smem s = carve_smem(smem_raw, p);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tmem_base = cta_setup<kProd>(p, s);
  pdl_release();
  if (warp < kProd / 32) {
    producer_role<2 * kSteps, kGroup, kProd>(p, s, threadIdx.x);
  } else if (warp == mma_warp_of(kProd)) {
    mma_role<kSteps, kGroup>(p, s, tmem_base);
    __syncwarp();
  } else if (warp == mma_warp_of(kProd) + 1) {
    if (lane == 0) control_role(p, s, &map_b);
    __syncwarp();
  } else {
    epilogue_role(p, s, tmem_base, warp & 3);
  }
  cta_teardown<kProd>(p, tmem_base);
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

// 2-D map over a row-major 16-bit matrix [rows][cols]; the box is box_rows x box_cols, swizzled by its width.
bool make_map(CUtensorMap* map, int dtype, const void* base, uint64_t cols, uint64_t rows, uint32_t box_cols,
              uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t elem[2] = {1, 1};
  const CUtensorMapSwizzle swz = box_cols * 2 == 32   ? CU_TENSOR_MAP_SWIZZLE_32B
                                 : box_cols * 2 == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                      : CU_TENSOR_MAP_SWIZZLE_128B;
  return fn(map, dtype == D3D_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
            const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
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

  TcParams p;
  p.table = a.table;
  p.tile_mask = reinterpret_cast<const uint32_t*>(reinterpret_cast<const unsigned char*>(a.table) +
                                                  table_ids_bytes(kvol, m_max));
  p.in_feats = a.in_feats;
  p.m_max = m_max;
  p.n_in_rows = (int32_t)a.max_num_act_in;
  p.kvol = kvol, p.cin = cin, p.cout = cout;
  p.num_tiles = (int)((m_max + kTileRows - 1) / kTileRows);
  p.row_bytes = (int)box_cols * 2;
  p.idx_bytes = (uint32_t)kvol * kTileRows * 4;
  // control data of a CTA: alignment slack, the two neighbour-id buffers, bias, barriers
  const size_t ctrl = 1024 + 2 * (size_t)p.idx_bytes + align_up((size_t)cout * 4 + 8, 16) + sizeof(Shared);
  const size_t budget_one = 227 * 1024 - ctrl;  // one CTA per SM
  // a block holds `kchunk` <= 128 input channels of one kernel offset; split further until two stages fit
  int kchunk = cin > 128 ? 128 : cin;
  while (kchunk > 64 &&
         2 * (align_up((size_t)kTileRows * kchunk * 2, 1024) + align_up((size_t)cout * kchunk * 2, 1024)) > budget_one)
    kchunk /= 2;
  int ksteps = 0;
  auto set_chunk = [&](int kc) {
    kchunk = kc, ksteps = kc / 16;
    p.kchunk = kc;
    p.kparts = cin / kc;
    p.chunks = kc <= 64 ? 1 : kc / 64;
    p.a_bytes = (uint32_t)align_up((size_t)kTileRows * kc * 2, 1024);
    p.b_bytes = (uint32_t)align_up((size_t)cout * kc * 2, 1024);
  };
  const int kchunk_one = kchunk;  // block width with one CTA per SM; two per SM use at most 64 channels per block
  set_chunk(kchunk_one);
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
  // Shared-memory plan for one CTA per SM (256 producer threads) or two (128 each, half the memory).  Small layers
  // keep all weight blocks resident instead of reloading one per stage; several offsets share a stage when their
  // blocks are small, so that the per-stage hand-over cost is amortised (a stage holds at most 8 K-step blocks).
  struct Plan {
    int resident, group, stages;
    size_t smem;
  };
  auto make_plan = [&](bool two_per_sm, Plan* out) -> bool {
    if (two_per_sm && (kchunk > 64 || ctrl + 2048 > 113 * 1024)) return false;
    const size_t bres_bytes = (size_t)kvol * p.b_bytes;
    const size_t budget = (two_per_sm ? 113 * 1024 : 227 * 1024) - ctrl;
    const size_t resident_limit = two_per_sm ? 32 * 1024 : 64 * 1024;
    Plan pl;
    pl.resident = (p.kparts == 1 && bres_bytes <= resident_limit) ? 1 : 0;
    if (pl.resident && bres_bytes + 2 * (size_t)p.a_bytes > budget) pl.resident = 0;
    const size_t ring = budget - (pl.resident ? bres_bytes : 0);
    const size_t blk = (size_t)p.a_bytes + (pl.resident ? 0 : p.b_bytes);
    const size_t stage_target = two_per_sm ? ring / 2 : 48 * 1024;
    pl.group = 1;
    if (p.kparts == 1)
      while (pl.group < kMaxGroup && (size_t)(2 * pl.group) * blk <= stage_target && 2 * pl.group * ksteps <= 8)
        pl.group *= 2;
    const size_t stage_bytes = (size_t)pl.group * blk;
    pl.stages = (int)(ring / stage_bytes);
    // the producers keep per-stage zero-row flags in one 64-bit word: 8 bits per stage, 16 when a thread owns more
    const int flag_bits = pl.group * ksteps * (two_per_sm ? 2 : 1) <= 8 ? 8 : 16;
    const int max_stages = 64 / flag_bits < kMaxStages ? 64 / flag_bits : kMaxStages;
    pl.stages = pl.stages > max_stages ? max_stages : pl.stages;
    if (pl.stages < 2) return false;
    pl.smem = ctrl + (size_t)pl.stages * stage_bytes + (pl.resident ? bres_bytes : 0);
    // pin the number of CTAs per SM through the request: more than half (a third) of the SM's shared memory
    const size_t floor_bytes = two_per_sm ? 80 * 1024 : 120 * 1024;
    if (pl.smem < floor_bytes) pl.smem = floor_bytes;
    *out = pl;
    return true;
  };
  Plan pl;
  bool two_per_sm = false;
  // 128 input channels: two CTAs per SM (K split in two) measure about even with one; they win for few tiles per
  // SM, where twice as many CTAs quantise the tile count better
  if (h->kernel_choice != 3 && (cin < 128 || (cin == 128 && p.num_tiles <= 8 * kNumSMs))) {
    set_chunk(kchunk_one < 64 ? kchunk_one : 64);
    two_per_sm = make_plan(true, &pl);
  }
  if (!two_per_sm) {
    set_chunk(kchunk_one);
    D3D_REQUIRE(make_plan(false, &pl), D3D_ERR_TOO_LARGE);
  }
  p.b_resident = pl.resident, p.group = pl.group, p.stages = pl.stages;
  const size_t smem = pl.smem;
  // one kernel instance per (MMAs per block, offsets per stage, producer threads)
  typedef void (*KernelFn)(const CUtensorMap, const TcParams);
  static const KernelFn kernels[2][4][4] = {
      {{spconv_mm_tc_kernel<1, 1, 256>, spconv_mm_tc_kernel<1, 2, 256>, spconv_mm_tc_kernel<1, 4, 256>,
        spconv_mm_tc_kernel<1, 8, 256>},
       {spconv_mm_tc_kernel<2, 1, 256>, spconv_mm_tc_kernel<2, 2, 256>, spconv_mm_tc_kernel<2, 4, 256>, nullptr},
       {spconv_mm_tc_kernel<4, 1, 256>, spconv_mm_tc_kernel<4, 2, 256>, nullptr, nullptr},
       {spconv_mm_tc_kernel<8, 1, 256>, nullptr, nullptr, nullptr}},
      {{spconv_mm_tc_kernel<1, 1, 128>, spconv_mm_tc_kernel<1, 2, 128>, spconv_mm_tc_kernel<1, 4, 128>,
        spconv_mm_tc_kernel<1, 8, 128>},
       {spconv_mm_tc_kernel<2, 1, 128>, spconv_mm_tc_kernel<2, 2, 128>, spconv_mm_tc_kernel<2, 4, 128>, nullptr},
       {spconv_mm_tc_kernel<4, 1, 128>, spconv_mm_tc_kernel<4, 2, 128>, nullptr, nullptr},
       {nullptr, nullptr, nullptr, nullptr}}};
  const int si = kchunk == 16 ? 0 : kchunk == 32 ? 1 : kchunk == 64 ? 2 : 3;
  const int gi = pl.group == 1 ? 0 : pl.group == 2 ? 1 : pl.group == 4 ? 2 : 3;
  const int di = two_per_sm ? 1 : 0;
  D3D_REQUIRE(kernels[di][si][gi] != nullptr, D3D_ERR_TOO_LARGE);
  static bool attr_set[64][2][4][4] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return D3D_ERR_CUDA;
  if (!attr_set[dev][di][si][gi]) {
    if (cudaFuncSetAttribute(kernels[di][si][gi], cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) !=
        cudaSuccess)
      return D3D_ERR_CUDA;
    attr_set[dev][di][si][gi] = true;
  }
  const int ctas = kNumSMs * (two_per_sm ? 2 : 1);
  const int grid = p.num_tiles < ctas ? p.num_tiles : ctas;
  // programmatic dependent launch (opt-in per handle): the prologue of this kernel (barriers, tensor memory,
  // weights) may overlap the tail of the preceding kernel of the stream; every role waits for that kernel before
  // it touches its data.  Measured on B200: 3-4 us less per launch for layers run back to back on one stream; a
  // loss where other streams have kernels that would otherwise fill the tail of the preceding kernel.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(threads_of(two_per_sm ? 128 : 256));
  cfg.dynamicSmemBytes = smem, cfg.stream = reinterpret_cast<cudaStream_t>(a.stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = h->dependent_launch ? 1 : 0;
  if (cudaLaunchKernelEx(&cfg, kernels[di][si][gi], st->map_b, p) != cudaSuccess) return D3D_ERR_CUDA;
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
