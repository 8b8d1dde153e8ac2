// SPConvMM on the 5th-generation tensor cores: output-stationary implicit GEMM.
//
// For a tile of 128 consecutive output voxels and every kernel offset k that feeds at least one of them:
//   A = the input rows named by the neighbour table, staged in shared memory in the K-major swizzled layout the
//       tensor core reads -- only the rows that exist: the table carries a 128-bit row mask per (tile, offset),
//   B = W[k]^T, K-major, loaded by a tiled TMA copy (once per kernel when all offsets fit, else once per stage),
//   D += A * B with tcgen05.mma (M = 128, N = Cout, K = 16 per instruction), fp32 accumulator in tensor memory,
//       issued with the inverted row mask as disable_output_lane: accumulator lanes of rows without an input are
//       not updated, so whatever an unused row of the operand ring holds is never seen (no zero fill).
// All offsets of a tile accumulate into the same TMEM columns; the epilogue reads them once with tcgen05.ld, adds
// bias (+ residual), applies ReLU, converts and stores the row, and writes zeros back (tcgen05.st) for the next tile.
// No atomics, no bias-initialisation pass.
// (The reference: gather iterator + mma.sync tiles of 64 pairs of one offset, fp16 accumulate, half2 atomicAdd
// scatter, trt/spconv/mm/kernel.h:84-179, mm/output_iterator.h:189-206.)
//
// The A rows are gathered with 16-byte cp.async written straight into the swizzled layout.  A TMA tile::gather4
// producer was measured on B200 at 11.4 ns per gathered row whatever the row width (a request-rate limit), three
// times slower than cp.async for these row sizes (microbench/gather_rows.cu measures both), and is not used.
//
// What bounds this kernel, measured on B200 (tuning builds with D3D_TC_PROFILE / D3D_TC_NO_MMA / D3D_TC_NO_COPY below,
// microbench/mma_issue.cu):
//   * the instruction streams of its roles.  With every MMA and every gather copy predicated off the layers still
//     take 52-80 % of their time.  One warp that waits for a stage, fences and issues eight M128 K16 MMAs needs about
//     750 cycles for what the tensor core executes in 320 to 512; two such warps on one SM keep it busy.  A lone
//     warp issues a dependent instruction every four cycles or so, so what a role executes per stage besides its
//     copies / MMAs (walking the stage sequence, waits, address arithmetic) costs as much as the work itself.
//   * for layers of 64 channels and more, weight traffic from L2 (W[k] is fetched again for every tile: as many
//     bytes as the gathered rows) and the shared-memory data pipe (128 B per clock and SM): every A row is written
//     once by cp.async and the whole block read once by the tensor core, every B block likewise.
// Hence:
//   * layers run TWO CTAs per SM wherever shared and tensor memory allow (two independent issue streams);
//   * the MMA warp keeps every value that feeds an MMA warp-uniform in a way the compiler can see (offset masks
//     pass through a shuffle from lane 0), computes all descriptors of a stage first and lets the lane chosen by
//     elect.sync issue the MMAs as straight-line code; it probes the following stage's barrier before it issues;
//     the row masks of a tile are loaded a tile ahead and parked, inverted, in shared memory;
//   * the neighbour ids and row-mask words are read from global memory by the producer lanes themselves, a stage
//     ahead (and the table lines of the next tile are prefetched into L2), not staged in shared memory;
//   * the producer warps work in teams of four that take the stages in turn, so that the per-stage overhead of a
//     warp is paid once per two stages of the pipeline; address arithmetic of all copies of a stage comes first,
//     the copies follow as independent instruction groups, predicated by the row-mask bit of their row;
//   * every role loads the offset mask of its next tile while it works on the current one;
//   * the epilogue handles 16 columns per tensor-memory load (two CTAs of 320 or 448 threads per SM fit).
// Roles of a CTA, for W = 4 or 8 producer warps:
//   W producer warps   teams of four; warp q of a team copies rows [32q, 32q + 32) of every A block of the team's
//                      stages: lane = (row, 16-byte piece), so its shared-memory offsets are constants
//   1 MMA warp         waits for a stage, one elected lane issues its tcgen05.mma and commits; owns the TMEM allocation
//   1 control warp     one lane loads B by TMA (all offsets once when they fit, else per stage)
//   4 epilogue warps   TMEM -> registers -> global, then zeros -> TMEM
// A tile row need not stand for output tile * 128 + row: the table carries the output row of every tile row, and a
// table rebuilt by d3d_spconv_mm_regroup lists its outputs sorted by offset mask, so that a tile keeps only the few
// offsets its like outputs share.  For such tables the kernel is instantiated with a second stage walk (kPacked: a
// stage takes the next offsets that are present instead of a fixed window of offsets) and a tile order that hands
// every CTA a like share of the costly tiles.
// Every role derives the stage sequence of a tile from the tile's offset mask (built with the neighbour table), so
// no per-stage metadata is exchanged.  Stages and accumulators are handed over through mbarriers; every wait is
// bounded (about one second) and on expiry raises an error word, lets the CTA drain and return instead of spinning.
#include <cuda.h>

#include <mutex>
#include <new>

#include "common.cuh"
#include "spconv_mm_internal.h"

namespace d3d {
namespace {

constexpr int kTileRows = 128;
constexpr int kMaxStages = 8;
constexpr int kNumAcc = 2;
constexpr int kMaxGroup = 8;  // kernel offsets that may share one pipeline stage
// Warp roles for W producer warps: producers first, then the MMA warp, the control warp and four epilogue warps
// (whose index mod 4 covers the four TMEM lane quarters).
__host__ __device__ constexpr int threads_of(int prod_warps) { return (prod_warps + 6) * 32; }
constexpr unsigned long long kWaitLimitNs = 1000ull * 1000ull * 1000ull;

__device__ int g_tc_error;  // 0 ok; otherwise the code of the first wait that gave up

// Tuning builds (python -m deploy3d_b200.build --tuning NAME -D...):
//   D3D_TC_PROFILE  cycle accounting per role (CTA 0 only), read back with d3d_debug_copy_prof
//   D3D_TC_NO_MMA   every tcgen05.mma predicated off     } timing experiments: what is left when a part of the
//   D3D_TC_NO_COPY  every gather copy predicated off     } work is removed (the results are meaningless)
#ifdef D3D_TC_NO_MMA
#define D3D_TC_MMA_RUN(run) ((run) & 0u)
#else
#define D3D_TC_MMA_RUN(run) (run)
#endif
#ifdef D3D_TC_NO_COPY
#define D3D_TC_COPY_RUN(run) ((run) & 0u)
#else
#define D3D_TC_COPY_RUN(run) (run)
#endif
#ifdef D3D_TC_PROFILE
__device__ long long g_prof[3][8];
#define PROF_DECL long long prof_[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long tprev_ = clock64();
#define PROF(x) do { long long n_ = clock64(); prof_[x] += n_ - tprev_; tprev_ = n_; } while (0)
#define PROF_STORE(role, cond) if (blockIdx.x == 0 && (cond)) for (int i_ = 0; i_ < 8; ++i_) g_prof[role][i_] = prof_[i_];
#else
#define PROF_DECL
#define PROF(x)
#define PROF_STORE(role, cond)
#endif

struct TcParams {
  const int32_t* table;        // [tiles][kvol][128]
  const uint32_t* tile_mask;   // [tiles] bit k set: offset k feeds the tile
  const uint32_t* row_masks;   // [tiles][kvol][4] bit r of word q set: row 32 q + r has an input under the offset
  const int32_t* perm;         // [tiles][128] output row of every tile row, -1 = none
  const void* in_feats;        // [n_in_rows][cin]
  int64_t m_max;
  int32_t n_in_rows;  // rows of the gathered tensor (an id outside [0, n_in_rows) = zero row)
  int kvol, cin, cout;
  int num_tiles;
  int stages;
  uint32_t a_bytes, b_bytes;  // per (offset, K part) block
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
// Non-blocking test of a barrier phase.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
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
// One lane waits, the warp learns the outcome.  __syncwarp orders the other lanes' later accesses after the
// observation of lane 0.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort_flag, code) ? 1 : 0;
  __syncwarp();
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

__device__ __forceinline__ void tma_load_2d(const CUtensorMap* map, uint64_t* bar, void* dst, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// 16-byte asynchronous copy, predicated on `run` != 0 instead of branched around.  No memory clobber: it touches
// only the operand ring, which the issuing thread never accesses with ordinary loads or stores, and the compiler may
// then overlap the id loads of the next stage with these copies.
__device__ __forceinline__ void cp_async_16_if(uint32_t run, uint32_t dst, const void* src) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.b32 q, %2, 0;\n\t"
      "@q cp.async.cg.shared.global [%0], [%1], 16;\n\t}" ::"r"(dst),
      "l"(src), "r"(D3D_TC_COPY_RUN(run)));
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
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t.reg .b32 r;\n\t"
      "elect.sync r|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// D += A * B on the accumulator lanes whose bit in `off` (lanes 0-31 in .x, ... 96-127 in .w) is clear; the other
// lanes keep their value whatever the corresponding rows of A hold.  Issued only when `run` != 0 (predicated, not
// branched around).
__device__ __forceinline__ void umma_f16_rows_if(uint32_t run, uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                                 uint32_t idesc, const uint4& off) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.eq.b32 p, 0, 0;\n\t"
      "setp.ne.b32 q, %4, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(D3D_TC_MMA_RUN(run)), "r"(off.x), "r"(off.y), "r"(off.z), "r"(off.w)
      : "memory");
}
// Writes `v` into 16 consecutive columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_st16_same(uint32_t taddr, uint32_t v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};"
      ::"r"(taddr), "r"(v) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

struct __align__(16) Shared {
  uint64_t full[kMaxStages];   // producers (+ the B load) -> MMA
  uint64_t empty[kMaxStages];  // MMA (tcgen05.commit) -> producers, control
  uint64_t acc_full[kNumAcc];
  uint64_t acc_empty[kNumAcc];
  uint64_t b_ready;  // resident weights have landed
  uint32_t tmem_base;
  int abort_flag;
  // row masks of the MMA warp's current and next tile, inverted (bit set = accumulator lane left alone), four words
  // per kernel offset; sized so that a whole window of kMaxGroup offsets starting below 32 stays inside
  __align__(16) uint32_t lanes_off[2][(32 + kMaxGroup) * 4];
};

// Carved dynamic shared memory: [stages x (group A blocks | group B blocks)] aligned to 1024, the resident weights,
// the bias, the control block.
struct Smem {
  unsigned char* tiles;
  unsigned char* bres;  // resident weights [kvol][b_bytes] (when p.b_resident)
  float* bias;
  Shared* sh;
  uint32_t stage_bytes;
};
template <int kGroup> __device__ __forceinline__ Smem carve_smem(unsigned char* raw, const TcParams& p) {
  Smem s;
  const uint32_t raw_addr = smem_u32(raw);
  s.tiles = raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  s.stage_bytes = (uint32_t)kGroup * (p.a_bytes + (p.b_resident ? 0u : p.b_bytes));
  s.bres = s.tiles + (size_t)p.stages * s.stage_bytes;
  s.bias = reinterpret_cast<float*>(s.bres + (p.b_resident ? (size_t)p.kvol * p.b_bytes : 0));
  s.sh = reinterpret_cast<Shared*>(s.bias + ((p.cout + 3) & ~3));
  return s;
}

// The stage sequence of a tile is derived identically by every role from the tile's offset mask, in ascending order of
// the offsets, one stage per K part (see stage_bits for the two ways a stage picks its offsets).
struct StageIter {
  int tile;
  int round;           // how many tiles of this CTA came before `tile`
  uint32_t rest;       // offsets of `tile` not yet handed out, including those of the current stage
  uint32_t mask_next;  // of the CTA's next tile, loaded while this one is walked (a load per tile is a round trip to L2)
  uint32_t bits;       // the offsets of the current stage: packed stages, absolute; windows, relative to `base`
  int base;            // windows only: first offset of the stage's window
  int part;
};
__device__ __forceinline__ uint32_t load_mask(const TcParams& p, int tile) {
  return tile < p.num_tiles ? __ldg(p.tile_mask + tile) : 0u;
}
// The CTA's tile of round r, or num_tiles when it has none.  A regrouped table holds its tiles in ascending order of
// their offset masks, the costly ones last: there the CTAs take the tiles round by round from the last tile down, in
// alternating direction, so that every CTA starts with a costly tile and the rounds pair a CTA's costlier tiles with
// cheaper ones.
template <bool kPacked> __device__ __forceinline__ int tile_at(const TcParams& p, int round) {
  const int g = (int)gridDim.x, c = (int)blockIdx.x;
  if (!kPacked) {  // plain tables: every tile costs about the same, the CTAs sweep them front to back
    const int idx = round * g + c;
    return idx < p.num_tiles ? idx : p.num_tiles;
  }
  const int idx = round * g + ((round & 1) ? g - 1 - c : c);
  return idx < p.num_tiles ? p.num_tiles - 1 - idx : p.num_tiles;
}
// Two ways a stage picks its offsets.  kPacked: the kGroup lowest offsets still present (tables whose outputs were
// regrouped have few offsets per tile, anywhere among the kVol).  Otherwise: the present offsets of the next window
// of kGroup consecutive offsets that has any -- a plain table has nearly all offsets in every tile, and with fixed
// windows the offset of slot e is window + e, so every address is the window's plus a constant.
template <int kGroup> __device__ __forceinline__ uint32_t lowest_bits(uint32_t m) {
  uint32_t r = m;
#pragma unroll
  for (int e = 0; e < kGroup; ++e) r &= r - 1u;
  return m & ~r;
}
// Offset of every slot of a stage (always a valid index) and, as bit e of the result, whether slot e is in use.
template <int kGroup, bool kPacked>
__device__ __forceinline__ uint32_t slot_offsets(uint32_t bits, int base, int (&k)[kGroup]) {
  if (kPacked) {
    const uint32_t used = (1u << __popc(bits)) - 1u;
#pragma unroll
    for (int e = 0; e < kGroup; ++e) {
      k[e] = bits ? __ffs(bits) - 1 : 0;
      bits &= bits - 1u;
    }
    return used;
  }
#pragma unroll
  for (int e = 0; e < kGroup; ++e) k[e] = base + e;
  return bits;
}
template <int kGroup, bool kPacked> __device__ __forceinline__ void first_tile(const TcParams& p, StageIter& it) {
  it.round = 0;
  it.tile = tile_at<kPacked>(p, 0);
  it.rest = load_mask(p, it.tile);
  it.mask_next = load_mask(p, tile_at<kPacked>(p, 1));
  it.bits = 0;
  it.base = -kGroup;
  it.part = p.kparts - 1;
}
// Moves to the next stage of this CTA's tiles; false when there is none.
template <int kGroup, bool kPacked> __device__ __forceinline__ bool next_stage(const TcParams& p, StageIter& it) {
  constexpr uint32_t gmask = (1u << kGroup) - 1u;
  if (++it.part < p.kparts) return true;
  it.part = 0;
  if (kPacked) it.rest &= ~it.bits;
  else it.base += kGroup;
  for (;;) {
    if (it.tile >= p.num_tiles) return false;
    if (kPacked) {
      if (it.rest) {
        it.bits = lowest_bits<kGroup>(it.rest);
        return true;
      }
    } else {
      while (it.base < p.kvol) {
        const uint32_t take = (it.rest >> it.base) & gmask;
        if (take) {
          it.bits = take;
          return true;
        }
        it.base += kGroup;
      }
      it.base = 0;
    }
    if (kPacked) {
      it.tile = tile_at<true>(p, ++it.round);
      it.rest = it.mask_next;
      it.mask_next = load_mask(p, tile_at<true>(p, it.round + 1));
    } else {  // front to back: the next tile is gridDim.x further
      it.tile += gridDim.x;
      it.rest = it.mask_next;
      it.mask_next = load_mask(p, it.tile + (int)gridDim.x);
    }
  }
}

// 16 accumulator columns starting at col0 of this thread's row: bias (+ residual), ReLU, convert, two 16-byte stores.
template <bool kBf16>
__device__ __forceinline__ void store_chunk(const uint32_t* acc, const float* bias_s, int col0, void* out_row,
                                            const void* res_row, int relu) {
  float v[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(acc[j]) + bias_s[col0 + j];
  if (relu == 2) {  // activation before the residual is added (sum of two activated branches)
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = fmaxf(v[j], 0.f);
  }
  if (res_row) {
    const uint4* r4 = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(res_row) + col0);
#pragma unroll
    for (int q = 0; q < 2; ++q) {
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
  uint4* o4 = reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(out_row) + col0);
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float a = v[q * 8 + 2 * e], b = v[q * 8 + 2 * e + 1];
      if (relu == 1) a = fmaxf(a, 0.f), b = fmaxf(b, 0.f);
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

// Barrier initialisation, bias staging and the TMEM allocation (by the MMA warp); returns the TMEM base address.
template <int kProdWarps>
__device__ __forceinline__ uint32_t cta_setup(const TcParams& p, const Smem& s) {
  Shared* sh = s.sh;
  if (threadIdx.x == 0) {
    // a stage is full once every producer thread's copies have landed and, when B travels with the stage, its
    // TMA bytes too (the control warp's expect_tx arrival)
    const int full_count = kTileRows + (p.b_resident ? 0 : 1);  // the four warps of one producer team
    for (int i = 0; i < p.stages; ++i) mbar_init(&sh->full[i], full_count), mbar_init(&sh->empty[i], 1);
    for (int a = 0; a < kNumAcc; ++a) mbar_init(&sh->acc_full[a], 1), mbar_init(&sh->acc_empty[a], 4);
    mbar_init(&sh->b_ready, 1);
    sh->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int c = threadIdx.x; c < p.cout; c += blockDim.x) s.bias[c] = p.bias[c];
  if ((int)(threadIdx.x >> 5) == kProdWarps) tmem_alloc(&sh->tmem_base, p.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  return sh->tmem_base;
}

// All roles meet, then the allocating warp returns the tensor memory.
template <int kProdWarps>
__device__ __forceinline__ void cta_teardown(const TcParams& p, uint32_t tmem_base) {
  tc_fence_before();
  __syncthreads();
  if ((int)(threadIdx.x >> 5) == kProdWarps) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

// ---- producers ---------------------------------------------------------------------------------------------------
// kPieces = 16-byte pieces per row of a 64-column block (2, 4 or 8), kChunks = 64-column blocks per A block.
// The producer warps form teams of four; a team fills a whole stage (warp q of the team copies rows [32q, 32q + 32)
// of every block) and the teams take the stages in turn.  What a warp spends per stage besides the copies -- walking
// the stage sequence, loading ids, waiting for the slot -- is then paid once per kTeams stages of the pipeline.
// A warp instruction covers 32 / kPieces whole rows (lane = row * kPieces + piece: whole rows on the global side,
// whole swizzle spans on the shared side); because a pass advances by a multiple of 4 rows and the warp's first row by
// a multiple of 32, the XOR swizzle term of the destination is a per-lane constant (128-byte rows: two constants,
// by pass parity).  Only rows that have an input are copied: the row mask of the (tile, offset, quarter) -- one word,
// the same for the whole warp -- predicates the copies, and the MMA warp keeps the other accumulator lanes out of the
// product, so whatever an unused row of the ring holds is never seen.  Ids and row masks come straight from global
// memory; the loads of the team's next stage are issued before the copies of this one.
template <int kPieces, int kChunks, int kGroup, int kProdWarps, bool kPacked>
__device__ __forceinline__ void producer_role(const TcParams& p, const Smem& s, int warp, int lane) {
  constexpr int kTeams = kProdWarps / 4;
  constexpr int kRows = 32;                   // rows of a block per warp
  constexpr int kRowsPerPass = 32 / kPieces;  // 16, 8 or 4
  constexpr int kPasses = kRows / kRowsPerPass;
  constexpr int kRowBytes = kPieces * 16;
  constexpr uint32_t kChunkBytes = kTileRows * kRowBytes;      // one 64-column block
  constexpr uint32_t kBlockBytes = kChunkBytes * kChunks;      // = p.a_bytes
  constexpr int kSwzShift = kRowBytes == 128 ? 0 : kRowBytes == 64 ? 1 : 2;
  constexpr int kSwzMask = kRowBytes == 128 ? 7 : kRowBytes == 64 ? 3 : 1;
  Shared* sh = s.sh;
  volatile int* abort_flag = &sh->abort_flag;
  const int team = warp / 4, quarter = warp % 4;
  const int j = lane % kPieces, rsub = lane / kPieces;
  const int row0 = kRows * quarter + rsub;  // the row this lane copies in pass 0
  const uint32_t dst_lane =
      (uint32_t)row0 * kRowBytes + ((uint32_t)(j ^ ((row0 >> kSwzShift) & kSwzMask)) << 4);
  const unsigned char* src_j = reinterpret_cast<const unsigned char*>(p.in_feats) + j * 16;
  const uint32_t row_src_bytes = (uint32_t)p.cin * 2;
  const uint32_t last_in_row = (uint32_t)p.n_in_rows - 1u;
  const uint32_t tiles_addr = smem_u32(s.tiles);

  struct Ids {
    int id[kGroup][kPasses];
    uint32_t rows[kGroup];  // row mask word of this warp's quarter, 0 for an offset the stage does not take
  };
  auto load_ids = [&](const StageIter& it, Ids& v) {
    const int64_t blk0 = (int64_t)it.tile * p.kvol;
    if (kPacked) {
      int k[kGroup];
      const uint32_t used = slot_offsets<kGroup, true>(it.bits, 0, k);
#pragma unroll
      for (int e = 0; e < kGroup; ++e) {
        const bool take = (used >> e) & 1u;
        const int32_t* base = p.table + (blk0 + k[e]) * kTileRows + row0;
        v.rows[e] = take ? __ldg(p.row_masks + (blk0 + k[e]) * 4 + quarter) : 0u;
#pragma unroll
        for (int i = 0; i < kPasses; ++i) v.id[e][i] = take ? __ldg(base + i * kRowsPerPass) : -1;
      }
    } else {  // the window's blocks follow each other in the table: constant offsets from its first block
      const int32_t* base = p.table + (blk0 + it.base) * kTileRows + row0;
      const uint32_t* rows = p.row_masks + (blk0 + it.base) * 4 + quarter;
#pragma unroll
      for (int e = 0; e < kGroup; ++e) {
        const bool take = (it.bits >> e) & 1u;
        v.rows[e] = take ? __ldg(rows + e * 4) : 0u;
#pragma unroll
        for (int i = 0; i < kPasses; ++i) v.id[e][i] = take ? __ldg(base + e * kTileRows + i * kRowsPerPass) : -1;
      }
    }
  };
  // the neighbour ids of a tile are kvol * 512 contiguous bytes: one 128-byte line per lane of a team
  auto prefetch_ids = [&](int tile) {
    const int line = quarter * 32 + lane;
    if (tile < p.num_tiles && line < p.kvol * 4) {
      const int32_t* a = p.table + (int64_t)tile * p.kvol * kTileRows + line * 32;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
    }
  };
  // the team's next stage: kTeams stages further in the sequence
  auto next_own = [&](StageIter& it) -> bool {
#pragma unroll
    for (int t = 0; t < kTeams; ++t)
      if (!next_stage<kGroup, kPacked>(p, it)) return false;
    return true;
  };
  pdl_wait();  // masks, ids and features may come from the preceding kernels
  prefetch_ids(tile_at<kPacked>(p, 1));
  int stage = team;  // slot of the team's current stage (at least two stages exist)
  uint32_t phase = 0;
  PROF_DECL
  // One stage: find the team's stage after `cur` and start the loads of its ids, then wait for the slot and copy
  // `cur`.  Returns false when `cur` was the team's last stage or a wait gave up.
  auto step = [&](const StageIter& cur, const Ids& ids, StageIter& nxt, Ids& ids_next) -> bool {
    PROF(0);
    nxt = cur;
    const bool have_next = next_own(nxt);
    if (have_next) load_ids(nxt, ids_next);
    // on entering a tile, pull the ids of the CTA's next tile towards the SM: they may come from DRAM, which takes
    // longer than the one stage the loads above run ahead
    if (have_next && nxt.tile != cur.tile)
      prefetch_ids(kPacked ? tile_at<true>(p, nxt.round + 1) : nxt.tile + (int)gridDim.x);
    PROF(1);
    if (!mbar_wait_warp(&sh->empty[stage], phase ^ 1, abort_flag, 12)) return false;
    PROF(2);
    const unsigned char* src_part = src_j + (size_t)cur.part * p.kchunk * 2;
    const uint32_t dst = tiles_addr + (uint32_t)stage * s.stage_bytes + dst_lane;
    // A lone warp issues a dependent instruction every four cycles or so, and the copies (volatile asm) keep their
    // order: so the source addresses of all copies of the stage come first -- independent chains the scheduler can
    // interleave -- and the copies themselves follow as short, independent instruction groups.  An id without an
    // input (-1) or beyond the tensor is clamped to the last row: its address stays inside the tensor whether or
    // not the copy is predicated off.
    const unsigned char* src[kGroup][kPasses];
#pragma unroll
    for (int e = 0; e < kGroup; ++e)
#pragma unroll
      for (int i = 0; i < kPasses; ++i)
      {
#ifdef DEPLOY3D_BOUNDS_CHECK  // ids of rows that have an input (the others are unspecified) are recorded when off
        if ((ids.rows[e] >> (rsub + i * kRowsPerPass)) & 1u)
          (void)D3D_BOUNDS_OK(ids.id[e][i], 0, (long long)last_in_row + 1, kSiteMmTcId);
#endif
        src[e][i] = src_part + (uint64_t)min((uint32_t)ids.id[e][i], last_in_row) * row_src_bytes;
      }
#pragma unroll
    for (int e = 0; e < kGroup; ++e) {
      const uint32_t mine = ids.rows[e] >> rsub;  // bit i * kRowsPerPass: this lane's row of pass i
#pragma unroll
      for (int i = 0; i < kPasses; ++i) {
        const uint32_t d = (kRowBytes == 128 ? (dst ^ (uint32_t)((i & 1) << 6)) : dst) +
                           (uint32_t)(e * kBlockBytes + i * kRowsPerPass * kRowBytes);
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
          cp_async_16_if(mine & (1u << (i * kRowsPerPass)), d + c * kChunkBytes, src[e][i] + c * 128);
      }
    }
    cp_async_arrive(&sh->full[stage]);  // one arrival per producer thread once its copies have landed
    PROF(3);
#pragma unroll
    for (int t = 0; t < kTeams; ++t)
      if (++stage == p.stages) stage = 0, phase ^= 1;
    return have_next;
  };
  // two id buffers used in turn: the loaded ids are first touched a whole stage after their loads were issued
  StageIter it_a, it_b;
  Ids ids_a, ids_b;
  first_tile<kGroup, kPacked>(p, it_a);
  bool have = true;
  for (int t = 0; t <= team && have; ++t) have = next_stage<kGroup, kPacked>(p, it_a);
  if (have) {
    load_ids(it_a, ids_a);
    while (step(it_a, ids_a, it_b, ids_b) && step(it_b, ids_b, it_a, ids_a)) {
    }
  }
  PROF_STORE(0, warp == 0 && lane == 0)
}

// ---- control warp (one lane) ---------------------------------------------------------------------------------------
// Brings in the weights: all of them once when they are resident, else the blocks of every stage as soon as the
// stage is free.
template <int kGroup, bool kPacked>
__device__ __forceinline__ void control_role(const TcParams& p, const Smem& s, const CUtensorMap* map_b) {
  Shared* sh = s.sh;
  volatile int* abort_flag = &sh->abort_flag;
  const uint32_t b_tx = (uint32_t)p.cout * p.kchunk * 2;
  if ((int)blockIdx.x >= p.num_tiles) return;
  // the weights are constants of the layer: their load does not wait for the preceding kernel
  if (p.b_resident) {  // in the layout the per-stage loads would have produced
    mbar_arrive_expect_tx(&sh->b_ready, (uint32_t)p.kvol * b_tx);
    for (int k = 0; k < p.kvol; ++k)
      for (int c = 0; c < p.chunks; ++c)
        tma_load_2d(map_b, &sh->b_ready, s.bres + (size_t)k * p.b_bytes + (size_t)c * p.cout * p.row_bytes, c * 64,
                    k * p.cout);
    return;
  }
  pdl_wait();  // the offset masks come from the preceding kernels
  StageIter it;
  first_tile<kGroup, kPacked>(p, it);
  int stage = 0;
  uint32_t phase = 0;
  while (next_stage<kGroup, kPacked>(p, it)) {
    if (!mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag, 11)) return;
    mbar_arrive_expect_tx(&sh->full[stage], (uint32_t)__popc(it.bits) * b_tx);
    unsigned char* b_dst = s.tiles + (size_t)stage * s.stage_bytes + (size_t)kGroup * p.a_bytes;
    int k[kGroup];
    const uint32_t used = slot_offsets<kGroup, kPacked>(it.bits, it.base, k);
#pragma unroll
    for (int e = 0; e < kGroup; ++e, b_dst += p.b_bytes) {
      if (!((used >> e) & 1u)) continue;
      for (int c = 0; c < p.chunks; ++c)
        tma_load_2d(map_b, &sh->full[stage], b_dst + (size_t)c * p.cout * p.row_bytes,
                    it.part * p.kchunk + c * 64, k[e] * p.cout);
    }
    if (++stage == p.stages) stage = 0, phase ^= 1;
  }
}

// ---- MMA warp ----------------------------------------------------------------------------------------------------
// Low word of a K-major operand descriptor: start address in 16-byte units, leading byte offset 1 (unused for the
// swizzled K-major layouts).  Advancing the operand by `d` bytes adds d / 16 to this word.
__device__ __forceinline__ uint32_t desc_lo(uint32_t smem_addr) { return ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16); }

// The whole warp walks the stage sequence; everything an MMA depends on (offset mask, stage slot) is kept
// warp-uniform in a form the compiler can see -- the mask goes through a shuffle from lane 0 -- so that descriptor
// arithmetic stays in the uniform datapath; one elected lane issues the straight line of predicated MMAs of a stage
// and the commit.  Every MMA accumulates (the epilogue hands the accumulators over zeroed) and updates only the
// accumulator lanes of rows that have an input under its offset: the row masks of a tile are loaded a tile ahead
// (one coalesced load per 32 words), parked inverted in shared memory, and the issuing lane reads four words per offset.
template <int kPieces, int kChunks, int kGroup, bool kPacked>
__device__ __forceinline__ void mma_role(const TcParams& p, const Smem& s, uint32_t tmem_base) {
  constexpr int kSteps = kPieces * kChunks / 2;  // tcgen05.mma instructions (K = 16 each) per block
  constexpr uint32_t kRowBytes = kPieces * 16;
  constexpr uint32_t a_step = (kTileRows * kRowBytes * kChunks) >> 4;  // = p.a_bytes / 16
  constexpr uint32_t cs_a = (kTileRows * kRowBytes) >> 4;              // between the 64-column blocks of A
  Shared* sh = s.sh;
  volatile int* abort_flag = &sh->abort_flag;
  const int lane = threadIdx.x & 31;
  // descriptor high word: stride between 8-row groups, version, swizzle mode
  const uint64_t desc_hi = (uint64_t)(((8u * kRowBytes) >> 4) | (1u << 14) | (p.layout_type << 29)) << 32;
  const uint32_t cs_b = (uint32_t)(p.cout * kRowBytes) >> 4;
  const uint32_t b_step = p.b_bytes >> 4, stage_step = s.stage_bytes >> 4;
  const uint32_t tiles_lo = desc_lo(smem_u32(s.tiles)), bres_lo = desc_lo(smem_u32(s.bres));
  const uint32_t idesc = p.idesc;
  const bool resident = p.b_resident != 0;
  if (resident && !__all_sync(0xffffffffu, mbar_wait(&sh->b_ready, 0, abort_flag, 23))) return;
  int stage = 0, acc = 0, buf = 0;
  uint32_t phase = 0, acc_phase = 0;
  const int num_stages = p.stages, kparts = p.kparts;
  const int row_words = p.kvol * 4;  // at most 128
  bool landed = false;  // the stage about to be waited for was already seen full by the probe below
  pdl_wait();
  PROF_DECL
  uint32_t rows_ahead[4];
  auto load_rows = [&](int tile) {
    const uint32_t* w = p.row_masks + (int64_t)tile * row_words + lane;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      rows_ahead[i] = (tile < p.num_tiles && lane + 32 * i < row_words) ? __ldg(w + 32 * i) : 0u;
  };
  uint32_t mask_ahead = load_mask(p, tile_at<kPacked>(p, 0));
  load_rows(tile_at<kPacked>(p, 0));
  for (int round = 0, tile; (tile = tile_at<kPacked>(p, round)) < p.num_tiles; ++round) {
    const uint32_t mask = __shfl_sync(0xffffffffu, mask_ahead, 0);
    uint32_t* lanes_off = sh->lanes_off[buf];
    if (mask != 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) lanes_off[lane + 32 * i] = ~rows_ahead[i];
    }
    // round trips to L2: in flight while this tile is issued
    mask_ahead = load_mask(p, tile_at<kPacked>(p, round + 1));
    load_rows(tile_at<kPacked>(p, round + 1));
    if (mask == 0) continue;  // a tile no offset feeds uses no accumulator: the epilogue writes its bias rows alone
    __syncwarp();
    PROF(0);
    if (!__all_sync(0xffffffffu, mbar_wait(&sh->acc_empty[acc], acc_phase, abort_flag, 22))) return;
    tc_fence_after();
    PROF(4);
    const uint32_t d_addr = tmem_base + (uint32_t)(acc * p.cout);
    // windows: for (base = 0; base < kvol; base += kGroup) over the windows that have an offset; packed stages:
    // while offsets are left, the kGroup lowest of them
    uint32_t rest = mask;
    for (int base = 0; kPacked ? rest != 0u : base < p.kvol; base += kPacked ? 0 : kGroup) {
      uint32_t bits;  // the offsets of the tile's next stage
      if (kPacked) {
        bits = lowest_bits<kGroup>(rest);
        rest &= ~bits;
      } else {
        bits = (mask >> base) & ((1u << kGroup) - 1u);
        if (bits == 0u) continue;
      }
      int k[kGroup];
      const uint32_t used = slot_offsets<kGroup, kPacked>(bits, base, k);
      for (int part = 0; part < kparts; ++part) {
        // the full barrier guards shared memory only: no tcgen05 fence is needed, but the rows written by
        // cp.async (generic proxy) must be made visible to the tensor core's reads (async proxy)
        PROF(0);
        if (!__all_sync(0xffffffffu, landed || mbar_wait(&sh->full[stage], phase, abort_flag, 21))) return;
        PROF(1);
        fence_proxy_async();
        PROF(2);
        // look at the following stage's barrier now: the answer (a round trip to shared memory) arrives while
        // this stage's MMAs are issued, and a stage that has already landed then costs no wait at all
        const bool wrap = stage + 1 == num_stages;
        const int stage_next = wrap ? 0 : stage + 1;
        const uint32_t phase_next = phase ^ (wrap ? 1u : 0u);
        const bool landed_next = mbar_test(&sh->full[stage_next], phase_next);
        const uint32_t a_lo = tiles_lo + (uint32_t)stage * stage_step;
        const uint32_t b_stage = a_lo + (uint32_t)kGroup * a_step;
        // descriptors of all MMAs of the stage first (independent, warp-uniform arithmetic), then the straight
        // line of MMAs: the issuing lane runs no dependent chain between two of them
        uint64_t desc_a[kGroup][kSteps], desc_b[kGroup][kSteps];
#pragma unroll
        for (int e = 0; e < kGroup; ++e) {
          // resident weights are indexed by the offset, streamed ones by the slot
          const uint32_t b_lo = resident ? bres_lo + (uint32_t)k[e] * b_step
                                         : b_stage + (uint32_t)e * b_step;
#pragma unroll
          for (int ks = 0; ks < kSteps; ++ks) {
            // 32 bytes per K step inside the swizzle span, the next 64-column block every 4 steps
            const uint32_t adv_a = (uint32_t)e * a_step + (uint32_t)(ks >> 2) * cs_a + (uint32_t)(ks & 3) * 2u;
            const uint32_t adv_b = (uint32_t)(ks >> 2) * cs_b + (uint32_t)(ks & 3) * 2u;
            desc_a[e][ks] = desc_hi | (a_lo + adv_a);
            desc_b[e][ks] = desc_hi | (b_lo + adv_b);
          }
        }
        if (elect_one()) {
          const uint4* off = reinterpret_cast<const uint4*>(lanes_off);
#pragma unroll
          for (int e = 0; e < kGroup; ++e) {
            const uint4 o = off[k[e]];
#pragma unroll
            for (int ks = 0; ks < kSteps; ++ks)
              umma_f16_rows_if((used >> e) & 1u, d_addr, desc_a[e][ks], desc_b[e][ks], idesc, o);
          }
          umma_commit(&sh->empty[stage]);  // the stage may be refilled once these MMAs have read it
        }
        __syncwarp();
        PROF(3);
        stage = stage_next, phase = phase_next, landed = landed_next;
      }
    }
    if (elect_one()) umma_commit(&sh->acc_full[acc]);
    __syncwarp();
    buf ^= 1;
    if (++acc == kNumAcc) acc = 0, acc_phase ^= 1;
  }
  PROF_STORE(1, (threadIdx.x & 31) == 0)
}

// ---- epilogue ----------------------------------------------------------------------------------------------------
// Epilogue warp `quad` (= warp index mod 4: it may touch TMEM lanes [32*quad, 32*quad + 32)).  The accumulators are
// handed to the MMA warp zeroed: once at the start, then every time one has been read.
template <bool kPacked>
__device__ __forceinline__ void epilogue_role(const TcParams& p, const Smem& s, uint32_t tmem_base, int quad) {
  Shared* sh = s.sh;
  volatile int* abort_flag = &sh->abort_flag;
  const int lane = threadIdx.x & 31;
  int acc = 0;
  uint32_t acc_phase = 0;
  const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
  for (int a = 0; a < kNumAcc; ++a) {
    for (int c0 = 0; c0 < p.cout; c0 += 16) tmem_st16_same(lane_base + (uint32_t)(a * p.cout + c0), 0u);
    tmem_st_wait();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(&sh->acc_empty[a]);
  }
  pdl_wait();  // residual rows come from an earlier layer; output rows may still be read by the preceding kernel
  uint32_t mask = load_mask(p, tile_at<kPacked>(p, 0));
  // the output a tile row stands for (the row itself, unless the table's outputs were regrouped): loaded a tile ahead
  auto load_row = [&](int tile) -> int {
#ifdef D3D_TC_NO_PERM
    return tile < p.num_tiles ? tile * kTileRows + quad * 32 + lane : -1;
#else
    return tile < p.num_tiles ? __ldg(p.perm + (int64_t)tile * kTileRows + quad * 32 + lane) : -1;
#endif
  };
  int row_ahead = load_row(tile_at<kPacked>(p, 0));
  PROF_DECL
  for (int round = 0, tile; (tile = tile_at<kPacked>(p, round)) < p.num_tiles; ++round) {
    const int next = tile_at<kPacked>(p, round + 1);
    const uint32_t next_mask = next < p.num_tiles ? __ldg(p.tile_mask + next) : 0u;
    const int64_t row = row_ahead;
    row_ahead = load_row(next);
    const bool empty_tile = mask == 0;  // bias (+ residual) only, no accumulator involved
    PROF(0);
    if (!empty_tile) {
      if (!mbar_wait(&sh->acc_full[acc], acc_phase, abort_flag, 31)) return;
      tc_fence_after();
    }
    PROF(1);
    const bool row_ok = row >= 0 && row < p.m_max;
    unsigned short* out_row = reinterpret_cast<unsigned short*>(p.out) + row * p.cout;
    const unsigned short* res_row =
        (p.residual && row_ok) ? reinterpret_cast<const unsigned short*>(p.residual) + row * p.cout : nullptr;
    const uint32_t taddr = lane_base + (uint32_t)(acc * p.cout);
    for (int c0 = 0; c0 < p.cout; c0 += 16) {
      uint32_t v[16];
      if (empty_tile) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0u;
      } else {
        tmem_ld16(taddr + c0, v);
        tmem_ld_wait();
        tmem_st16_same(taddr + c0, 0u);  // the next tile of this accumulator starts from zero
      }
      if (row_ok) {
        if (p.is_bf16) store_chunk<true>(v, s.bias, c0, out_row, res_row, p.relu);
        else store_chunk<false>(v, s.bias, c0, out_row, res_row, p.relu);
      }
    }
    if (!empty_tile) {
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->acc_empty[acc]);
      if (++acc == kNumAcc) acc = 0, acc_phase ^= 1;
    }
    PROF(2);
    mask = next_mask;
  }
  PROF_STORE(2, quad == 0 && lane == 0)
}

// kPieces x kChunks = 16-byte pieces per A row (2, 4, 8, 16), kGroup = offsets per stage, kProdWarps = 4 or 8,
// kCtas = CTAs per SM the launch is planned for (1 or 2).
template <int kPieces, int kChunks, int kGroup, int kProdWarps, int kCtas, bool kPacked>
__global__ void __launch_bounds__(threads_of(kProdWarps), kCtas)
spconv_mm_tc_kernel(const __grid_constant__ CUtensorMap map_b, const TcParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const Smem s = carve_smem<kGroup>(smem_raw, p);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tmem_base = cta_setup<kProdWarps>(p, s);
  pdl_release();
  if (warp < kProdWarps) {
    producer_role<kPieces, kChunks, kGroup, kProdWarps, kPacked>(p, s, warp, lane);
  } else if (warp == kProdWarps) {
    mma_role<kPieces, kChunks, kGroup, kPacked>(p, s, tmem_base);
    __syncwarp();
  } else if (warp == kProdWarps + 1) {
    if (lane == 0) control_role<kGroup, kPacked>(p, s, &map_b);
    __syncwarp();
  } else {
    epilogue_role<kPacked>(p, s, tmem_base, warp & 3);
  }
  cta_teardown<kProdWarps>(p, tmem_base);
}

// ---- host --------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      return reinterpret_cast<EncodeTiledFn>(ptr);
    return static_cast<EncodeTiledFn>(nullptr);
  }();  // initialised once, thread-safe
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

// Tuning override for experiments (0 = automatic): offsets per stage and pipeline stages.
int g_plan_group = 0, g_plan_stages = 0, g_plan_prod_warps = 0;

typedef void (*KernelFn)(const CUtensorMap, const TcParams);
struct KernelEntry {
  int pieces, chunks, group, prod_warps, ctas;
  KernelFn fn[2];  // fixed windows of offsets per stage / the offsets present packed into the stages
};
#define D3D_TC_K(P, C, G, W, N) \
  {P, C, G, W, N, {spconv_mm_tc_kernel<P, C, G, W, N, false>, spconv_mm_tc_kernel<P, C, G, W, N, true>}}
// One kernel instance per (row width of a block, offsets per stage, CTAs per SM).
const KernelEntry kKernels[] = {
    D3D_TC_K(2, 1, 8, 8, 2), D3D_TC_K(2, 1, 4, 8, 2), D3D_TC_K(2, 1, 2, 8, 2), D3D_TC_K(2, 1, 1, 8, 2),
    D3D_TC_K(4, 1, 4, 8, 2), D3D_TC_K(4, 1, 3, 8, 2), D3D_TC_K(4, 1, 2, 8, 2), D3D_TC_K(4, 1, 1, 8, 2),
    D3D_TC_K(8, 1, 2, 8, 2), D3D_TC_K(8, 1, 1, 8, 2),
    D3D_TC_K(2, 1, 8, 4, 2), D3D_TC_K(4, 1, 3, 4, 2), D3D_TC_K(8, 1, 1, 4, 2), D3D_TC_K(8, 1, 2, 4, 2),
    D3D_TC_K(2, 1, 8, 8, 1), D3D_TC_K(2, 1, 4, 8, 1), D3D_TC_K(2, 1, 2, 8, 1), D3D_TC_K(2, 1, 1, 8, 1),
    D3D_TC_K(4, 1, 4, 8, 1), D3D_TC_K(4, 1, 3, 8, 1), D3D_TC_K(4, 1, 2, 8, 1), D3D_TC_K(4, 1, 1, 8, 1),
    D3D_TC_K(8, 1, 2, 8, 1), D3D_TC_K(8, 1, 1, 8, 1), D3D_TC_K(8, 2, 1, 8, 1),
};
#undef D3D_TC_K
constexpr int kNumKernels = sizeof(kKernels) / sizeof(kKernels[0]);

const KernelEntry* find_kernel(int pieces, int chunks, int group, int prod_warps, int ctas) {
  for (int i = 0; i < kNumKernels; ++i)
    if (kKernels[i].pieces == pieces && kKernels[i].chunks == chunks && kKernels[i].group == group &&
        kKernels[i].prod_warps == prod_warps && kKernels[i].ctas == ctas)
      return &kKernels[i];
  return nullptr;
}

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

// Creates the per-handle state of the tensor-core path (the tensor map over the transposed weights).  Called from
// d3d_spconv_mm_configure, so that an enqueue neither allocates nor encodes.
int spconv_mm_tc_prepare(d3d_spconv_mm_s* h, int dtype) {
  if (!spconv_mm_tc_eligible(h, dtype)) return D3D_OK;
  const int cin = h->p.in_channels, cout = h->p.out_channels, kvol = h->p.kernel_vol;
  TcState* st = new (std::nothrow) TcState();
  D3D_REQUIRE(st, D3D_ERR_INVALID_ARGUMENT);
  const uint32_t box_cols = cin < 64 ? cin : 64;
  st->map_b_ok = make_map(&st->map_b, dtype, h->wt_dev, cin, (uint64_t)kvol * cout, box_cols, cout);
  h->tc_state = st;
  return st->map_b_ok ? D3D_OK : D3D_ERR_CUDA;
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
  TcState* st = reinterpret_cast<TcState*>(h->tc_state);
  D3D_REQUIRE(st && st->map_b_ok, D3D_ERR_INVALID_ARGUMENT);  // configure() creates it

  TcParams p;
  p.table = a.table;
  p.tile_mask = reinterpret_cast<const uint32_t*>(reinterpret_cast<const unsigned char*>(a.table) +
                                                  table_ids_bytes(kvol, m_max));
  p.row_masks = reinterpret_cast<const uint32_t*>(reinterpret_cast<const unsigned char*>(p.tile_mask) +
                                                  table_mask_bytes(m_max));
  p.perm = reinterpret_cast<const int32_t*>(reinterpret_cast<const unsigned char*>(p.row_masks) +
                                            table_rows_bytes(kvol, m_max));
  p.in_feats = a.in_feats;
  p.m_max = m_max;
  p.n_in_rows = (int32_t)a.max_num_act_in;
  p.kvol = kvol, p.cin = cin, p.cout = cout;
  p.num_tiles = (int)((m_max + kTileRows - 1) / kTileRows);
  const int box_cols = cin < 64 ? cin : 64;
  p.row_bytes = box_cols * 2;
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

  // Shared-memory plan.  Control data of a CTA: alignment slack, bias, barriers and row flags.
  const size_t ctrl = 1024 + align_up((size_t)cout * 4 + 8, 16) + sizeof(Shared);
  const size_t swizzle_repeat = (size_t)8 * p.row_bytes;  // operand blocks start on a multiple of it
  struct Plan {
    int kchunk, resident, group, stages;
    size_t smem;
    const KernelEntry* kernel;
  };
  // `two_per_sm`: 4 producer warps and half the SM's shared memory and tensor-memory columns per CTA.
  auto make_plan = [&](bool two_per_sm, int kchunk, Plan* out) -> bool {
    if (two_per_sm && (kchunk > 64 || cols > 256)) return false;
    const int pieces = kchunk >= 64 ? 8 : kchunk / 8, chunks = kchunk > 64 ? kchunk / 64 : 1;
    const int ksteps = kchunk / 16, kparts = cin / kchunk;
    const size_t a_bytes = (size_t)kTileRows * kchunk * 2;
    const size_t b_bytes = align_up((size_t)cout * kchunk * 2, swizzle_repeat);
    const size_t limit = two_per_sm ? 113 * 1024 : 227 * 1024;
    if (ctrl + 2 * (a_bytes + b_bytes) > limit) return false;
    // two producer teams, except for 32-channel blocks, which measured better with one (B200: 94 vs 102 us at
    // 463 k voxels; 64 channels: 102 vs 116 us, 128: 68 vs 73 us the other way round)
    const int prod_warps = g_plan_prod_warps ? g_plan_prod_warps : (two_per_sm && kchunk == 32 ? 4 : 8);
    const size_t budget = limit - ctrl;
    const size_t bres_bytes = (size_t)kvol * b_bytes;
    Plan best;
    best.stages = 0, best.group = 0, best.kernel = nullptr;
    int best_score = -1;
    for (int resident = 1; resident >= 0; --resident) {
      // resident weights whenever two stages still fit beside them, streamed per stage only otherwise: a streamed
      // W[k] crosses from L2 once per tile and sits in the hand-over loop (B200, 463 k voxels: 32 -> 32 85.6 vs
      // 88.2 us, 16 -> 32 36.9 vs 39.9 us)
      if (resident && (kparts != 1 || bres_bytes + 2 * a_bytes > budget)) continue;
      if (!resident && best_score >= 0) continue;
      const size_t ring = budget - (resident ? bres_bytes : 0);
      const size_t blk = a_bytes + (resident ? 0 : b_bytes);
      for (int group = kMaxGroup; group >= 1; --group) {
        const KernelEntry* k = find_kernel(pieces, chunks, group, prod_warps, two_per_sm ? 2 : 1);
        if (!k) continue;
        if (g_plan_group && group != g_plan_group) continue;
        if (group > 1 && (group * ksteps > 8 || group > kvol)) continue;
        // with K parts, offsets that share a stage would accumulate part by part instead of offset by offset: keep
        // the one accumulation order every plan produces
        if (group > 1 && kparts > 1) continue;
        int stages = (int)(ring / ((size_t)group * blk));
        if (stages > kMaxStages) stages = kMaxStages;
        if (g_plan_stages && stages > g_plan_stages) stages = g_plan_stages;
        if (stages < 2) continue;
        // eight MMAs per hand-over first (B200, 64 -> 64 at 238 k voxels: two offsets per stage in two stages 84 us,
        // one offset per stage in four stages 94 us), then up to three stages (more add little), then more MMAs
        const int depth = stages >= 3 ? 3 : stages;
        const int mmas = group * ksteps;
        const int score = (mmas > 8 ? 8 : mmas) * 400 + depth * 1000 + mmas * 10 + (stages > 4 ? 4 : stages) + resident * 5;
        if (score > best_score) {
          best_score = score;
          best.kchunk = kchunk, best.resident = resident, best.group = group, best.stages = stages, best.kernel = k;
          best.smem = ctrl + (size_t)stages * group * blk + (resident ? bres_bytes : 0);
        }
      }
    }
    if (best_score < 0) return false;
    // pin the number of CTAs per SM through the request: more than a third (half) of the SM's shared memory
    const size_t floor_bytes = two_per_sm ? 80 * 1024 : 120 * 1024;
    if (best.smem < floor_bytes) best.smem = floor_bytes;
    *out = best;
    return true;
  };
  Plan pl;
  bool two_per_sm = false;
  if (h->kernel_choice != 3) two_per_sm = make_plan(true, cin < 64 ? cin : 64, &pl) && pl.stages >= 2;
  if (!two_per_sm) {
    Plan wide, narrow;
    const bool have_wide = cin >= 128 && make_plan(false, 128, &wide);
    const bool have_narrow = make_plan(false, cin < 64 ? cin : 64, &narrow);
    D3D_REQUIRE(have_wide || have_narrow, D3D_ERR_TOO_LARGE);
    // 128-channel blocks (eight MMAs per hand-over) when three of them fit, else 64-channel K parts
    pl = (have_wide && (wide.stages >= 3 || !have_narrow)) ? wide : narrow;
  }
  p.kchunk = pl.kchunk;
  p.kparts = cin / pl.kchunk;
  p.chunks = pl.kchunk <= 64 ? 1 : pl.kchunk / 64;
  p.a_bytes = (uint32_t)((size_t)kTileRows * pl.kchunk * 2);
  p.b_bytes = (uint32_t)align_up((size_t)cout * pl.kchunk * 2, swizzle_repeat);
  p.b_resident = pl.resident, p.stages = pl.stages;
  const int packed = a.regrouped ? 1 : 0;
  const KernelFn kernel = pl.kernel->fn[packed];
  {
    // raising the dynamic shared memory limit is per function and per device; once each, under a lock
    static std::mutex attr_lock;
    static bool attr_set[64][kNumKernels][2] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return D3D_ERR_CUDA;
    const int ki = (int)(pl.kernel - kKernels);
    std::lock_guard<std::mutex> guard(attr_lock);
    if (!attr_set[dev][ki][packed]) {
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
        return D3D_ERR_CUDA;
      attr_set[dev][ki][packed] = true;
    }
  }
  const int ctas = kNumSMs * (two_per_sm ? 2 : 1);
  const int grid = p.num_tiles < ctas ? p.num_tiles : ctas;
  // programmatic dependent launch (opt-in per handle): the prologue of this kernel (barriers, tensor memory,
  // weights) may overlap the tail of the preceding kernel of the stream; every role waits for that kernel before
  // it touches its data.  Measured on B200: 3-4 us less per launch for layers run back to back on one stream; a
  // loss where other streams have kernels that would otherwise fill the tail of the preceding kernel.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(threads_of(pl.kernel->prod_warps));
  cfg.dynamicSmemBytes = pl.smem, cfg.stream = reinterpret_cast<cudaStream_t>(a.stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = h->dependent_launch ? 1 : 0;
  if (cudaLaunchKernelEx(&cfg, kernel, st->map_b, p) != cudaSuccess) return D3D_ERR_CUDA;
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

#ifdef D3D_TC_PROFILE
extern "C" int d3d_debug_copy_prof(long long* dst) {
  cudaDeviceSynchronize();
  return (int)cudaMemcpyFromSymbol(dst, d3d::g_prof, sizeof(long long) * 24);
}
#endif

// Tuning aid without a reference counterpart: overrides the pipeline plan of the tensor-core kernel for every later
// launch of this process (kernel offsets per stage, maximum number of stages, producer warps; 0 = automatic).  Not thread-safe.
extern "C" int d3d_debug_set_tc_plan(int group, int max_stages, int prod_warps) {
  if (group < 0 || group > d3d::kMaxGroup || max_stages < 0 || max_stages > d3d::kMaxStages ||
      !(prod_warps == 0 || prod_warps == 4 || prod_warps == 8))
    return D3D_ERR_INVALID_ARGUMENT;
  d3d::g_plan_group = group, d3d::g_plan_stages = max_stages, d3d::g_plan_prod_warps = prod_warps;
  return D3D_OK;
}
