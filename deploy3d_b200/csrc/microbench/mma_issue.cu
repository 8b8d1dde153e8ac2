// Stand-alone measurement, not part of the library:
//     nvcc -gencode arch=compute_100a,code=sm_100a -O2 -o mma_issue mma_issue.cu && ./mma_issue
// What one warp spends per pipeline stage when it hands a stage of M=128, K=16 tcgen05.mma instructions to the tensor
// core, for N = 32 / 64 / 128, 8 or 16 MMAs per stage, and 1, 2 or 4 issuing warps per SM (each with its own
// accumulator and barriers).  Operands are zeroed shared memory; a ring of 4 stage slots; the per-stage offset mask
// comes from a volatile shared load, so the compiler cannot know it.  `flags` switches the parts of the hand-over on:
// 1 = wait on a (completed) full barrier, 2 = fence.proxy.async, 4 = tcgen05.commit to the slot's empty barrier,
// 8 = the offset mask goes through a shuffle from lane 0 (warp-uniform for the compiler).  take = ff issues every MMA,
// take = 00 none (what the hand-over alone costs).  Every wait is bounded.  Prints cycles per stage and warp.
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               :: "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_if(uint32_t run, uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               :: "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc), "r"(run) : "memory");
}
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred P;\n\t.reg .b32 r;\n\telect.sync r|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
  return pred;
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ void commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void commit_if(uint32_t run, uint64_t* bar) {
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(smem_u32(bar)), "r"(run) : "memory");
}

struct R { long long issue[4], total[4]; int err; };
// Every issuing warp w (< nwarps) runs its own ring of 4 slots, its own TMEM columns and barriers.
// flags: 1 try_wait, 2 fence.proxy.async, 4 commit per stage, 8 take via shfl (uniform) else raw volatile
template <int MMAS>
__global__ void __launch_bounds__(256, 1) k(int n, int row_bytes, int layout, int reps, int take_in, int flags, int nwarps, R* out) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ uint64_t bar[4], full[4][4], empty[4][4]; __shared__ uint32_t tbase;
  for (int i = threadIdx.x; i < 200 * 1024 / 4; i += blockDim.x) ((uint32_t*)smem)[i] = 0;
  if (threadIdx.x == 0) {
    for (int w = 0; w < 4; ++w) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar[w])));
      for (int i = 0; i < 4; ++i) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&full[w][i])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&empty[w][i])));
      }
    }
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tbase)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tb = tbase;
  __shared__ volatile uint32_t sbase[8];
  if (threadIdx.x < 8) sbase[threadIdx.x] = threadIdx.x & 1;
  __syncthreads();
  const int w = threadIdx.x >> 5;
  if (w < nwarps) {
    const uint32_t idesc = (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((128u >> 4) << 24);
    const uint32_t a0 = smem_u32(smem) + w * 32 * 1024, b0 = smem_u32(smem) + 160 * 1024;
    const uint64_t desc_hi = (uint64_t)(((8u * row_bytes) >> 4) | (1u << 14) | ((uint32_t)layout << 29)) << 32;
    const uint32_t a_lo0 = ((a0 & 0x3FFFFu) >> 4) | (1u << 16), b_lo0 = ((b0 & 0x3FFFFu) >> 4) | (1u << 16);
    const uint32_t td = tb + w * 128;
    long long t0 = clock64();
    int stage = 0;
    uint32_t accv = 0;
    for (int r = 0; r < reps; ++r) {
      uint32_t take = take_in + sbase[r & 7] * 0;  // value unknown to the compiler
      if (flags & 8) take = __shfl_sync(0xffffffffu, take, 0);
      if (flags & 1) for (int spin = 0; spin < 1000 && !mbar_try_wait(&full[w][stage], 1); ++spin) {}
      if (flags & 2) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      const uint32_t a_lo = a_lo0 + stage * 256, b_lo = b_lo0;
      if (elect_one()) {
#pragma unroll
        for (int e = 0; e < MMAS; ++e) {
          const uint32_t present = (take >> (e & 7)) & 1u;
          umma_if(present, td, desc_hi | (a_lo + (e & 7) * 16), desc_hi | (b_lo + (e & 7) * 8), idesc, accv);
          accv |= present;
        }
        if (flags & 4) commit(&empty[w][stage]);
      }
      accv = __shfl_sync(0xffffffffu, accv, 0) | (take != 0);
      if (++stage == 4) stage = 0;
    }
    long long t1 = clock64();
    if ((threadIdx.x & 31) == 0) {
      commit(&bar[w]);
      int err = 1;
      for (int it = 0; it < 4000000; ++it) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(smem_u32(&bar[w])), "r"(0) : "memory");
        if (ok) { err = 0; break; }
      }
      long long t2 = clock64();
      if (blockIdx.x == 0) { out->issue[w] = t1 - t0; out->total[w] = t2 - t0; if (err) out->err = err; }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x < 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tb), "r"(512) : "memory");
}
template <int MMAS> void run(R* d, int n, int take, int flags, int nwarps) {
  const int reps = 256;
  cudaFuncSetAttribute(k<MMAS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  cudaMemset(d, 0, sizeof(R));
  const int rb = n >= 64 ? 128 : 64, lay = n >= 64 ? 2 : 4;
  k<MMAS><<<148, 256, 200 * 1024>>>(n, rb, lay, reps, take, flags, nwarps, d);
  R h;
  cudaError_t e = cudaMemcpy(&h, d, sizeof(R), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) { printf("cuda error %s\n", cudaGetErrorString(e)); exit(1); }
  printf("N %3d mmas/stage %2d take %02x flags %2d warps %d: per-warp total cyc/stage", n, MMAS, take, flags, nwarps);
  for (int w = 0; w < nwarps; ++w) printf(" %6.1f", (double)h.total[w] / reps);
  printf("  err %d\n", h.err);
}
int main() {
  R* d; cudaMalloc(&d, sizeof(R));
  for (int take : {0xFF, 0x00}) {
    for (int flags : {8, 9, 10, 12, 15, 7}) run<8>(d, 32, take, flags, 1);
    run<16>(d, 32, take, 15, 1);
    run<8>(d, 32, take, 15, 2);
    run<8>(d, 32, take, 15, 4);
    run<16>(d, 32, take, 15, 2);
  }
  for (int n : {16, 64, 128}) { run<8>(d, n, 0xFF, 8, 1); run<8>(d, n, 0xFF, 15, 1); run<8>(d, n, 0xFF, 15, 2); }
  return 0;
}
