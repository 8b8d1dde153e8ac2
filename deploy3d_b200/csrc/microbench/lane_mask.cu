// Stand-alone check, not part of the library:
//     nvcc -gencode arch=compute_100a,code=sm_100a -O2 -o lane_mask lane_mask.cu && ./lane_mask
// Two properties the SPConvMM kernel relies on: (1) tcgen05.mma with a disable_output_lane vector leaves the masked
// TMEM lanes untouched whatever the corresponding rows of A hold, with and without accumulation; (2) tcgen05.st
// initialises an accumulator that a later accumulating MMA then adds to.  One CTA, M=128 N=16 K=16; A row r holds
// r % 8 + 1 in every k, B is all ones, so D[r][n] = 16 * (r % 8 + 1).  Every wait is bounded.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void umma_masked(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc,
                                            uint32_t m0, uint32_t m1, uint32_t m2, uint32_t m3) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(idesc), "r"(acc), "r"(m0), "r"(m1), "r"(m2), "r"(m3)
      : "memory");
}
__device__ __forceinline__ void commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool wait_bounded(uint64_t* bar, uint32_t parity) {
  for (int it = 0; it < 4000000; ++it) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
// out[0]: after st(7) + masked accumulate; out[1]: after a further masked overwrite (accumulate = 0, other mask)
__global__ void __launch_bounds__(128, 1) k(float* out, int* err, uint4 ma, uint4 mb) {
  __shared__ __align__(1024) unsigned char a_s[128 * 32];
  __shared__ __align__(1024) unsigned char b_s[16 * 32];
  __shared__ uint64_t bar;
  __shared__ uint32_t tbase;
  const int t = threadIdx.x;
  for (int i = 0; i < 16; ++i) reinterpret_cast<__half*>(a_s)[t * 16 + i] = __float2half((float)(t % 8 + 1));
  if (t < 16) for (int i = 0; i < 16; ++i) reinterpret_cast<__half*>(b_s)[t * 16 + i] = __float2half(1.f);
  if (t == 0) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar)));
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  if (t < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tbase)), "r"(32) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tb = tbase;
  const uint32_t taddr = tb + ((uint32_t)((t >> 5) * 32) << 16);
  uint32_t v[16];
  for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(7.f);
  tmem_st16(taddr, v);
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t idesc = (1u << 4) | ((uint32_t)(16 >> 3) << 17) | ((128u >> 4) << 24);
  const uint64_t desc_hi = (uint64_t)(((8u * 32) >> 4) | (1u << 14) | (6u << 29)) << 32;
  const uint64_t da = desc_hi | (((smem_u32(a_s) & 0x3FFFFu) >> 4) | (1u << 16));
  const uint64_t db = desc_hi | (((smem_u32(b_s) & 0x3FFFFu) >> 4) | (1u << 16));
  int bad = 0;
  for (int round = 0; round < 2; ++round) {
    if (t == 0) {
      const uint4 m = round == 0 ? ma : mb;
      umma_masked(tb, da, db, idesc, round == 0 ? 1u : 0u, m.x, m.y, m.z, m.w);
      commit(&bar);
    }
    if (!wait_bounded(&bar, round & 1)) bad = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    tmem_ld16(taddr, v);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    for (int i = 0; i < 16; ++i) out[(round * 128 + t) * 16 + i] = __uint_as_float(v[i]);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }
  if (bad) *err = 1;
  if (t < 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tb), "r"(32) : "memory");
}
int main() {
  float* d; int* e;
  cudaMalloc(&d, 2 * 128 * 16 * 4); cudaMalloc(&e, 4); cudaMemset(e, 0, 4); cudaMemset(d, 0, 2 * 128 * 16 * 4);
  const uint4 ma = make_uint4(0x0000FFFFu, 0u, 0xFFFFFFFFu, 0xAAAAAAAAu);  // set bit = lane NOT updated
  const uint4 mb = make_uint4(0xFFFF0000u, 0xFFFFFFFFu, 0u, 0x55555555u);
  k<<<1, 128>>>(d, e, ma, mb);
  static float h[2 * 128 * 16]; int he = 0;
  cudaError_t rc = cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
  cudaMemcpy(&he, e, 4, cudaMemcpyDeviceToHost);
  printf("cuda %s wait_err %d\n", cudaGetErrorString(rc), he);
  const uint32_t a[4] = {ma.x, ma.y, ma.z, ma.w}, b[4] = {mb.x, mb.y, mb.z, mb.w};
  int wrong0 = 0, wrong1 = 0;
  for (int r = 0; r < 128; ++r) {
    const float prod = 16.f * (r % 8 + 1);
    const bool dis_a = (a[r >> 5] >> (r & 31)) & 1, dis_b = (b[r >> 5] >> (r & 31)) & 1;
    const float e0 = dis_a ? 7.f : 7.f + prod;
    const float e1 = dis_b ? e0 : prod;
    for (int c = 0; c < 16; ++c) {
      if (h[r * 16 + c] != e0) { if (wrong0 < 5) printf("round0 r%d c%d got %g want %g\n", r, c, h[r * 16 + c], e0); ++wrong0; }
      if (h[(128 + r) * 16 + c] != e1) { if (wrong1 < 5) printf("round1 r%d c%d got %g want %g\n", r, c, h[(128 + r) * 16 + c], e1); ++wrong1; }
    }
  }
  printf("round0 wrong %d  round1 wrong %d (of 2048 each)\n", wrong0, wrong1);
  return 0;
}
