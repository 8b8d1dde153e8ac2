// Stand-alone measurement, not part of the library:
//     nvcc -gencode arch=compute_100a,code=sm_100a -O2 -o gather_rows gather_rows.cu -lcuda && ./gather_rows
// How fast one SM gathers arbitrary rows of a row-major fp16 matrix [460 000][C] (C = 16, 32, 64: rows of 32, 64,
// 128 bytes) into blocks of 128 rows in shared memory, laid out K-major with the swizzle of the row width, by
//   mode 0  16-byte cp.async: four warps, lane = (row, 16-byte piece), the XOR swizzle applied to the destination,
//           three blocks in flight (cp.async groups);
//   mode 1  TMA tile::gather4: one warp, every lane issues one cp.async.bulk.tensor.2d...tile::gather4 (four rows)
//           per block onto the block's mbarrier, a ring of four blocks in flight.
// One CTA per SM, 148 CTAs, 2000 blocks each, random row ids (same ids for both modes).  Prints nanoseconds per
// gathered row and SM, and rows per second of the whole GPU.  Every wait is bounded.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  for (int it = 0; it < 20000000; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

constexpr int kRowsPerBlock = 128;
constexpr int kRing = 4;

template <int kRowBytes>
__global__ void __launch_bounds__(128, 1)
gather_kernel(const __grid_constant__ CUtensorMap map, const unsigned char* feats, const int* ids, int blocks, int mode,
              int* err, unsigned long long* sink) {
  extern __shared__ __align__(1024) unsigned char raw[];
  unsigned char* ring = raw + ((1024u - (smem_u32(raw) & 1023u)) & 1023u);
  __shared__ uint64_t full[kRing];
  constexpr uint32_t kBlockBytes = kRowsPerBlock * kRowBytes;
  constexpr int kPieces = kRowBytes / 16;
  constexpr int kRowsPerPass = 128 / kPieces;  // rows all 128 threads cover per pass
  constexpr int kPasses = kRowsPerBlock / kRowsPerPass;
  constexpr int kSwzShift = kRowBytes == 128 ? 0 : kRowBytes == 64 ? 1 : 2;
  constexpr int kSwzMask = kRowBytes == 128 ? 7 : kRowBytes == 64 ? 3 : 1;
  const int t = threadIdx.x, lane = t & 31;
  if (t == 0)
    for (int i = 0; i < kRing; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&full[i])));
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncthreads();
  const int* my_ids = ids + (size_t)blockIdx.x * blocks * kRowsPerBlock;
  if (mode == 0) {
    const int j = t % kPieces, rsub = t / kPieces;
    for (int b = 0; b < blocks; ++b) {
      const uint32_t dst = smem_u32(ring) + (uint32_t)(b % kRing) * kBlockBytes;
#pragma unroll
      for (int i = 0; i < kPasses; ++i) {
        const int row = i * kRowsPerPass + rsub;
        const int id = __ldg(my_ids + b * kRowsPerBlock + row);
        const unsigned char* src = feats + (size_t)id * kRowBytes + j * 16;
        const uint32_t d = dst + (uint32_t)row * kRowBytes + ((uint32_t)(j ^ ((row >> kSwzShift) & kSwzMask)) << 4);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src));
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 3;" ::: "memory");  // at most three blocks in flight besides this one
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (t < 32) {
    for (int b = 0; b < blocks; ++b) {
      const int slot = b % kRing;
      // the slot's previous gather (kRing blocks ago) must have landed before it is overwritten
      if (b >= kRing && !mbar_wait_bounded(&full[slot], ((b / kRing) - 1) & 1)) {
        *err = 1;
        break;
      }
      if (lane == 0)
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&full[slot])),
                     "r"(kBlockBytes)
                     : "memory");
      __syncwarp();
      const int4 rows = __ldg(reinterpret_cast<const int4*>(my_ids + b * kRowsPerBlock) + lane);
      unsigned char* dst = ring + (size_t)slot * kBlockBytes + (size_t)4 * lane * kRowBytes;
      asm volatile(
          "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes"
          " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
          :
          : "r"(smem_u32(dst)), "l"((uint64_t)&map), "r"(smem_u32(&full[slot])), "r"(0), "r"(rows.x), "r"(rows.y),
            "r"(rows.z), "r"(rows.w)
          : "memory");
    }
    // drain: the last kRing blocks
    for (int b = blocks > kRing ? blocks - kRing : 0; b < blocks; ++b)
      if (!mbar_wait_bounded(&full[b % kRing], (b / kRing) & 1)) *err = 1;
  }
  __syncthreads();
  // keep the copies observable
  if (t == 0) sink[blockIdx.x] = *reinterpret_cast<unsigned long long*>(ring);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

template <int kRowBytes>
void run(EncodeTiledFn encode, const unsigned char* feats, const int* ids, int n_rows, int* err,
         unsigned long long* sink) {
  const int cols = kRowBytes / 2, blocks = 2000, ctas = 148;
  CUtensorMap map;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)n_rows};
  cuuint64_t strides[1] = {(cuuint64_t)kRowBytes};
  cuuint32_t box[2] = {(cuuint32_t)cols, 1};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = kRowBytes == 32   ? CU_TENSOR_MAP_SWIZZLE_32B
                                : kRowBytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                  : CU_TENSOR_MAP_SWIZZLE_128B;
  if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<unsigned char*>(feats), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
    printf("tensor map encode failed\n");
    exit(1);
  }
  const size_t smem = (size_t)kRing * kRowsPerBlock * kRowBytes + 1024;
  cudaFuncSetAttribute(gather_kernel<kRowBytes>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0), cudaEventCreate(&e1);
  for (int mode = 0; mode < 2; ++mode) {
    cudaMemset(err, 0, sizeof(int));
    gather_kernel<kRowBytes><<<ctas, 128, smem>>>(map, feats, ids, blocks, mode, err, sink);  // warm-up
    cudaEventRecord(e0);
    gather_kernel<kRowBytes><<<ctas, 128, smem>>>(map, feats, ids, blocks, mode, err, sink);
    cudaEventRecord(e1);
    int herr = 0;
    cudaError_t rc = cudaMemcpy(&herr, err, sizeof(int), cudaMemcpyDeviceToHost);
    if (rc != cudaSuccess) {
      printf("cuda error: %s\n", cudaGetErrorString(rc));
      exit(1);
    }
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    const double rows_per_cta = (double)blocks * kRowsPerBlock;
    printf("row %3d B  %-18s %7.2f ns per row and SM  %8.1f M rows/s per GPU  %7.1f GB/s  wait_error %d\n", kRowBytes,
           mode == 0 ? "cp.async 16 B" : "TMA tile::gather4", ms * 1e6 / rows_per_cta,
           rows_per_cta * ctas / (ms * 1e-3) / 1e6, rows_per_cta * ctas * kRowBytes / (ms * 1e-3) / 1e9, herr);
  }
}

int main() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess) {
    printf("cuTensorMapEncodeTiled not available\n");
    return 1;
  }
  const int n_rows = 460000, blocks = 2000, ctas = 148;
  unsigned char* feats;
  cudaMalloc(&feats, (size_t)n_rows * 128);
  cudaMemset(feats, 0x3c, (size_t)n_rows * 128);
  std::vector<int> h((size_t)ctas * blocks * kRowsPerBlock);
  uint64_t s = 88172645463325252ull;
  for (auto& v : h) {
    s ^= s << 13, s ^= s >> 7, s ^= s << 17;
    v = (int)(s % n_rows);
  }
  int *ids, *err;
  unsigned long long* sink;
  cudaMalloc(&ids, h.size() * sizeof(int));
  cudaMemcpy(ids, h.data(), h.size() * sizeof(int), cudaMemcpyHostToDevice);
  cudaMalloc(&err, sizeof(int));
  cudaMalloc(&sink, ctas * sizeof(unsigned long long));
  run<32>((EncodeTiledFn)fn, feats, ids, n_rows, err, sink);
  run<64>((EncodeTiledFn)fn, feats, ids, n_rows, err, sink);
  run<128>((EncodeTiledFn)fn, feats, ids, n_rows, err, sink);
  return 0;
}
