// Stand-alone measurement, not part of the library:
//     nvcc -gencode arch=compute_100a,code=sm_100a -O2 -o hash_probe_styles hash_probe_styles.cu && ./hash_probe_styles
// Three ways to look up the 27 neighbours of every voxel in the open-addressing table the SubM rulebook uses
// (64-bit slots key << 32 | value, all ones = empty, buckets of four slots = one 32-byte sector chosen by a hash of
// key >> 2, slot in the bucket = key & 3, so x-neighbours share a sector; next probe = same slot of the next bucket;
// capacity = power of two >= 4 x the keys):
//   A  one thread per voxel, 8-byte probes, the nine probes of a kernel plane issued together (what the library does)
//   B  one thread per voxel, one 32-byte load per bucket: the three x-neighbours of a kernel row share one or two
//   C  warp-cooperative: the warp takes its 32 voxels' queries one at a time, lane l reads slot l of the 32 slots
//      (eight buckets) following the home bucket, a ballot finds the key or an empty slot
// 463 000 voxels in a 41 x 1440 x 1440 grid, laid out in short runs along x (about a fifth of the probes hit).
// Prints microseconds per style (best of five) and a checksum (sum of the values found) that must agree.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <unordered_set>
#include <vector>

constexpr unsigned long long kEmpty = ~0ull;
__host__ __device__ inline uint32_t mix(uint32_t h) {
  h ^= h >> 16, h *= 0x85ebca6bu, h ^= h >> 13, h *= 0xc2b2ae35u, h ^= h >> 16;
  return h;
}
__host__ __device__ inline uint32_t home_slot(uint32_t key, uint32_t mask) {
  return ((mix(key >> 2) << 2) | (key & 3u)) & mask;
}
constexpr int Z = 41, Y = 1440, X = 1440;

__device__ __forceinline__ bool neighbour_key(int z, int y, int x, int k, uint32_t* key) {
  const int nz = z + k / 9 - 1, ny = y + (k / 3) % 3 - 1, nx = x + k % 3 - 1;
  *key = (uint32_t)((nz * Y + ny) * X + nx);
  return (unsigned)nz < (unsigned)Z && (unsigned)ny < (unsigned)Y && (unsigned)nx < (unsigned)X;
}

// A: 8-byte probes, nine in flight
__global__ void probe_a(const unsigned long long* __restrict__ table, uint32_t mask, const int4* __restrict__ vox, int n,
                        unsigned long long* out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int4 c = vox[i];
  unsigned long long acc = 0;
  for (int plane = 0; plane < 3; ++plane) {
    uint32_t key[9], slot[9];
    unsigned long long cur[9];
    uint32_t pending = 0;
#pragma unroll
    for (int b = 0; b < 9; ++b) {
      const bool ok = neighbour_key(c.x, c.y, c.z, plane * 9 + b, &key[b]);
      slot[b] = home_slot(key[b], mask);
      cur[b] = ok ? __ldg(table + slot[b]) : kEmpty;
    }
#pragma unroll
    for (int b = 0; b < 9; ++b) {
      if ((uint32_t)(cur[b] >> 32) == key[b]) acc += (uint32_t)cur[b];
      else if (cur[b] != kEmpty) pending |= 1u << b;
    }
    for (int round = 0; pending && round < 64; ++round) {
#pragma unroll
      for (int b = 0; b < 9; ++b)
        if ((pending >> b) & 1u) {
          slot[b] = (slot[b] + 4u) & mask;
          const unsigned long long v = __ldg(table + slot[b]);
          if ((uint32_t)(v >> 32) == key[b]) acc += (uint32_t)v, pending &= ~(1u << b);
          else if (v == kEmpty) pending &= ~(1u << b);
        }
    }
  }
  out[i] = acc;
}

// B: whole buckets, one 32-byte load each
__device__ __forceinline__ void load_bucket(const unsigned long long* p, unsigned long long (&s)[4]) {
  asm volatile("ld.global.nc.v4.u64 {%0, %1, %2, %3}, [%4];" : "=l"(s[0]), "=l"(s[1]), "=l"(s[2]), "=l"(s[3]) : "l"(p));
}
__global__ void probe_b(const unsigned long long* __restrict__ table, uint32_t mask, const int4* __restrict__ vox, int n,
                        unsigned long long* out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int4 c = vox[i];
  unsigned long long acc = 0;
  for (int row = 0; row < 9; ++row) {
    uint32_t key[3];
    bool ok[3];
#pragma unroll
    for (int b = 0; b < 3; ++b) ok[b] = neighbour_key(c.x, c.y, c.z, row * 3 + b, &key[b]);
    // keys of a row are consecutive: they fall into one or two buckets
    uint32_t done = 0;
#pragma unroll
    for (int b = 0; b < 3; ++b) {
      if (!ok[b] || ((done >> b) & 1u)) continue;
      uint32_t bucket = home_slot(key[b] & ~3u, mask);
      uint32_t want = 0;  // keys of this row that live in this bucket chain
#pragma unroll
      for (int d = b; d < 3; ++d)
        if (ok[d] && (key[d] >> 2) == (key[b] >> 2)) want |= 1u << d;
      done |= want;
      for (int round = 0; want && round < 64; ++round) {
        unsigned long long s[4];
        load_bucket(table + bucket, s);
#pragma unroll
        for (int d = 0; d < 3; ++d)
          if ((want >> d) & 1u) {
            const unsigned long long v = s[key[d] & 3u];
            if ((uint32_t)(v >> 32) == key[d]) acc += (uint32_t)v, want &= ~(1u << d);
            else if (v == kEmpty) want &= ~(1u << d);
          }
        bucket = (bucket + 4u) & mask;
      }
    }
  }
  out[i] = acc;
}

// C: warp-cooperative, 32 consecutive slots per probe
__global__ void probe_c(const unsigned long long* __restrict__ table, uint32_t mask, const int4* __restrict__ vox, int n,
                        unsigned long long* out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31;
  const int4 c = i < n ? vox[i] : make_int4(-9, -9, -9, 0);
  unsigned long long acc = 0;
  for (int k = 0; k < 27; ++k) {
    uint32_t my_key;
    const bool my_ok = i < n && neighbour_key(c.x, c.y, c.z, k, &my_key);
    for (int src = 0; src < 32; ++src) {  // the warp serves its lanes' queries one at a time
      const uint32_t key = __shfl_sync(0xffffffffu, my_key, src);
      if (!__shfl_sync(0xffffffffu, (int)my_ok, src)) continue;
      uint32_t base = home_slot(key & ~3u, mask);
      for (int round = 0; round < 8; ++round) {
        const unsigned long long v = __ldg(table + ((base + lane) & mask));
        // the key can only sit in slots whose position in their bucket is key & 3
        const bool mine = (lane & 3) == (int)(key & 3u);
        const unsigned hit = __ballot_sync(0xffffffffu, mine && (uint32_t)(v >> 32) == key);
        const unsigned empty = __ballot_sync(0xffffffffu, mine && v == kEmpty);
        if (hit) {  // found, unless an empty slot of the probe sequence comes first
          const unsigned first_empty = empty ? (unsigned)__ffs(empty) : 33u;
          const uint32_t value = __shfl_sync(0xffffffffu, (uint32_t)v, __ffs(hit) - 1);
          if ((unsigned)__ffs(hit) < first_empty && lane == src) acc += value;
          break;
        }
        if (empty) break;
        base = (base + 32u) & mask;
      }
    }
  }
  if (i < n) out[i] = acc;
}

int main() {
  const int n = 463000;
  std::vector<int4> vox;
  std::unordered_set<uint32_t> seen;
  uint64_t s = 0x9E3779B97F4A7C15ull;
  auto rnd = [&]() {
    s ^= s << 13, s ^= s >> 7, s ^= s << 17;
    return s;
  };
  while ((int)vox.size() < n) {  // runs of up to eight voxels along x, two or three layers thick now and then
    const int z = (int)(rnd() % Z), y = (int)(rnd() % Y), x = (int)(rnd() % (X - 8));
    const int len = 1 + (int)(rnd() % 8), thick = 1 + (int)(rnd() % 3 == 0);
    for (int t = 0; t < thick; ++t)
      for (int d = 0; d < len && (int)vox.size() < n; ++d) {
        const int yy = std::min(Y - 1, y + t);
        const uint32_t key = (uint32_t)((z * Y + yy) * X + x + d);
        if (seen.insert(key).second) vox.push_back(make_int4(z, yy, x + d, 0));
      }
  }
  uint32_t cap = 1;
  while (cap < 4u * n) cap <<= 1;
  const uint32_t mask = cap - 1;
  std::vector<unsigned long long> table(cap, kEmpty);
  for (int i = 0; i < n; ++i) {
    const uint32_t key = (uint32_t)((vox[i].x * Y + vox[i].y) * X + vox[i].z);
    uint32_t slot = home_slot(key, mask);
    while (table[slot] != kEmpty) slot = (slot + 4u) & mask;
    table[slot] = ((unsigned long long)key << 32) | (uint32_t)(i + 1);
  }
  unsigned long long *d_table, *d_sum;
  int4* d_vox;
  cudaMalloc(&d_table, (size_t)cap * 8), cudaMalloc(&d_vox, (size_t)n * sizeof(int4)), cudaMalloc(&d_sum, (size_t)n * 8);
  cudaMemcpy(d_table, table.data(), (size_t)cap * 8, cudaMemcpyHostToDevice);
  cudaMemcpy(d_vox, vox.data(), (size_t)n * sizeof(int4), cudaMemcpyHostToDevice);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0), cudaEventCreate(&e1);
  const char* names[3] = {"A 8-byte probes, nine in flight per thread", "B one 32-byte load per bucket",
                          "C warp-cooperative, 32 slots per probe"};
  for (int style = 0; style < 3; ++style) {
    float best = 1e30f;
    unsigned long long sum = 0;
    for (int rep = 0; rep < 5; ++rep) {
      cudaMemset(d_sum, 0, (size_t)n * 8);
      cudaEventRecord(e0);
      if (style == 0) probe_a<<<(n + 255) / 256, 256>>>(d_table, mask, d_vox, n, d_sum);
      if (style == 1) probe_b<<<(n + 255) / 256, 256>>>(d_table, mask, d_vox, n, d_sum);
      if (style == 2) probe_c<<<(n + 255) / 256, 256>>>(d_table, mask, d_vox, n, d_sum);
      cudaEventRecord(e1);
      std::vector<unsigned long long> h(n);
      if (cudaMemcpy(h.data(), d_sum, (size_t)n * 8, cudaMemcpyDeviceToHost) != cudaSuccess) {
        printf("cuda error: %s\n", cudaGetErrorString(cudaGetLastError()));
        return 1;
      }
      sum = 0;
      for (unsigned long long v : h) sum += v;
      float ms = 0;
      cudaEventElapsedTime(&ms, e0, e1);
      best = std::min(best, ms);
    }
    printf("%-46s %8.1f us   checksum %llu\n", names[style], best * 1e3f, sum);
  }
  return 0;
}
