// SPConvIdx: rulebook ("index") generation for submanifold, strided and transposed sparse convolution.
//
// Replaces spconv::func::createSparseSubMIndex / createSparseConvIndex of the reference
// (trt/spconv/index.cu:253-476) behind the I/O contract of SPConvIdxPlugin (trt/spconv/index_trt.cu:52-249).
//
// Pipeline (all counts stay on the device, no host synchronisation):
//   SubM : table reset -> insert inputs -> probe neighbours (pair table + per-CTA counts) -> segment scan
//          -> compaction -> padding fill
//   Conv : table reset -> insert outputs (first-touch pair id wins) -> count winners -> scan -> number
//          outputs + coordinates -> translate slots to output ids (+ per-CTA counts) -> segment scan
//          -> compaction -> padding fill
// Work decomposition: one thread per (input voxel, kernel row), a kernel row being the run of offsets along the
// fastest axis; a warp holds 32 consecutive inputs of one row so the pair table is written with 128-byte
// coalesced stores and the probes of one thread fall into one 32-byte hash bucket (see common.cuh).
#include "common.cuh"

namespace d3d {
namespace {

constexpr int kIdxThreads = 256;  // inputs per CTA in every pass; the granularity of the per-CTA counts
constexpr int kSegment = 128;     // every kernel-offset segment starts at a multiple of 128 (trt/spconv/index.cu:21)
constexpr int kMaxKernelVol = 512;
// SubM tables are sized for a load factor of at most 0.25: four of five neighbour probes miss, and a miss walks on
// until it meets an empty slot, so the sectors a miss touches (what bounds the probe kernel) fall with the load
constexpr int kSubmFan = 2;

struct Geometry {
  int ndim;
  int kvol;
  int rows;    // kvol / ksize[ndim-1]
  int klast;   // ksize[ndim-1]
  int transpose;
  int ksize[D3D_MAX_NDIM], stride[D3D_MAX_NDIM], pad[D3D_MAX_NDIM], dil[D3D_MAX_NDIM];
  int shape[D3D_MAX_NDIM + 1];  // extent of the key space: [B, D0', D1', ..]
};

__device__ __forceinline__ void load_coor(const int32_t* __restrict__ coors, int ndim, int64_t i, int* c) {
  if (ndim == 3) {
    int4 v = __ldg(reinterpret_cast<const int4*>(coors) + i);
    c[0] = v.x, c[1] = v.y, c[2] = v.z, c[3] = v.w;
  } else {
    for (int d = 0; d <= ndim; ++d) c[d] = __ldg(coors + i * (ndim + 1) + d);
  }
}

// Output coordinate along dimension d for kernel tap kd (trt/spconv/geometry.h:41-49 forward, :66-72 transposed).
__device__ __forceinline__ bool out_coord(const Geometry& g, int d, int in, int kd, int* out) {
  int o;
  if (g.transpose) {
    o = in * g.stride[d] - g.pad[d] + kd * g.dil[d];
  } else {
    int dc = in + g.pad[d] - kd * g.dil[d];
    if (dc < 0) return false;  // would map to a negative output coordinate or fail the divisibility test
    const int st = g.stride[d];
    if (st == 1) {
      o = dc;
    } else if (st == 2) {  // the common strides need no integer division
      if (dc & 1) return false;
      o = dc >> 1;
    } else {
      if (dc % st != 0) return false;
      o = dc / st;
    }
  }
  *out = o;
  return o >= 0 && o < g.shape[d + 1];
}

// Resolve the leading (all but fastest) taps of kernel row `row`; returns false when the row is out of range
// for this input. *prefix receives the packed key of the leading coordinates.
__device__ __forceinline__ bool row_prefix(const Geometry& g, const int* c, int row, uint32_t* prefix) {
  if (c[0] < 0 || c[0] >= g.shape[0]) return false;
  int taps[D3D_MAX_NDIM];
  int rem = row;
  for (int d = g.ndim - 2; d >= 0; --d) {
    taps[d] = rem % g.ksize[d];
    rem /= g.ksize[d];
  }
  uint32_t key = (uint32_t)c[0];
  for (int d = 0; d < g.ndim - 1; ++d) {
    int o;
    if (!out_coord(g, d, c[d + 1], taps[d], &o)) return false;
    key = key * (uint32_t)g.shape[d + 1] + (uint32_t)o;
  }
  *prefix = key;
  return true;
}

__device__ __forceinline__ void decode_key(const Geometry& g, uint32_t key, int32_t* out) {
  for (int d = g.ndim; d >= 1; --d) {
    out[d] = (int32_t)(key % (uint32_t)g.shape[d]);
    key /= (uint32_t)g.shape[d];
  }
  out[0] = (int32_t)key;
}

__device__ __forceinline__ int live_count(const int32_t* num_act_in, int64_t n_max) {
  int n = *num_act_in;
  n = n < 0 ? 0 : n;
  return n > n_max ? (int)n_max : n;
}

// ---------------------------------------------------------------------------------------------
__global__ void reset_table_kernel(unsigned long long* table, const int32_t* num_act_in, int64_t n_max, int fan,
                                   uint32_t cap_max, int32_t* __restrict__ state) {
  if (blockIdx.x == 0 && threadIdx.x == 0) state[2] = 0;  // the ticket of this call's segment_scan_kernel
  uint32_t cap = hash_capacity((long long)live_count(num_act_in, n_max) * fan, cap_max);
  ulonglong2* t2 = reinterpret_cast<ulonglong2*>(table);
  for (uint32_t s = blockIdx.x * blockDim.x + threadIdx.x; s < cap / 2; s += gridDim.x * blockDim.x)
    t2[s] = make_ulonglong2(kEmptySlot, kEmptySlot);
}

__global__ void subm_insert_kernel(unsigned long long* table, const int32_t* __restrict__ coors,
                                   const int32_t* num_act_in, int64_t n_max, Geometry g, uint32_t cap_max,
                                   int32_t* status) {
  int n = live_count(num_act_in, n_max);
  uint32_t mask = hash_capacity((long long)n * kSubmFan, cap_max) - 1;
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int c[D3D_MAX_NDIM + 1];
  load_coor(coors, g.ndim, i, c);
  uint32_t key = 0;
  for (int d = 0; d <= g.ndim; ++d) {
    if (c[d] < 0 || c[d] >= g.shape[d]) return;
    key = key * (uint32_t)g.shape[d] + (uint32_t)c[d];
  }
  if (hash_insert_min_claim_first(table, mask, key, (uint32_t)i) == 0xFFFFFFFFu)
    report_status(status, D3D_STATUS_HASH_FULL);
}

// SubM probe: pair_out[k][i] = id of the active voxel at (coor_i + pad - k*dil), or -1 (trt/spconv/index.cu:48-84).
// CTA (x = input block, y = kernel row); also emits the number of hits per (k, input block).
__global__ void subm_probe_kernel(const unsigned long long* __restrict__ table, const int32_t* __restrict__ coors,
                                  const int32_t* num_act_in, int64_t n_max, Geometry g, uint32_t cap_max,
                                  int32_t* __restrict__ pair_out, int32_t* __restrict__ block_counts, int nblk) {
  constexpr int kBatch = 4;  // lookups in flight per thread
  __shared__ int cnt[kBatch];
  int n = live_count(num_act_in, n_max);
  if ((int64_t)blockIdx.x * kIdxThreads >= n) return;
  uint32_t mask = hash_capacity((long long)n * kSubmFan, cap_max) - 1;
  int row = blockIdx.y;
  int i = blockIdx.x * kIdxThreads + threadIdx.x;
  int c[D3D_MAX_NDIM + 1];
  uint32_t prefix = 0;
  bool row_ok = false;
  if (i < n) {
    load_coor(coors, g.ndim, i, c);
    row_ok = row_prefix(g, c, row, &prefix);
  }
  int dl = g.ndim - 1;
  for (int kl0 = 0; kl0 < g.klast; kl0 += kBatch) {
    if (threadIdx.x < kBatch) cnt[threadIdx.x] = 0;
    __syncthreads();
    int v[kBatch];
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {  // independent probes: their memory latencies overlap
      int o;
      v[b] = -1;
      if (kl0 + b < g.klast && row_ok && out_coord(g, dl, c[dl + 1], kl0 + b, &o))
        v[b] = hash_lookup(table, mask, prefix * (uint32_t)g.shape[dl + 1] + (uint32_t)o);
    }
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      if (kl0 + b < g.klast) {
        int k = row * g.klast + kl0 + b;
        if (i < n) pair_out[(int64_t)k * n_max + i] = v[b];
        unsigned hits = __ballot_sync(0xffffffffu, v[b] >= 0);
        if (lane_id() == 0 && hits) atomicAdd(&cnt[b], __popc(hits));
      }
    }
    __syncthreads();
    if (threadIdx.x < kBatch && kl0 + threadIdx.x < g.klast)
      block_counts[(int64_t)(row * g.klast + kl0 + threadIdx.x) * nblk + blockIdx.x] = cnt[threadIdx.x];
    __syncthreads();
  }
}

// 3-D specialisation of the SubM probe, same outputs.  One thread per input voxel walks all kernel offsets with
// its coordinates in registers; the probes of one kernel row are independent loads in flight together, and the
// per-(offset, CTA) counts are collected in shared memory with a single barrier at the end.
// kPlane3x3: the two trailing kernel extents are 3 x 3 (the usual case); the nine probes of a leading tap are
// then issued together.
// With `nbr` != null (a mirror-symmetric rulebook: odd kernel, padding = dilation * (k - 1) / 2 on every axis) the
// kernel also writes the output-stationary neighbour table SPConvMM consumes, [tile of 128 outputs][kvol][128]: the
// voxel found for offset k is, read the other way round, the input that feeds voxel i through offset kvol - 1 - k,
// so thread i fills its own column of the table -- coalesced stores, no scatter pass, no fill pass.  The ballot of
// a warp over "neighbour found" is at once the row mask of its 32 rows under that offset (`nbr_rows`, four words
// per (tile, offset)); the per-tile offset masks are collected with shared-memory atomics.  `nbr_tiles` = tiles
// the table holds.
template <bool kPlane3x3>
__global__ void __launch_bounds__(kIdxThreads, 4)
subm_probe3_kernel(const unsigned long long* __restrict__ table, const int32_t* __restrict__ coors,
                   const int32_t* num_act_in, int64_t n_max, Geometry g, uint32_t cap_max,
                   int32_t* __restrict__ pair_out, int32_t* __restrict__ block_counts, int nblk,
                   int32_t* __restrict__ nbr, uint32_t* __restrict__ nbr_mask, uint32_t* __restrict__ nbr_rows,
                   int32_t* __restrict__ nbr_perm, int64_t nbr_tiles) {
  constexpr int kBatch = 4;  // probes in flight per thread
  constexpr int kTilesPerCta = kIdxThreads / 128;
  __shared__ int cnt[kMaxKernelVol];
  __shared__ unsigned tile_bits[kTilesPerCta];
  const int n = live_count(num_act_in, n_max);
  const int64_t tile0 = (int64_t)blockIdx.x * kTilesPerCta;
  if (nbr && tile0 + (threadIdx.x >> 7) < nbr_tiles) {  // tile row p of the table stands for output p
    const int64_t pos = (int64_t)blockIdx.x * kIdxThreads + threadIdx.x;
    nbr_perm[pos] = pos < n_max ? (int32_t)pos : -1;
  }
  if ((int64_t)blockIdx.x * kIdxThreads >= n) {
    // no live voxel here: the tiles of this CTA take part in no offset and hold no neighbour
    if (nbr) {
      if (threadIdx.x < kTilesPerCta && tile0 + threadIdx.x < nbr_tiles) nbr_mask[tile0 + threadIdx.x] = 0u;
      const int64_t tile = tile0 + (threadIdx.x >> 7);
      if (tile < nbr_tiles) {
        // (the ids of rows without an input are never read: only the row masks need a value)
        for (int w = threadIdx.x & 127; w < g.kvol * 4; w += 128) nbr_rows[tile * g.kvol * 4 + w] = 0u;
      }
    }
    return;
  }
  for (int t = threadIdx.x; t < g.kvol; t += kIdxThreads) cnt[t] = 0;
  if (threadIdx.x < kTilesPerCta) tile_bits[threadIdx.x] = 0u;
  __syncthreads();
  const int my_tile = threadIdx.x >> 7;
  // this thread's column of the table: entry of offset k' at nbr_col[k' * 128]
  int32_t* nbr_col = nullptr;
  uint32_t* rows_word = nullptr;  // this warp's word of the row masks: entry of offset k' at rows_word[k' * 4]
  if (nbr && tile0 + my_tile < nbr_tiles) {
    nbr_col = nbr + ((tile0 + my_tile) * g.kvol) * 128 + (threadIdx.x & 127);
    rows_word = nbr_rows + ((tile0 + my_tile) * g.kvol) * 4 + ((threadIdx.x >> 5) & 3);
  }
  const uint32_t mask = hash_capacity((long long)n * kSubmFan, cap_max) - 1;
  const int i = blockIdx.x * kIdxThreads + threadIdx.x;
  const bool live = i < n;
  int4 c = make_int4(-1, 0, 0, 0);
  if (live) c = __ldg(reinterpret_cast<const int4*>(coors) + i);
  const bool batch_ok = live && c.x >= 0 && c.x < g.shape[0];
  // SubM: stride 1, never transposed, so the neighbour along d is c_d + pad_d - k_d * dil_d (geometry.h:41-49 with
  // stride 1) and its key differs from the key of (c + pad) by a per-offset constant: no division per probe.
  const int b0 = c.y + g.pad[0], b1 = c.z + g.pad[1], b2 = c.w + g.pad[2];
  const uint32_t s1 = (uint32_t)g.shape[1], s2 = (uint32_t)g.shape[2], s3 = (uint32_t)g.shape[3];
  const uint32_t key_base = (((uint32_t)c.x * s1 + (uint32_t)b0) * s2 + (uint32_t)b1) * s3 + (uint32_t)b2;
  int k = 0;
  for (int k0 = 0; k0 < g.ksize[0]; ++k0) {
    const int o0 = b0 - k0 * g.dil[0];
    const bool ok0 = batch_ok && (uint32_t)o0 < s1;
    if (kPlane3x3) {
      int v[9];
      uint32_t key[9];
      unsigned long long first[9];
      bool probe[9];
      const uint32_t key_k0 = key_base - (uint32_t)(k0 * g.dil[0]) * s2 * s3;
#pragma unroll
      for (int b = 0; b < 9; ++b) {  // first probes of the whole plane: independent loads
        const int k1 = b / 3, k2 = b % 3;
        const int o1 = b1 - k1 * g.dil[1], o2 = b2 - k2 * g.dil[2];
        probe[b] = ok0 && (uint32_t)o1 < s2 && (uint32_t)o2 < s3;
        key[b] = key_k0 - (uint32_t)(k1 * g.dil[1]) * s3 - (uint32_t)(k2 * g.dil[2]);
        first[b] = probe[b] ? __ldg(&table[home_slot(key[b], mask)]) : kEmptySlot;
      }
      // resolve all nine in lock step: a collision moves on to its next bucket together with the other unresolved
      // probes, so the dependent-load chain is the longest probe sequence, not the sum of them
      uint32_t slot[9];
      uint32_t pending = 0;
#pragma unroll
      for (int b = 0; b < 9; ++b) {
        v[b] = -1;
        if (probe[b]) {
          if ((uint32_t)(first[b] >> 32) == key[b]) v[b] = (int32_t)(uint32_t)first[b];
          else if (first[b] != kEmptySlot) pending |= 1u << b;
        }
        slot[b] = (home_slot(key[b], mask) + 4u) & mask;
      }
      for (uint32_t round = 0; pending && round <= (mask >> 2); ++round) {
        unsigned long long cur[9];
#pragma unroll
        for (int b = 0; b < 9; ++b) cur[b] = ((pending >> b) & 1u) ? __ldg(&table[slot[b]]) : kEmptySlot;
#pragma unroll
        for (int b = 0; b < 9; ++b) {
          if ((pending >> b) & 1u) {
            if ((uint32_t)(cur[b] >> 32) == key[b]) v[b] = (int32_t)(uint32_t)cur[b], pending &= ~(1u << b);
            else if (cur[b] == kEmptySlot) pending &= ~(1u << b);
            else slot[b] = (slot[b] + 4u) & mask;
          }
        }
      }
#pragma unroll
      for (int b = 0; b < 9; ++b) {
        if (live) pair_out[(int64_t)(k + b) * n_max + i] = v[b];
        const unsigned hits = __ballot_sync(0xffffffffu, v[b] >= 0);
        if (lane_id() == 0 && hits) atomicAdd(&cnt[k + b], __popc(hits));
        if (nbr_col && v[b] >= 0) nbr_col[(g.kvol - 1 - (k + b)) * 128] = v[b];  // ids without a row-mask bit are never read
        if (rows_word && lane_id() == 0) rows_word[(g.kvol - 1 - (k + b)) * 4] = hits;
        if (nbr && lane_id() == 0 && hits) atomicOr(&tile_bits[my_tile], 1u << (g.kvol - 1 - (k + b)));
      }
      k += 9;
      continue;
    }
    for (int k1 = 0; k1 < g.ksize[1]; ++k1) {
      const int o1 = b1 - k1 * g.dil[1];
      const bool ok1 = ok0 && (uint32_t)o1 < s2;
      const uint32_t key_row = key_base - ((uint32_t)(k0 * g.dil[0]) * s2 + (uint32_t)(k1 * g.dil[1])) * s3;
      for (int k2 = 0; k2 < g.klast; k2 += kBatch) {
        int v[kBatch];
        uint32_t key[kBatch];
        unsigned long long first[kBatch];
        bool probe[kBatch];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {  // first probes of the batch: independent loads
          const int o2 = b2 - (k2 + b) * g.dil[2];
          probe[b] = ok1 && k2 + b < g.klast && (uint32_t)o2 < s3;
          key[b] = key_row - (uint32_t)((k2 + b) * g.dil[2]);
          first[b] = probe[b] ? __ldg(&table[home_slot(key[b], mask)]) : kEmptySlot;
        }
#pragma unroll
        for (int b = 0; b < kBatch; ++b) v[b] = probe[b] ? hash_lookup_resolve(table, mask, key[b], first[b]) : -1;
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
          if (k2 + b < g.klast) {
            if (live) pair_out[(int64_t)(k + b) * n_max + i] = v[b];
            const unsigned hits = __ballot_sync(0xffffffffu, v[b] >= 0);
            if (lane_id() == 0 && hits) atomicAdd(&cnt[k + b], __popc(hits));
            if (nbr_col && v[b] >= 0) nbr_col[(g.kvol - 1 - (k + b)) * 128] = v[b];  // ids without a row-mask bit are never read
            if (rows_word && lane_id() == 0) rows_word[(g.kvol - 1 - (k + b)) * 4] = hits;
            if (nbr && lane_id() == 0 && hits) atomicOr(&tile_bits[my_tile], 1u << (g.kvol - 1 - (k + b)));
          }
        }
        k += (g.klast - k2 < kBatch) ? g.klast - k2 : kBatch;
      }
    }
  }
  __syncthreads();
  for (int t = threadIdx.x; t < g.kvol; t += kIdxThreads) block_counts[(int64_t)t * nblk + blockIdx.x] = cnt[t];
  if (nbr && threadIdx.x < kTilesPerCta && tile0 + threadIdx.x < nbr_tiles)
    nbr_mask[tile0 + threadIdx.x] = tile_bits[threadIdx.x];
}

// Conv insert: every valid (input, offset) inserts its output key with value = i*kvol + k; the smallest pair id
// survives in the slot.  pair_out[k][i] receives the slot (>= 0) or -1.
__global__ void conv_insert_kernel(unsigned long long* table, const int32_t* __restrict__ coors,
                                   const int32_t* num_act_in, int64_t n_max, Geometry g, int fan, uint32_t cap_max,
                                   int32_t* __restrict__ pair_out, int32_t* status) {
  int n = live_count(num_act_in, n_max);
  if ((int64_t)blockIdx.x * kIdxThreads >= n) return;
  uint32_t mask = hash_capacity((long long)n * fan, cap_max) - 1;
  int row = blockIdx.y;
  int i = blockIdx.x * kIdxThreads + threadIdx.x;
  if (i >= n) return;
  int c[D3D_MAX_NDIM + 1];
  uint32_t prefix = 0;
  load_coor(coors, g.ndim, i, c);
  bool row_ok = row_prefix(g, c, row, &prefix);
  int dl = g.ndim - 1;
  for (int kl = 0; kl < g.klast; ++kl) {
    int k = row * g.klast + kl;
    int v = -1, o;
    if (row_ok && out_coord(g, dl, c[dl + 1], kl, &o)) {
      uint32_t slot = hash_insert_min(table, mask, prefix * (uint32_t)g.shape[dl + 1] + (uint32_t)o,
                                      (uint32_t)(i * g.kvol + k));
      v = slot == 0xFFFFFFFFu ? -1 : (int)slot;
      if (slot == 0xFFFFFFFFu) report_status(status, D3D_STATUS_HASH_FULL);
    }
    pair_out[(int64_t)k * n_max + i] = v;
  }
}

// Packed candidate list of a strided rulebook.  A forward convolution with stride s reaches an output only through
// the taps whose offset has the right remainder modulo s, so an input has at most prod(ceil(ksize / stride)) valid
// offsets (8 of 27 for the usual 3x3x3 / stride 2).  Instead of kvol entries per input, most of them -1, the strided
// path then keeps kPackedSlots entries per input, ascending by offset: entry = offset << 26 | value (a hash slot,
// later an output id; both below 2^26), -1 = unused.  Every pass over the pair table reads and writes 8 rows of it
// instead of 27; the index tensor that comes out is the same.
constexpr int kPackedSlots = 8;
constexpr int kPackedShift = 26;
constexpr int kPackedValueMask = (1 << kPackedShift) - 1;
__device__ __forceinline__ int pack_entry(int k, int v) { return (k << kPackedShift) | v; }
__device__ __forceinline__ int entry_offset(int e) { return e >> kPackedShift; }
__device__ __forceinline__ int entry_value(int e) { return e & kPackedValueMask; }

// 3-D specialisation for kernels of at most 3 taps per axis, same outputs.  One thread per input voxel: the output
// coordinate of every tap is resolved once per axis (3 + 3 + 3 small computations, the only divisions), then the
// offsets are walked with those in registers; only the combinations valid on all three axes touch the hash table.
template <bool kPacked>
__global__ void __launch_bounds__(kIdxThreads)
conv_insert3_kernel(unsigned long long* table, const int32_t* __restrict__ coors, const int32_t* num_act_in,
                    int64_t n_max, Geometry g, int fan, uint32_t cap_max, int32_t* __restrict__ pair_out,
                    int32_t* status) {
  constexpr bool kPacked_ = kPacked;
  const int n = live_count(num_act_in, n_max);
  const int i = blockIdx.x * kIdxThreads + threadIdx.x;
  if (i >= n) return;
  const uint32_t mask = hash_capacity((long long)n * fan, cap_max) - 1;
  const int4 c = __ldg(reinterpret_cast<const int4*>(coors) + i);
  const bool batch_ok = c.x >= 0 && c.x < g.shape[0];
  int o0[3], o1[3], o2[3];  // output coordinate per tap, -1 = this tap reaches no output
#pragma unroll
  for (int t = 0; t < 3; ++t) {
    int o;
    o0[t] = (t < g.ksize[0] && out_coord(g, 0, c.y, t, &o)) ? o : -1;
    o1[t] = (t < g.ksize[1] && out_coord(g, 1, c.z, t, &o)) ? o : -1;
    o2[t] = (t < g.ksize[2] && out_coord(g, 2, c.w, t, &o)) ? o : -1;
  }
  const uint32_t s1 = (uint32_t)g.shape[1], s2 = (uint32_t)g.shape[2], s3 = (uint32_t)g.shape[3];
  const uint32_t pair_base = (uint32_t)(i * g.kvol);
  int filled = 0;  // packed form: entries written so far
#pragma unroll
  for (int k0 = 0; k0 < 3; ++k0) {
#pragma unroll
    for (int k1 = 0; k1 < 3; ++k1) {
#pragma unroll
      for (int k2 = 0; k2 < 3; ++k2) {
        if (k0 < g.ksize[0] && k1 < g.ksize[1] && k2 < g.ksize[2]) {
          const int k = (k0 * g.ksize[1] + k1) * g.ksize[2] + k2;
          int v = -1;
          if (batch_ok && o0[k0] >= 0 && o1[k1] >= 0 && o2[k2] >= 0) {
            const uint32_t key = (((uint32_t)c.x * s1 + (uint32_t)o0[k0]) * s2 + (uint32_t)o1[k1]) * s3 + (uint32_t)o2[k2];
            const uint32_t slot = hash_insert_min_claim_first(table, mask, key, pair_base + (uint32_t)k);
            v = slot == 0xFFFFFFFFu ? -1 : (int)slot;
            if (slot == 0xFFFFFFFFu) report_status(status, D3D_STATUS_HASH_FULL);
          }
          if (!kPacked_) {
            pair_out[(int64_t)k * n_max + i] = v;
          } else if (v >= 0 && filled < kPackedSlots) {
            pair_out[(int64_t)filled * n_max + i] = pack_entry(k, v);
            ++filled;
          }
        }
      }
    }
  }
  if (kPacked_)
    for (; filled < kPackedSlots; ++filled) pair_out[(int64_t)filled * n_max + i] = -1;
}

// A pair "wins" its output voxel when its id is the one left in the slot.
__device__ __forceinline__ bool is_winner(const unsigned long long* table, int slot, uint32_t pair_id) {
  return slot >= 0 && (uint32_t)table[slot] == pair_id;
}

// Bit k of the result: pair (i, k) wins.  Loads are issued nine offsets at a time (two dependent gathers each).
// Valid for kvol <= 32.
__device__ __forceinline__ uint32_t winner_bits(const unsigned long long* __restrict__ table,
                                                const int32_t* __restrict__ pair_out, int64_t n_max, int kvol,
                                                int i) {
  constexpr int kBatch = 9;
  uint32_t bits = 0;
  for (int k0 = 0; k0 < kvol; k0 += kBatch) {
    int slot[kBatch];
    unsigned long long cur[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) slot[j] = k0 + j < kvol ? __ldg(pair_out + (int64_t)(k0 + j) * n_max + i) : -1;
#pragma unroll
    for (int j = 0; j < kBatch; ++j) cur[j] = slot[j] >= 0 ? __ldg(table + slot[j]) : kEmptySlot;
#pragma unroll
    for (int j = 0; j < kBatch; ++j)
      if (slot[j] >= 0 && (uint32_t)cur[j] == (uint32_t)(i * kvol + k0 + j)) bits |= 1u << (k0 + j);
  }
  return bits;
}

// Packed form of the same test: bit j of the result = entry j of input i wins its output voxel.
__device__ __forceinline__ uint32_t winner_bits_packed(const unsigned long long* __restrict__ table,
                                                       const int32_t* __restrict__ pair_out, int64_t n_max, int kvol,
                                                       int i) {
  int e[kPackedSlots];
  unsigned long long cur[kPackedSlots];
#pragma unroll
  for (int j = 0; j < kPackedSlots; ++j) e[j] = __ldg(pair_out + (int64_t)j * n_max + i);
#pragma unroll
  for (int j = 0; j < kPackedSlots; ++j) cur[j] = e[j] >= 0 ? __ldg(table + entry_value(e[j])) : kEmptySlot;
  uint32_t bits = 0;
#pragma unroll
  for (int j = 0; j < kPackedSlots; ++j)
    if (e[j] >= 0 && (uint32_t)cur[j] == (uint32_t)(i * kvol + entry_offset(e[j]))) bits |= 1u << j;
  return bits;
}

__global__ void conv_count_winners_kernel(const unsigned long long* __restrict__ table,
                                          const int32_t* __restrict__ pair_out, const int32_t* num_act_in,
                                          int64_t n_max, int kvol, bool packed, int32_t* __restrict__ winners,
                                          uint32_t* __restrict__ win_bits) {
  __shared__ int scratch[40];
  int n = live_count(num_act_in, n_max);
  int i = blockIdx.x * kIdxThreads + threadIdx.x;
  int cnt = 0;
  if (i < n) {
    if (kvol <= 32) {
      const uint32_t bits = packed ? winner_bits_packed(table, pair_out, n_max, kvol, i)
                                   : winner_bits(table, pair_out, n_max, kvol, i);
      win_bits[i] = bits;  // kept for the numbering pass: it needs the same two dependent gathers per offset
      cnt = __popc(bits);
    } else
      for (int k = 0; k < kvol; ++k)
        cnt += is_winner(table, pair_out[(int64_t)k * n_max + i], (uint32_t)(i * kvol + k));
  }
  int total;
  block_exclusive_scan(cnt, scratch, &total);
  if (threadIdx.x == 0) winners[blockIdx.x] = total;
}

// Number the output voxels in pair-id order and write their coordinates (index.cu:104-121).
__global__ void conv_assign_kernel(const unsigned long long* __restrict__ table, const int32_t* __restrict__ pair_out,
                                   const int32_t* num_act_in, int64_t n_max, Geometry g,
                                   const int32_t* __restrict__ winners_base,
                                   const uint32_t* __restrict__ win_bits, int32_t max_out, bool packed,
                                   int32_t* __restrict__ slot_out, int32_t* __restrict__ out_coors) {
  __shared__ int scratch[40];
  int n = live_count(num_act_in, n_max);
  if ((int64_t)blockIdx.x * kIdxThreads >= n) return;
  int i = blockIdx.x * kIdxThreads + threadIdx.x;
  int cnt = 0;
  uint32_t bits = 0;
  const bool small = g.kvol <= 32;
  if (i < n) {
    if (small) {
      bits = win_bits[i];
      cnt = __popc(bits);
    } else {
      for (int k = 0; k < g.kvol; ++k)
        cnt += is_winner(table, pair_out[(int64_t)k * n_max + i], (uint32_t)(i * g.kvol + k));
    }
  }
  int total;
  int id = winners_base[blockIdx.x] + block_exclusive_scan(cnt, scratch, &total);
  if (i >= n || cnt == 0) return;
  if (packed) {
    // the bits run over the entries of the input (ascending by offset, so the numbering is the same): all entries,
    // then all keys of the winning ones (independent gathers), then the writes
    int slot[kPackedSlots];
    unsigned long long kv[kPackedSlots];
#pragma unroll
    for (int j = 0; j < kPackedSlots; ++j)
      slot[j] = ((bits >> j) & 1u) ? entry_value(__ldg(pair_out + (int64_t)j * n_max + i)) : -1;
#pragma unroll
    for (int j = 0; j < kPackedSlots; ++j) kv[j] = slot[j] >= 0 ? __ldg(table + slot[j]) : 0ull;
#pragma unroll
    for (int j = 0; j < kPackedSlots; ++j) {
      if (slot[j] < 0) continue;
      if (id < max_out) {
        slot_out[slot[j]] = id;
        int32_t oc[D3D_MAX_NDIM + 1];
        decode_key(g, (uint32_t)(kv[j] >> 32), oc);
        for (int d = 0; d <= g.ndim; ++d) out_coors[(int64_t)id * (g.ndim + 1) + d] = oc[d];
      } else {
        slot_out[slot[j]] = -1;  // beyond maxNumActOut: the pair is dropped (index.cu:158-172)
      }
      ++id;
    }
    return;
  }
  const int steps = g.kvol;
  for (int k = 0; k < steps; ++k) {
    if (small && !((bits >> k) & 1u)) continue;
    const int slot = pair_out[(int64_t)k * n_max + i];
    if (!small && !is_winner(table, slot, (uint32_t)(i * g.kvol + k))) continue;
    if (id < max_out) {
      slot_out[slot] = id;
      int32_t oc[D3D_MAX_NDIM + 1];
      decode_key(g, (uint32_t)(table[slot] >> 32), oc);
      for (int d = 0; d <= g.ndim; ++d) out_coors[(int64_t)id * (g.ndim + 1) + d] = oc[d];
    } else {
      slot_out[slot] = -1;  // beyond maxNumActOut: the pair is dropped (index.cu:158-172)
    }
    ++id;
  }
}

// pair_out: slot -> output id; per-(k, input block) hit counts.  One CTA per input block walks all offsets
// (kvol <= kMaxKernelVol) with nine gathers in flight per thread and a single barrier.
__global__ void __launch_bounds__(kIdxThreads)
conv_translate_all_kernel(int32_t* __restrict__ pair_out, const int32_t* __restrict__ slot_out,
                          const int32_t* num_act_in, int64_t n_max, int kvol, int32_t* __restrict__ block_counts,
                          int nblk) {
  constexpr int kBatch = 9;
  __shared__ int cnt[kMaxKernelVol];
  const int n = live_count(num_act_in, n_max);
  if ((int64_t)blockIdx.x * kIdxThreads >= n) return;
  for (int t = threadIdx.x; t < kvol; t += kIdxThreads) cnt[t] = 0;
  __syncthreads();
  const int i = blockIdx.x * kIdxThreads + threadIdx.x;
  for (int k0 = 0; k0 < kvol; k0 += kBatch) {
    int v[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) v[j] = (i < n && k0 + j < kvol) ? pair_out[(int64_t)(k0 + j) * n_max + i] : -1;
#pragma unroll
    for (int j = 0; j < kBatch; ++j) v[j] = v[j] >= 0 ? __ldg(slot_out + v[j]) : -1;
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (k0 + j < kvol) {
        if (i < n) pair_out[(int64_t)(k0 + j) * n_max + i] = v[j];
        const unsigned hits = __ballot_sync(0xffffffffu, v[j] >= 0);
        if (lane_id() == 0 && hits) atomicAdd(&cnt[k0 + j], __popc(hits));
      }
    }
  }
  __syncthreads();
  for (int t = threadIdx.x; t < kvol; t += kIdxThreads) block_counts[(int64_t)t * nblk + blockIdx.x] = cnt[t];
}

// Packed form: entries keep their offset, the value becomes the output id (or the entry becomes -1 when the output
// voxel fell beyond maxNumActOut); the per-(offset, input block) counts are collected with shared-memory atomics.
__global__ void __launch_bounds__(kIdxThreads)
conv_translate_packed_kernel(int32_t* __restrict__ pair_out, const int32_t* __restrict__ slot_out,
                             const int32_t* num_act_in, int64_t n_max, int kvol, int32_t* __restrict__ block_counts,
                             int nblk) {
  __shared__ int cnt[kMaxKernelVol];
  const int n = live_count(num_act_in, n_max);
  if ((int64_t)blockIdx.x * kIdxThreads >= n) return;
  for (int t = threadIdx.x; t < kvol; t += kIdxThreads) cnt[t] = 0;
  __syncthreads();
  const int i = blockIdx.x * kIdxThreads + threadIdx.x;
  if (i < n) {
    int e[kPackedSlots], id[kPackedSlots];
#pragma unroll
    for (int j = 0; j < kPackedSlots; ++j) e[j] = pair_out[(int64_t)j * n_max + i];
#pragma unroll
    for (int j = 0; j < kPackedSlots; ++j) id[j] = e[j] >= 0 ? __ldg(slot_out + entry_value(e[j])) : -1;
#pragma unroll
    for (int j = 0; j < kPackedSlots; ++j) {
      if (e[j] < 0) continue;  // entries are dense from the front, but -1 is written once and stays
      const int k = entry_offset(e[j]);
      pair_out[(int64_t)j * n_max + i] = id[j] >= 0 ? pack_entry(k, id[j]) : -1;
      if (id[j] >= 0) atomicAdd(&cnt[k], 1);
    }
  }
  __syncthreads();
  for (int t = threadIdx.x; t < kvol; t += kIdxThreads) block_counts[(int64_t)t * nblk + blockIdx.x] = cnt[t];
}

// One CTA of 1024 threads per kernel offset: an exclusive scan of the offset's per-CTA counts, in place; the CTA that
// finishes last (a ticket in `state[2]`, which reset_table_kernel zeroes at the start of every call) then produces
// the segment starts (each rounded up to 128, trt/spconv/index.cu:148-156) and numIndex (index.cu:139-144).
// seg[0..kvol] = start of each segment (seg[kvol] = numIndex), seg[kvol+1 .. 2*kvol] = pair count of each offset.
// `state` (words kept in the workspace between calls): [0] where the padding fill of this call ends, [1] the
// num_index of this call.  A caller that owns the index buffer across calls (`persistent`) and did not pass
// `first` gets only [num_index, previous num_index) refilled: everything beyond is still -1 from earlier calls.
__global__ void __launch_bounds__(1024) segment_scan_kernel(int32_t* __restrict__ block_counts, int nblk, int kvol,
                                                            const int32_t* num_act_in, int64_t n_max,
                                                            int32_t* __restrict__ seg, int32_t* num_index,
                                                            int32_t* __restrict__ state, int persistent, int first,
                                                            int64_t row_len) {
  __shared__ int warp_sum[32];
  __shared__ int carry_s, chunk_total;
  __shared__ bool last;
  const int n = live_count(num_act_in, n_max);
  const int live_blk = (n + kIdxThreads - 1) / kIdxThreads;
  const int warp = threadIdx.x >> 5, lane = lane_id();
  const int k = blockIdx.x;
  int32_t* row = block_counts + (int64_t)k * nblk;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < live_blk; base += 1024) {  // 1024 counts at a time
    const int j = base + (int)threadIdx.x;
    const int v = j < live_blk ? row[j] : 0;
    int inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, inc, d);
      if (lane >= d) inc += t;
    }
    if (lane == 31) warp_sum[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      const int w = warp_sum[lane];
      int winc = w;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, winc, d);
        if (lane >= d) winc += t;
      }
      warp_sum[lane] = winc - w;  // exclusive over the warps
      if (lane == 31) chunk_total = winc;
    }
    __syncthreads();
    const int carry = carry_s;
    if (j < live_blk) row[j] = carry + warp_sum[warp] + inc - v;
    __syncthreads();  // everyone has read the carry and the warp offsets
    if (threadIdx.x == 0) carry_s = carry + chunk_total;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    seg[kvol + 1 + k] = carry_s;
    __threadfence();
    last = atomicAdd(&state[2], 1) == kvol - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  // the other CTAs' totals: loaded side by side (one after the other they would cost a round trip to L2 each)
  __shared__ int counts[kMaxKernelVol];
  const volatile int32_t* totals = seg + kvol + 1;
  for (int q = threadIdx.x; q < kvol; q += blockDim.x) counts[q] = totals[q];
  __syncthreads();
  if (threadIdx.x != 0) return;
  int pos = 0;
  for (int q = 0; q < kvol; ++q) {
    seg[q] = pos;
    pos += (counts[q] + kSegment - 1) / kSegment * kSegment;
  }
  seg[kvol] = pos;
  *num_index = pos;
  const int64_t prev = state[1];
  const bool partial = persistent && !first && prev >= 0 && prev <= row_len;
  state[0] = (int32_t)(partial ? (prev > pos ? prev : pos) : row_len);
  state[1] = pos;
  state[2] = 0;
}

// Write the compacted (gatherIn, scatterOut, kernelOffset) triples (trt/spconv/index.cu:123-146).
__global__ void compact_kernel(const int32_t* __restrict__ pair_out, const int32_t* __restrict__ block_prefix,
                               const int32_t* __restrict__ seg, const int32_t* num_act_in, int64_t n_max, int nblk,
                               int32_t* __restrict__ index, int64_t row_len) {
  __shared__ int warp_off[kIdxThreads / 32 + 1];
  int n = live_count(num_act_in, n_max);
  if ((int64_t)blockIdx.x * kIdxThreads >= n) return;
  int k = blockIdx.y;
  int i = blockIdx.x * kIdxThreads + threadIdx.x;
  int v = i < n ? pair_out[(int64_t)k * n_max + i] : -1;
  unsigned hits = __ballot_sync(0xffffffffu, v >= 0);
  int warp = threadIdx.x >> 5;
  if (lane_id() == 0) warp_off[warp + 1] = __popc(hits);
  __syncthreads();
  if (threadIdx.x == 0) {
    warp_off[0] = 0;
    for (int w = 1; w <= kIdxThreads / 32; ++w) warp_off[w] += warp_off[w - 1];
  }
  __syncthreads();
  if (v < 0) return;
  int64_t pos = (int64_t)seg[k] + block_prefix[(int64_t)k * nblk + blockIdx.x] + warp_off[warp] +
                __popc(hits & lanemask_lt());
  if (pos >= row_len) return;
  index[pos] = i;
  index[row_len + pos] = v;
  index[2 * row_len + pos] = k;
}

// Same result for small kernels (kvol <= kCompactAllMaxVol): one CTA per input block walks all offsets, with a
// single barrier between counting and writing instead of two per (block, offset).
constexpr int kCompactAllMaxVol = 64;
constexpr int kCompactHeld = 27;  // kernel volumes up to 3 x 3 x 3 keep an input's entries in registers
template <bool kHold>
__global__ void __launch_bounds__(kIdxThreads)
compact_all_kernel(const int32_t* __restrict__ pair_out, const int32_t* __restrict__ block_prefix,
                   const int32_t* __restrict__ seg, const int32_t* num_act_in, int64_t n_max, int nblk, int kvol,
                   int32_t* __restrict__ index, int64_t row_len) {
  constexpr int kWarps = kIdxThreads / 32;
  __shared__ int warp_cnt[kCompactAllMaxVol][kWarps];
  const int n = live_count(num_act_in, n_max);
  if ((int64_t)blockIdx.x * kIdxThreads >= n) return;
  constexpr int kBatch = 9;  // loads in flight per thread
  const int i = blockIdx.x * kIdxThreads + threadIdx.x;
  const int warp = threadIdx.x >> 5;
  int held[kHold ? kCompactHeld : 1];
  if (kHold) {  // one read of the pair table: all loads first, then the ballots
#pragma unroll
    for (int k = 0; k < kCompactHeld; ++k)
      held[k] = (i < n && k < kvol) ? __ldg(pair_out + (int64_t)k * n_max + i) : -1;
#pragma unroll
    for (int k = 0; k < kCompactHeld; ++k) {
      const unsigned hits = __ballot_sync(0xffffffffu, held[k] >= 0);
      if (lane_id() == 0 && k < kvol) warp_cnt[k][warp] = __popc(hits);
    }
  } else {
    for (int k0 = 0; k0 < kvol; k0 += kBatch) {
      int v[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j)
        v[j] = (i < n && k0 + j < kvol) ? __ldg(pair_out + (int64_t)(k0 + j) * n_max + i) : -1;
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const unsigned hits = __ballot_sync(0xffffffffu, v[j] >= 0);
        if (lane_id() == 0 && k0 + j < kvol) warp_cnt[k0 + j][warp] = __popc(hits);
      }
    }
  }
  __syncthreads();
  // counts -> first output position of every (offset, warp) of this CTA
  if (threadIdx.x < kvol) {
    const int k = threadIdx.x;
    int pos = seg[k] + block_prefix[(int64_t)k * nblk + blockIdx.x];
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const int c = warp_cnt[k][w];
      warp_cnt[k][w] = pos;
      pos += c;
    }
  }
  __syncthreads();
  auto put = [&](int k, int v) {
    const unsigned hits = __ballot_sync(0xffffffffu, v >= 0);
    if (v >= 0) {
      const int64_t pos = (int64_t)warp_cnt[k][warp] + __popc(hits & lanemask_lt());
      if (pos < row_len) {
        index[pos] = i;
        index[row_len + pos] = v;
        index[2 * row_len + pos] = k;
      }
    }
  };
  if (kHold) {
#pragma unroll
    for (int k = 0; k < kCompactHeld; ++k)
      if (k < kvol) put(k, held[k]);  // warp-uniform condition
  } else {
    for (int k0 = 0; k0 < kvol; k0 += kBatch) {
      int v[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j)
        v[j] = (i < n && k0 + j < kvol) ? __ldg(pair_out + (int64_t)(k0 + j) * n_max + i) : -1;
#pragma unroll
      for (int j = 0; j < kBatch; ++j)
        if (k0 + j < kvol) put(k0 + j, v[j]);
    }
  }
}

// compact_all_kernel for the packed pair table (kvol <= 32): the entries of an input sit in registers; for every
// offset a ballot of the lanes that hold it gives the position inside the segment, ascending by input index.
__global__ void __launch_bounds__(kIdxThreads)
compact_packed_kernel(const int32_t* __restrict__ pair_out, const int32_t* __restrict__ block_prefix,
                      const int32_t* __restrict__ seg, const int32_t* num_act_in, int64_t n_max, int nblk, int kvol,
                      int32_t* __restrict__ index, int64_t row_len) {
  constexpr int kWarps = kIdxThreads / 32;
  __shared__ int warp_cnt[32][kWarps];
  const int n = live_count(num_act_in, n_max);
  if ((int64_t)blockIdx.x * kIdxThreads >= n) return;
  const int i = blockIdx.x * kIdxThreads + threadIdx.x;
  const int warp = threadIdx.x >> 5;
  __shared__ int value_of[32][kIdxThreads];  // [offset][thread]: the output id this input pairs with at that offset
  uint32_t kmask = 0;                        // offsets this input holds
#pragma unroll
  for (int j = 0; j < kPackedSlots; ++j) {
    const int e = i < n ? __ldg(pair_out + (int64_t)j * n_max + i) : -1;
    if (e >= 0) {
      kmask |= 1u << entry_offset(e);
      value_of[entry_offset(e)][threadIdx.x] = entry_value(e);
    }
  }
  for (int k = 0; k < kvol; ++k) {
    const unsigned hits = __ballot_sync(0xffffffffu, (kmask >> k) & 1u);
    if (lane_id() == 0) warp_cnt[k][warp] = __popc(hits);
  }
  __syncthreads();
  if (threadIdx.x < kvol) {
    const int k = threadIdx.x;
    int pos = seg[k] + block_prefix[(int64_t)k * nblk + blockIdx.x];
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const int c = warp_cnt[k][w];
      warp_cnt[k][w] = pos;
      pos += c;
    }
  }
  __syncthreads();
  for (int k = 0; k < kvol; ++k) {
    const bool has = (kmask >> k) & 1u;
    const unsigned hits = __ballot_sync(0xffffffffu, has);
    if (!has) continue;
    const int v = value_of[k][threadIdx.x];  // written by this thread above
    const int64_t pos = (int64_t)warp_cnt[k][warp] + __popc(hits & lanemask_lt());
    if (pos < row_len) {
      index[pos] = i;
      index[row_len + pos] = v;
      index[2 * row_len + pos] = k;
    }
  }
}

// Everything that is not a pair is -1: the unused tail of each 128-aligned segment and the rows beyond
// numIndex (the reference memsets the three rows beforehand, trt/spconv/index.cu:352-354).
__global__ void fill_padding_kernel(const int32_t* __restrict__ seg, int kvol, int32_t* __restrict__ index,
                                    int64_t row_len, const int32_t* __restrict__ state) {
  int num_index = seg[kvol];
  const int64_t fill_end = state[0];  // row_len, or where the previous rulebook in this buffer ended
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  // in-segment padding: at most 127 entries per offset
  for (int64_t t = tid; t < (int64_t)kvol * kSegment; t += nthreads) {
    int k = (int)(t / kSegment), j = (int)(t % kSegment);
    int64_t pos = (int64_t)seg[k] + seg[kvol + 1 + k] + j;
    if (pos < seg[k + 1] && pos < row_len) {
      index[pos] = -1;
      index[row_len + pos] = -1;
      index[2 * row_len + pos] = -1;
    }
  }
  // tail of the three rows; num_index is a multiple of 128, so 16-byte stores work whenever the rows themselves
  // start 16-byte aligned
  const int64_t tail = fill_end - num_index;  // both multiples of 128
  if (tail <= 0) return;
  if ((row_len & 3) == 0 && (reinterpret_cast<uintptr_t>(index) & 15) == 0) {
    const int64_t tail4 = tail >> 2;
    const int4 fill = make_int4(-1, -1, -1, -1);
    for (int r = 0; r < 3; ++r) {
      int4* dst = reinterpret_cast<int4*>(index + r * row_len + num_index);
      int64_t p = tid;
      for (; p + 3 * nthreads < tail4; p += 4 * nthreads) {  // four independent 16-byte stores in flight
        dst[p] = fill;
        dst[p + nthreads] = fill;
        dst[p + 2 * nthreads] = fill;
        dst[p + 3 * nthreads] = fill;
      }
      for (; p < tail4; p += nthreads) dst[p] = fill;
    }
  } else {
    for (int r = 0; r < 3; ++r)
      for (int64_t p = tid; p < tail; p += nthreads) index[r * row_len + num_index + p] = -1;
  }
}

struct Plan {
  Geometry g;
  int64_t n_max;
  int64_t row_len;
  int nblk;
  int fan;
  uint32_t cap_max;
  // workspace
  unsigned long long* table;
  int32_t* pair_out;
  int32_t* block_counts;
  int32_t* seg;
  int32_t* slot_out;
  int32_t* winners;
  uint32_t* win_bits;  // per input: which of its offsets won an output voxel (kvol <= 32)
  int32_t* state;      // words that survive between calls, and the ticket of segment_scan_kernel
  bool packed;         // strided rulebook kept as kPackedSlots entries per input instead of kvol
  size_t bytes;
};

int make_plan(const d3d_spconv_index_params* p, const d3d_tensor_desc* in, int n_in, void* workspace, Plan* plan) {
  D3D_REQUIRE(p && in && n_in >= 3, D3D_ERR_INVALID_ARGUMENT);
  int ndim = p->ndim;
  D3D_REQUIRE(ndim >= 1 && ndim <= D3D_MAX_NDIM, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(in[0].nb_dims == 2 && in[0].dims[1] == ndim + 1, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(in[2].nb_dims == ndim + 2, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(in[0].dtype == D3D_INT32 && in[1].dtype == D3D_INT32, D3D_ERR_UNSUPPORTED_DTYPE);
  Geometry& g = plan->g;
  g.ndim = ndim;
  g.kvol = 1;
  g.transpose = p->transpose && !p->subm;
  for (int d = 0; d < D3D_MAX_NDIM; ++d) g.ksize[d] = g.stride[d] = g.dil[d] = 1, g.pad[d] = 0;
  int64_t fan = 1;
  for (int d = 0; d < ndim; ++d) {
    D3D_REQUIRE(p->kernel_size[d] >= 1 && p->stride[d] >= 1 && p->dilation[d] >= 1, D3D_ERR_INVALID_ARGUMENT);
    g.ksize[d] = p->kernel_size[d], g.stride[d] = p->stride[d], g.pad[d] = p->padding[d], g.dil[d] = p->dilation[d];
    g.kvol *= g.ksize[d];
    // taps that can reach an output from one input: those with the right remainder modulo the stride; when the
    // dilation shares a factor with the stride the remainders repeat sooner, so every tap is counted then
    int common = g.stride[d], rest = g.dil[d] % g.stride[d];
    while (rest) { const int t = common % rest; common = rest, rest = t; }  // gcd(stride, dilation)
    fan *= (g.transpose || common != 1) ? g.ksize[d] : (g.ksize[d] + g.stride[d] - 1) / g.stride[d];
  }
  D3D_REQUIRE(g.kvol <= kMaxKernelVol, D3D_ERR_TOO_LARGE);
  g.klast = g.ksize[ndim - 1];
  g.rows = g.kvol / g.klast;
  // key space = output spatial shape (input shape for SubM, index_trt.cu:212-226)
  int64_t vol = in[2].dims[0];
  g.shape[0] = (int)in[2].dims[0];
  for (int d = 0; d < ndim; ++d) {
    int64_t e = in[2].dims[d + 2];
    if (!p->subm) {
      if (g.transpose)
        e = (e - 1) * g.stride[d] - 2 * g.pad[d] + (g.ksize[d] - 1) * g.dil[d] + p->out_padding[d] + 1;
      else
        e = (e + 2 * g.pad[d] - g.dil[d] * (g.ksize[d] - 1) - 1) / g.stride[d] + 1;
    }
    D3D_REQUIRE(e >= 1, D3D_ERR_INVALID_ARGUMENT);
    g.shape[d + 1] = (int)e;
    vol *= e;
    D3D_REQUIRE(vol < (1ll << 31), D3D_ERR_TOO_LARGE);  // keys are 31-bit linear offsets, as in the reference
  }
  plan->n_max = in[0].dims[0];
  D3D_REQUIRE(plan->n_max >= 0 && plan->n_max * (int64_t)g.kvol < (1ll << 31), D3D_ERR_TOO_LARGE);
  plan->row_len = (int64_t)g.kvol * (plan->n_max + 128);
  plan->nblk = (int)ceil_div(plan->n_max > 0 ? plan->n_max : 1, kIdxThreads);
  plan->fan = p->subm ? kSubmFan : (int)(fan < g.kvol ? fan : g.kvol);
  size_t cap = next_pow2((size_t)(plan->n_max > 8 ? plan->n_max : 8) * plan->fan * 2);
  D3D_REQUIRE(cap <= (1ull << 30), D3D_ERR_TOO_LARGE);
  plan->cap_max = (uint32_t)(cap < 16 ? 16 : cap);
  Carver w(workspace);
  plan->table = w.take<unsigned long long>(plan->cap_max);
  plan->pair_out = w.take<int32_t>((size_t)g.kvol * (plan->n_max > 0 ? plan->n_max : 1));
  plan->block_counts = w.take<int32_t>((size_t)g.kvol * plan->nblk);
  plan->seg = w.take<int32_t>(2 * (size_t)g.kvol + 2);
  plan->slot_out = p->subm ? nullptr : w.take<int32_t>(plan->cap_max);
  plan->winners = p->subm ? nullptr : w.take<int32_t>((size_t)plan->nblk + 1);
  plan->win_bits = p->subm ? nullptr : w.take<uint32_t>((size_t)(plan->n_max > 0 ? plan->n_max : 1));
  plan->packed = !p->subm && !g.transpose && ndim == 3 && g.ksize[0] <= 3 && g.ksize[1] <= 3 && g.ksize[2] <= 3 &&
                 fan <= kPackedSlots && g.kvol > kPackedSlots /* the pair table has kvol rows */ && plan->cap_max <= (1u << kPackedShift) &&
                 p->max_num_act_out <= (1 << kPackedShift);
  plan->state = w.take<int32_t>(4);
  plan->bytes = w.off;
  return D3D_OK;
}

}  // namespace
}  // namespace d3d

using namespace d3d;

extern "C" int d3d_spconv_index_parse(int ndim, const void* data_s, size_t len, d3d_spconv_index_params* p) {
  D3D_REQUIRE(data_s && p && ndim >= 1 && ndim <= D3D_MAX_NDIM, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(len >= (size_t)(5 * ndim + 1) * 4 + 2, D3D_ERR_BAD_BLOB);
  const uint8_t* b = reinterpret_cast<const uint8_t*>(data_s);
  memset(p, 0, sizeof(*p));
  p->ndim = ndim;
  int32_t* fields[5] = {p->kernel_size, p->stride, p->padding, p->dilation, p->out_padding};
  for (int f = 0; f < 5; ++f) memcpy(fields[f], b + (size_t)f * ndim * 4, (size_t)ndim * 4);
  memcpy(&p->max_num_act_out, b + (size_t)5 * ndim * 4, 4);
  p->subm = b[(size_t)5 * ndim * 4 + 4] != 0;
  p->transpose = b[(size_t)5 * ndim * 4 + 5] != 0;
  return D3D_OK;
}

extern "C" int d3d_spconv_index_num_outputs(const d3d_spconv_index_params* p) {
  D3D_REQUIRE(p, D3D_ERR_INVALID_ARGUMENT);
  return p->subm ? 2 : 5;
}

extern "C" int d3d_spconv_index_output_desc(const d3d_spconv_index_params* p, const d3d_tensor_desc* in, int n_in,
                                            int out_index, d3d_tensor_desc* out) {
  D3D_REQUIRE(p && in && out && n_in >= 3, D3D_ERR_INVALID_ARGUMENT);
  int ndim = p->ndim;
  memset(out, 0, sizeof(*out));
  out->dtype = D3D_INT32;
  int64_t kvol = 1;
  for (int d = 0; d < ndim; ++d) kvol *= p->kernel_size[d];
  switch (out_index) {
    case 0:
      out->nb_dims = 2, out->dims[0] = 3, out->dims[1] = kvol * (in[0].dims[0] + 128);
      return D3D_OK;
    case 1:
    case 3: out->nb_dims = 1, out->dims[0] = 1; return D3D_OK;
    case 2: out->nb_dims = 2, out->dims[0] = p->max_num_act_out, out->dims[1] = ndim + 1; return D3D_OK;
    case 4:
      *out = in[2];
      for (int d = 0; d < ndim; ++d) {
        int64_t e = in[2].dims[d + 2];
        if (p->transpose)
          e = (e - 1) * p->stride[d] - 2 * p->padding[d] + (p->kernel_size[d] - 1) * p->dilation[d] +
              p->out_padding[d] + 1;
        else
          e = (e + 2 * p->padding[d] - p->dilation[d] * (p->kernel_size[d] - 1) - 1) / p->stride[d] + 1;
        out->dims[d + 2] = e;
      }
      return D3D_OK;
    default: return D3D_ERR_INVALID_ARGUMENT;
  }
}

extern "C" int d3d_spconv_index_workspace(const d3d_spconv_index_params* p, const d3d_tensor_desc* in, int n_in,
                                          size_t* bytes) {
  D3D_REQUIRE(bytes, D3D_ERR_INVALID_ARGUMENT);
  Plan plan;
  int rc = make_plan(p, in, n_in, nullptr, &plan);
  if (rc != D3D_OK) return rc;
  *bytes = plan.bytes;
  return D3D_OK;
}

extern "C" int d3d_spconv_index_enqueue(const d3d_spconv_index_params* p, const d3d_tensor_desc* in, int n_in,
                                        const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                                        void* const* outputs, void* workspace, size_t workspace_bytes, void* stream) {
  D3D_NVTX_RANGE("d3d_spconv_index_enqueue");
  return d3d_spconv_index_enqueue_ex(p, in, n_in, out, n_out, inputs, outputs, workspace, workspace_bytes, stream,
                                     nullptr);
}

extern "C" int d3d_spconv_index_subm_table_ok(const d3d_spconv_index_params* p) {
  if (!p || !p->subm || p->ndim != 3) return 0;
  for (int d = 0; d < 3; ++d)
    if (p->kernel_size[d] % 2 == 0 || p->stride[d] != 1 ||
        p->padding[d] != p->dilation[d] * (p->kernel_size[d] - 1) / 2)
      return 0;
  return 1;
}

extern "C" int d3d_spconv_index_enqueue_ex(const d3d_spconv_index_params* p, const d3d_tensor_desc* in, int n_in,
                                           const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                                           void* const* outputs, void* workspace, size_t workspace_bytes,
                                           void* stream, const d3d_spconv_index_extras* extras) {
  D3D_NVTX_RANGE("d3d_spconv_index_enqueue_ex");
  D3D_REQUIRE(inputs && outputs && out, D3D_ERR_INVALID_ARGUMENT);
  const int persistent = extras ? extras->persistent_buffers : 0;
  const int first = extras ? extras->first_call : 1;
  int32_t* nbr = extras ? reinterpret_cast<int32_t*>(extras->subm_table) : nullptr;
  int32_t* status = extras ? extras->status : nullptr;
  D3D_REQUIRE(!nbr || d3d_spconv_index_subm_table_ok(p), D3D_ERR_INVALID_ARGUMENT);
  Plan plan;
  int rc = make_plan(p, in, n_in, workspace, &plan);
  if (rc != D3D_OK) return rc;
  D3D_REQUIRE(n_out >= (p->subm ? 2 : 5), D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(workspace && workspace_bytes >= plan.bytes, D3D_ERR_WORKSPACE_TOO_SMALL);
  D3D_REQUIRE(out[0].nb_dims == 2 && out[0].dims[0] == 3 && out[0].dims[1] == plan.row_len, D3D_ERR_INVALID_ARGUMENT);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int32_t* coors = reinterpret_cast<const int32_t*>(inputs[0]);
  const int32_t* num_act_in = reinterpret_cast<const int32_t*>(inputs[1]);
  int32_t* index = reinterpret_cast<int32_t*>(outputs[0]);
  int32_t* num_index = reinterpret_cast<int32_t*>(outputs[1]);
  const Geometry& g = plan.g;
  const int64_t n_max = plan.n_max;
  if (n_max == 0) {
    cudaMemsetAsync(num_index, 0, sizeof(int32_t), st);
    if (!p->subm) cudaMemsetAsync(outputs[3], 0, sizeof(int32_t), st);
    D3D_CHECK_LAUNCH();
    return D3D_OK;
  }
  D3D_REQUIRE(coors && num_act_in && index && num_index, D3D_ERR_INVALID_ARGUMENT);
  const int nblk = plan.nblk;
  reset_table_kernel<<<stream_grid(plan.cap_max / 2, 256), 256, 0, st>>>(plan.table, num_act_in, n_max, plan.fan,
                                                                         plan.cap_max, plan.state);
  if (p->subm) {
    subm_insert_kernel<<<nblk, kIdxThreads, 0, st>>>(plan.table, coors, num_act_in, n_max, g, plan.cap_max, status);
    if (g.ndim == 3 && !g.transpose && g.stride[0] == 1 && g.stride[1] == 1 && g.stride[2] == 1) {
      // the fused neighbour table covers ceil(n_max / 128) tiles; offset masks, then row masks, right behind the ids
      // (SPConvMM's layout)
      const int64_t nbr_tiles = (n_max + 127) / 128;
      uint32_t* nbr_mask = nbr ? reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(nbr) +
                                                             align_up((size_t)g.kvol * nbr_tiles * 128 * 4, 256))
                               : nullptr;
      uint32_t* nbr_rows = nbr ? reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(nbr_mask) +
                                                             align_up((size_t)nbr_tiles * sizeof(uint32_t), 256))
                               : nullptr;
      int32_t* nbr_perm = nbr ? reinterpret_cast<int32_t*>(reinterpret_cast<unsigned char*>(nbr_rows) +
                                                           align_up((size_t)nbr_tiles * g.kvol * 16, 256))
                              : nullptr;
      // one CTA per 256 rows up to the end of the table, so that rows beyond the live count get their -1 / masks
      const int nblk_t = nbr ? (int)ceil_div(nbr_tiles * 128, kIdxThreads) : nblk;
      if (g.ksize[1] == 3 && g.klast == 3)
        subm_probe3_kernel<true><<<nblk_t, kIdxThreads, 0, st>>>(plan.table, coors, num_act_in, n_max, g, plan.cap_max,
                                                                 plan.pair_out, plan.block_counts, nblk, nbr, nbr_mask,
                                                                 nbr_rows, nbr_perm, nbr_tiles);
      else
        subm_probe3_kernel<false><<<nblk_t, kIdxThreads, 0, st>>>(plan.table, coors, num_act_in, n_max, g,
                                                                  plan.cap_max, plan.pair_out, plan.block_counts, nblk,
                                                                  nbr, nbr_mask, nbr_rows, nbr_perm, nbr_tiles);
    } else {
      D3D_REQUIRE(!nbr, D3D_ERR_INVALID_ARGUMENT);
      subm_probe_kernel<<<dim3(nblk, g.rows), kIdxThreads, 0, st>>>(plan.table, coors, num_act_in, n_max, g,
                                                                    plan.cap_max, plan.pair_out, plan.block_counts,
                                                                    nblk);
    }
  } else {
    int32_t* out_coors = reinterpret_cast<int32_t*>(outputs[2]);
    int32_t* num_act_out = reinterpret_cast<int32_t*>(outputs[3]);
    D3D_REQUIRE(out_coors && num_act_out, D3D_ERR_INVALID_ARGUMENT);
    D3D_REQUIRE(out[2].dims[0] >= p->max_num_act_out, D3D_ERR_INVALID_ARGUMENT);
    if (plan.packed)
      conv_insert3_kernel<true><<<nblk, kIdxThreads, 0, st>>>(plan.table, coors, num_act_in, n_max, g, plan.fan,
                                                              plan.cap_max, plan.pair_out, status);
    else if (g.ndim == 3 && g.ksize[0] <= 3 && g.ksize[1] <= 3 && g.ksize[2] <= 3)
      conv_insert3_kernel<false><<<nblk, kIdxThreads, 0, st>>>(plan.table, coors, num_act_in, n_max, g, plan.fan,
                                                               plan.cap_max, plan.pair_out, status);
    else
      conv_insert_kernel<<<dim3(nblk, g.rows), kIdxThreads, 0, st>>>(plan.table, coors, num_act_in, n_max, g,
                                                                     plan.fan, plan.cap_max, plan.pair_out, status);
    conv_count_winners_kernel<<<nblk, kIdxThreads, 0, st>>>(plan.table, plan.pair_out, num_act_in, n_max, g.kvol,
                                                            plan.packed, plan.winners, plan.win_bits);
    scan_totals_kernel<<<1, 1024, 0, st>>>(plan.winners, nblk, p->max_num_act_out, num_act_out, status);
    conv_assign_kernel<<<nblk, kIdxThreads, 0, st>>>(plan.table, plan.pair_out, num_act_in, n_max, g, plan.winners,
                                                     plan.win_bits,
                                                     p->max_num_act_out, plan.packed, plan.slot_out, out_coors);
    if (plan.packed)
      conv_translate_packed_kernel<<<nblk, kIdxThreads, 0, st>>>(plan.pair_out, plan.slot_out, num_act_in, n_max,
                                                                 g.kvol, plan.block_counts, nblk);
    else
      conv_translate_all_kernel<<<nblk, kIdxThreads, 0, st>>>(plan.pair_out, plan.slot_out, num_act_in, n_max, g.kvol,
                                                              plan.block_counts, nblk);
  }
  segment_scan_kernel<<<g.kvol, 1024, 0, st>>>(plan.block_counts, nblk, g.kvol, num_act_in, n_max, plan.seg, num_index,
                                          plan.state, persistent, first, plan.row_len);
  if (!p->subm && plan.packed)
    compact_packed_kernel<<<nblk, kIdxThreads, 0, st>>>(plan.pair_out, plan.block_counts, plan.seg, num_act_in, n_max,
                                                        nblk, g.kvol, index, plan.row_len);
  else if (g.kvol <= kCompactAllMaxVol)
    (g.kvol <= kCompactHeld ? compact_all_kernel<true> : compact_all_kernel<false>)<<<nblk, kIdxThreads, 0, st>>>(
        plan.pair_out, plan.block_counts, plan.seg, num_act_in, n_max, nblk, g.kvol, index, plan.row_len);
  else
    compact_kernel<<<dim3(nblk, g.kvol), kIdxThreads, 0, st>>>(plan.pair_out, plan.block_counts, plan.seg,
                                                               num_act_in, n_max, nblk, index, plan.row_len);
  fill_padding_kernel<<<stream_grid(3 * plan.row_len, 256), 256, 0, st>>>(plan.seg, g.kvol, index, plan.row_len,
                                                                          plan.state);
  D3D_CHECK_LAUNCH();
  return D3D_OK;
}
