// SimpleMeanEncoder and CylinderEncoder: point cloud -> voxels.
//
// Replace voxel_encoder::func::simpleMeanEncoder (trt/voxel_encoder/simple_mean_trt.cu:121-168, kernels :28-102)
// and voxel_encoder::func::CylinderEncoder (trt/voxel_encoder/cylinder_trt.cu:130-174, kernels :28-111).
// Both share one scheme: each point inserts its voxel key into the open-addressing table with its own index as
// value (the smallest index survives), the points that "own" their voxel are counted and ranked with a two-level
// scan, which numbers the voxels by first touch; a last pass reduces the points into their voxels.
// The reference numbers voxels by hash-slot rank (a scan over the whole 2N-slot table) instead.
#include <math.h>

#include "common.cuh"

namespace d3d {
namespace {

constexpr int kEncThreads = 256;

__global__ void enc_reset_kernel(unsigned long long* table, uint32_t cap, int32_t* count, int64_t m_max,
                                 float* zero_feats, int64_t zero_elems) {
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
  for (int64_t s = tid; s < cap; s += nth) table[s] = kEmptySlot;
  for (int64_t s = tid; s < m_max; s += nth) count[s] = 0;
  for (int64_t s = tid; s < zero_elems; s += nth) zero_feats[s] = 0.f;
}

__device__ __forceinline__ bool all_finite(const float* __restrict__ p, int c) {
  bool ok = true;
  for (int f = 0; f < c; ++f) ok = ok && isfinite(p[f]);
  return ok;
}

// trt/voxel_encoder/simple_mean_trt.cu:28-60: truncation toward zero, bounds check, insert.
__global__ void voxelize_kernel(unsigned long long* table, uint32_t cap_mask, const float* __restrict__ pts,
                                const int32_t* __restrict__ batch, const float* __restrict__ cfg, int64_t n, int c,
                                int sb, int sz, int sy, int sx, int32_t* __restrict__ slot_of, int32_t* status) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float* p = pts + i * c;
  int slot = -1;
  int b = batch[i];
  if (all_finite(p, c) && b >= 0 && b < sb) {
    int cx = (int)__fdiv_rn(__fsub_rn(p[0], cfg[0]), cfg[3]);
    int cy = (int)__fdiv_rn(__fsub_rn(p[1], cfg[1]), cfg[4]);
    int cz = (int)__fdiv_rn(__fsub_rn(p[2], cfg[2]), cfg[5]);
    if (cx >= 0 && cx < sx && cy >= 0 && cy < sy && cz >= 0 && cz < sz) {
      uint32_t key = (((uint32_t)b * sz + cz) * sy + cy) * sx + cx;
      uint32_t s = hash_insert_min_claim_first(table, cap_mask, key, (uint32_t)i);
      slot = s == 0xFFFFFFFFu ? -1 : (int)s;
      if (s == 0xFFFFFFFFu) report_status(status, D3D_STATUS_HASH_FULL);
    }
  }
  slot_of[i] = slot;
}

// trt/voxel_encoder/cylinder_trt.cu:28-85.  cfg = (zmin, phimin, rhomin, zmax, phimax, rhomax), dims (rho, phi, z).
__global__ void cylinderize_kernel(unsigned long long* table, uint32_t cap_mask, const float* __restrict__ pts,
                                   const int32_t* __restrict__ batch, const float* __restrict__ cfg, int64_t n, int c,
                                   int sb, int sr, int sp, int sz, int32_t* __restrict__ slot_of,
                                   float* __restrict__ aug) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float* p = pts + i * c;
  float* a = aug + i * (c + 5);
  int slot = -1;
  bool wrote = false;
  if (all_finite(p, c)) {
    int b = batch[i];
    float x = p[0], y = p[1], z = p[2];
    float rho = sqrtf(__fadd_rn(__fmul_rn(x, x), __fmul_rn(y, y)));
    float phi = atan2f(y, x);
    if (b >= 0 && b < sb) {
      float zmin = cfg[0], pmin = cfg[1], rmin = cfg[2];
      float zs = __fdiv_rn(__fsub_rn(cfg[3], cfg[0]), (float)sz);
      float ps = __fdiv_rn(__fsub_rn(cfg[4], cfg[1]), (float)sp);
      float rs = __fdiv_rn(__fsub_rn(cfg[5], cfg[2]), (float)sr);
      int zc = (int)__fdiv_rn(__fsub_rn(z, zmin), zs);
      int pc = (int)__fdiv_rn(__fsub_rn(phi, pmin), ps);
      int rc = (int)__fdiv_rn(__fsub_rn(rho, rmin), rs);
      if (pc >= 0 && pc < sp && rc >= 0 && rc < sr) {
        zc = zc < 0 ? 0 : zc;  // z is clamped, not dropped (cylinder_trt.cu:64-66)
        zc = zc >= sz ? sz - 1 : zc;
        uint32_t key = (((uint32_t)b * sr + rc) * sp + pc) * sz + zc;
        uint32_t s = hash_insert_min_claim_first(table, cap_mask, key, (uint32_t)i);
        slot = s == 0xFFFFFFFFu ? -1 : (int)s;
        a[0] = z;
        a[1] = phi;
        a[2] = rho;
        a[3] = z - ((zc + 0.5f) * zs + zmin);
        a[4] = phi - ((pc + 0.5f) * ps + pmin);
        a[5] = rho - ((rc + 0.5f) * rs + rmin);
        a[6] = x;
        a[7] = y;
        for (int f = 3; f < c; ++f) a[f + 5] = p[f];
        wrote = true;
      }
    }
  }
  if (!wrote)
    for (int f = 0; f < c + 5; ++f) a[f] = 0.f;  // the reference memsets the tensor (cylinder_trt.cu:162)
  slot_of[i] = slot;
}

__device__ __forceinline__ bool owns_voxel(const unsigned long long* table, int slot, int64_t i) {
  return slot >= 0 && (uint32_t)table[slot] == (uint32_t)i;
}

__global__ void count_owners_kernel(const unsigned long long* __restrict__ table, const int32_t* __restrict__ slot_of,
                                    int64_t n, int32_t* __restrict__ owners) {
  __shared__ int scratch[40];
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int v = i < n && owns_voxel(table, slot_of[i], i);
  int total;
  block_exclusive_scan(v, scratch, &total);
  if (threadIdx.x == 0) owners[blockIdx.x] = total;
}

// Owners number their voxel and write its coordinates (decoded from the key, 4 columns, last extent fastest).
__global__ void number_voxels_kernel(const unsigned long long* __restrict__ table, const int32_t* __restrict__ slot_of,
                                     int64_t n, const int32_t* __restrict__ owners_base, int64_t m_max, int e1, int e2,
                                     int e3, int32_t* __restrict__ slot_vid, int32_t* __restrict__ out_coors) {
  __shared__ int scratch[40];
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int slot = i < n ? slot_of[i] : -1;
  int v = i < n && owns_voxel(table, slot, i);
  int total;
  int vid = owners_base[blockIdx.x] + block_exclusive_scan(v, scratch, &total);
  if (!v) return;
  if (vid < m_max) {
    slot_vid[slot] = vid;
    uint32_t key = (uint32_t)(table[slot] >> 32);
    int c3 = key % e3;
    key /= e3;
    int c2 = key % e2;
    key /= e2;
    int c1 = key % e1;
    key /= e1;
    reinterpret_cast<int4*>(out_coors)[vid] = make_int4((int)key, c1, c2, c3);
  } else {
    slot_vid[slot] = -1;  // beyond maxNumActOut (simple_mean_trt.cu:75, cylinder_trt.cu:101)
  }
}

// trt/voxel_encoder/simple_mean_trt.cu:62-91: per-voxel sums and point counts.
__global__ void mean_accumulate_kernel(const int32_t* __restrict__ slot_of, const int32_t* __restrict__ slot_vid,
                                       const float* __restrict__ pts, int64_t n, int c, float* __restrict__ out_feats,
                                       int32_t* __restrict__ count) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int slot = slot_of[i];
  if (slot < 0) return;
  int vid = slot_vid[slot];
  if (vid < 0) return;
  atomicAdd(&count[vid], 1);
  const float* p = pts + i * c;
  float* o = out_feats + (int64_t)vid * c;
  int f = 0;
  if ((c & 3) == 0) {
    for (; f < c; f += 4) {
      float4 v = *reinterpret_cast<const float4*>(p + f);
      atomicAdd(reinterpret_cast<float4*>(o + f), v);  // one 16-byte reduction per four channels
    }
  }
  for (; f < c; ++f) atomicAdd(o + f, p[f]);
}

// trt/voxel_encoder/simple_mean_trt.cu:93-102
// With `lp` != null the mean is also written in half / bfloat16 into rows of `lp_c` >= c channels (the extra
// channels zero): the tensor the first sparse convolution reads, without a separate cast-and-pad kernel.
// One thread per voxel: its c sums become means in place; the low-precision row is put together in registers and
// leaves as 16-byte stores where the row width allows.
template <class LP>
__global__ void mean_divide_kernel(float* __restrict__ out_feats, const int32_t* __restrict__ count,
                                   const int32_t* num_act_out, int c, LP* __restrict__ lp, int lp_c) {
  const int n = *num_act_out;
  const bool wide = lp && lp_c % 8 == 0 && (reinterpret_cast<uintptr_t>(lp) & 15) == 0;
  for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < n; v += gridDim.x * blockDim.x) {
    const float cnt = (float)count[v];
    float* row = out_feats + (int64_t)v * c;
    for (int ch = 0; ch < c; ++ch) row[ch] = __fdiv_rn(row[ch], cnt);
    if (!lp) continue;
    LP* lrow = lp + (int64_t)v * lp_c;
    if (wide) {
      for (int z0 = 0; z0 < lp_c; z0 += 8) {
        __align__(16) LP h[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) h[q] = LP(z0 + q < c ? row[z0 + q] : 0.f);
        *reinterpret_cast<uint4*>(lrow + z0) = *reinterpret_cast<const uint4*>(h);
      }
    } else {
      for (int z = 0; z < lp_c; ++z) lrow[z] = LP(z < c ? row[z] : 0.f);
    }
  }
}

// trt/voxel_encoder/cylinder_trt.cu:87-111
__global__ void scatter_ids_kernel(const int32_t* __restrict__ slot_of, const int32_t* __restrict__ slot_vid,
                                   int64_t n, int32_t* __restrict__ scatter_to, int32_t* __restrict__ scatter_count) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int slot = slot_of[i];
  int vid = slot >= 0 ? slot_vid[slot] : -1;
  scatter_to[i] = vid;
  if (vid >= 0) atomicAdd(&scatter_count[vid], 1);
}

struct EncPlan {
  int64_t n;
  int c;
  int nblk;
  uint32_t cap;
  int dims[4];
  unsigned long long* table;
  int32_t* slot_of;
  int32_t* slot_vid;
  int32_t* owners;
  int32_t* count;
  size_t bytes;
};

int make_enc_plan(const d3d_voxel_encoder_params* p, const d3d_tensor_desc* in, int n_in, void* workspace,
                  bool need_count, EncPlan* plan) {
  D3D_REQUIRE(p && in && n_in >= 4, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(in[0].nb_dims == 2 && in[1].nb_dims == 1 && in[3].nb_dims == 5, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(in[0].dtype == D3D_FLOAT, D3D_ERR_UNSUPPORTED_DTYPE);
  D3D_REQUIRE(in[1].dims[0] == in[0].dims[0] && p->max_num_act_out >= 0, D3D_ERR_INVALID_ARGUMENT);
  plan->n = in[0].dims[0];
  plan->c = (int)in[0].dims[1];
  D3D_REQUIRE(plan->c >= 3, D3D_ERR_INVALID_ARGUMENT);
  int64_t vol = 1;
  const int src[4] = {0, 2, 3, 4};
  for (int d = 0; d < 4; ++d) {
    plan->dims[d] = (int)in[3].dims[src[d]];
    D3D_REQUIRE(plan->dims[d] >= 1, D3D_ERR_INVALID_ARGUMENT);
    vol *= plan->dims[d];
    D3D_REQUIRE(vol < (1ll << 31), D3D_ERR_TOO_LARGE);
  }
  D3D_REQUIRE(plan->n < (1ll << 30), D3D_ERR_TOO_LARGE);
  plan->nblk = (int)ceil_div(plan->n > 0 ? plan->n : 1, kEncThreads);
  plan->cap = (uint32_t)next_pow2((size_t)(plan->n > 8 ? plan->n : 8) * 2);
  Carver w(workspace);
  plan->table = w.take<unsigned long long>(plan->cap);
  plan->slot_of = w.take<int32_t>(plan->n > 0 ? plan->n : 1);
  plan->slot_vid = w.take<int32_t>(plan->cap);
  plan->owners = w.take<int32_t>((size_t)plan->nblk + 1);
  plan->count = need_count ? w.take<int32_t>(p->max_num_act_out > 0 ? p->max_num_act_out : 1) : nullptr;
  plan->bytes = w.off;
  return D3D_OK;
}

}  // namespace
}  // namespace d3d

using namespace d3d;

static int parse_max_out(const void* data_s, size_t len, d3d_voxel_encoder_params* p) {
  D3D_REQUIRE(data_s && p, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(len >= 4, D3D_ERR_BAD_BLOB);
  memcpy(&p->max_num_act_out, data_s, 4);
  return D3D_OK;
}

extern "C" int d3d_simple_mean_encoder_parse(const void* data_s, size_t len, d3d_voxel_encoder_params* p) {
  return parse_max_out(data_s, len, p);
}
extern "C" int d3d_cylinder_encoder_parse(const void* data_s, size_t len, d3d_voxel_encoder_params* p) {
  return parse_max_out(data_s, len, p);
}

extern "C" int d3d_simple_mean_encoder_workspace(const d3d_voxel_encoder_params* p, const d3d_tensor_desc* in,
                                                 int n_in, size_t* bytes) {
  D3D_REQUIRE(bytes, D3D_ERR_INVALID_ARGUMENT);
  EncPlan plan;
  int rc = make_enc_plan(p, in, n_in, nullptr, true, &plan);
  if (rc == D3D_OK) *bytes = plan.bytes;
  return rc;
}
extern "C" int d3d_cylinder_encoder_workspace(const d3d_voxel_encoder_params* p, const d3d_tensor_desc* in, int n_in,
                                              size_t* bytes) {
  D3D_REQUIRE(bytes, D3D_ERR_INVALID_ARGUMENT);
  EncPlan plan;
  int rc = make_enc_plan(p, in, n_in, nullptr, false, &plan);
  if (rc == D3D_OK) *bytes = plan.bytes;
  return rc;
}

extern "C" int d3d_simple_mean_encoder_enqueue(const d3d_voxel_encoder_params* p, const d3d_tensor_desc* in, int n_in,
                                               const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                                               void* const* outputs, void* workspace, size_t workspace_bytes,
                                               void* stream) {
  D3D_NVTX_RANGE("d3d_simple_mean_encoder_enqueue");
  return d3d_simple_mean_encoder_enqueue_ex(p, in, n_in, out, n_out, inputs, outputs, workspace, workspace_bytes,
                                            stream, nullptr);
}

extern "C" int d3d_simple_mean_encoder_enqueue_ex(const d3d_voxel_encoder_params* p, const d3d_tensor_desc* in,
                                                  int n_in, const d3d_tensor_desc* out, int n_out,
                                                  const void* const* inputs, void* const* outputs, void* workspace,
                                                  size_t workspace_bytes, void* stream,
                                                  const d3d_mean_encoder_extras* extras) {
  D3D_NVTX_RANGE("d3d_simple_mean_encoder_enqueue_ex");
  D3D_REQUIRE(inputs && outputs && out && n_out >= 3, D3D_ERR_INVALID_ARGUMENT);
  void* lp = extras ? extras->lp_feats : nullptr;
  int32_t* status = extras ? extras->status : nullptr;
  D3D_REQUIRE(!lp || ((extras->lp_dtype == D3D_HALF || extras->lp_dtype == D3D_BF16) &&
                      extras->lp_channels >= in[0].dims[1]),
              D3D_ERR_INVALID_ARGUMENT);
  EncPlan pl;
  int rc = make_enc_plan(p, in, n_in, workspace, true, &pl);
  if (rc != D3D_OK) return rc;
  D3D_REQUIRE(workspace && workspace_bytes >= pl.bytes, D3D_ERR_WORKSPACE_TOO_SMALL);
  D3D_REQUIRE(out[0].dims[0] == p->max_num_act_out && out[0].dims[1] == pl.c, D3D_ERR_INVALID_ARGUMENT);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const float* pts = reinterpret_cast<const float*>(inputs[0]);
  const int32_t* batch = reinterpret_cast<const int32_t*>(inputs[1]);
  const float* cfg = reinterpret_cast<const float*>(inputs[2]);
  float* out_feats = reinterpret_cast<float*>(outputs[0]);
  int32_t* out_coors = reinterpret_cast<int32_t*>(outputs[1]);
  int32_t* num_act_out = reinterpret_cast<int32_t*>(outputs[2]);
  const int64_t m_max = p->max_num_act_out;
  enc_reset_kernel<<<stream_grid(pl.cap, 256), 256, 0, st>>>(pl.table, pl.cap, pl.count, m_max, out_feats,
                                                             m_max * pl.c);
  if (pl.n > 0) {
    voxelize_kernel<<<pl.nblk, kEncThreads, 0, st>>>(pl.table, pl.cap - 1, pts, batch, cfg, pl.n, pl.c, pl.dims[0],
                                                     pl.dims[1], pl.dims[2], pl.dims[3], pl.slot_of, status);
    count_owners_kernel<<<pl.nblk, kEncThreads, 0, st>>>(pl.table, pl.slot_of, pl.n, pl.owners);
  }
  scan_totals_kernel<<<1, 1024, 0, st>>>(pl.owners, pl.n > 0 ? pl.nblk : 0, (int32_t)m_max, num_act_out, status);
  if (pl.n > 0 && m_max > 0) {
    number_voxels_kernel<<<pl.nblk, kEncThreads, 0, st>>>(pl.table, pl.slot_of, pl.n, pl.owners, m_max, pl.dims[1],
                                                          pl.dims[2], pl.dims[3], pl.slot_vid, out_coors);
    mean_accumulate_kernel<<<pl.nblk, kEncThreads, 0, st>>>(pl.slot_of, pl.slot_vid, pts, pl.n, pl.c, out_feats,
                                                            pl.count);
    if (lp && extras->lp_dtype == D3D_BF16)
      mean_divide_kernel<__nv_bfloat16><<<stream_grid(m_max, 256), 256, 0, st>>>(
          out_feats, pl.count, num_act_out, pl.c, reinterpret_cast<__nv_bfloat16*>(lp), extras->lp_channels);
    else
      mean_divide_kernel<__half><<<stream_grid(m_max, 256), 256, 0, st>>>(
          out_feats, pl.count, num_act_out, pl.c, reinterpret_cast<__half*>(lp), lp ? extras->lp_channels : 0);
  }
  D3D_CHECK_LAUNCH();
  return D3D_OK;
}

extern "C" int d3d_cylinder_encoder_enqueue(const d3d_voxel_encoder_params* p, const d3d_tensor_desc* in, int n_in,
                                            const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                                            void* const* outputs, void* workspace, size_t workspace_bytes,
                                            void* stream) {
  D3D_NVTX_RANGE("d3d_cylinder_encoder_enqueue");
  D3D_REQUIRE(inputs && outputs && out && n_out >= 5, D3D_ERR_INVALID_ARGUMENT);
  EncPlan pl;
  int rc = make_enc_plan(p, in, n_in, workspace, false, &pl);
  if (rc != D3D_OK) return rc;
  D3D_REQUIRE(workspace && workspace_bytes >= pl.bytes, D3D_ERR_WORKSPACE_TOO_SMALL);
  D3D_REQUIRE(out[0].dims[0] == pl.n && out[0].dims[1] == pl.c + 5, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(out[2].dims[0] == p->max_num_act_out, D3D_ERR_INVALID_ARGUMENT);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const float* pts = reinterpret_cast<const float*>(inputs[0]);
  const int32_t* batch = reinterpret_cast<const int32_t*>(inputs[1]);
  const float* cfg = reinterpret_cast<const float*>(inputs[2]);
  float* aug = reinterpret_cast<float*>(outputs[0]);
  int32_t* scatter_to = reinterpret_cast<int32_t*>(outputs[1]);
  int32_t* scatter_count = reinterpret_cast<int32_t*>(outputs[2]);
  int32_t* out_coors = reinterpret_cast<int32_t*>(outputs[3]);
  int32_t* num_act_out = reinterpret_cast<int32_t*>(outputs[4]);
  const int64_t m_max = p->max_num_act_out;
  enc_reset_kernel<<<stream_grid(pl.cap, 256), 256, 0, st>>>(pl.table, pl.cap, scatter_count, m_max, nullptr, 0);
  if (pl.n > 0) {
    cylinderize_kernel<<<pl.nblk, kEncThreads, 0, st>>>(pl.table, pl.cap - 1, pts, batch, cfg, pl.n, pl.c, pl.dims[0],
                                                        pl.dims[1], pl.dims[2], pl.dims[3], pl.slot_of, aug);
    count_owners_kernel<<<pl.nblk, kEncThreads, 0, st>>>(pl.table, pl.slot_of, pl.n, pl.owners);
  }
  scan_totals_kernel<<<1, 1024, 0, st>>>(pl.owners, pl.n > 0 ? pl.nblk : 0, (int32_t)m_max, num_act_out);
  if (pl.n > 0) {
    number_voxels_kernel<<<pl.nblk, kEncThreads, 0, st>>>(pl.table, pl.slot_of, pl.n, pl.owners, m_max, pl.dims[1],
                                                          pl.dims[2], pl.dims[3], pl.slot_vid, out_coors);
    scatter_ids_kernel<<<pl.nblk, kEncThreads, 0, st>>>(pl.slot_of, pl.slot_vid, pl.n, scatter_to, scatter_count);
  }
  D3D_CHECK_LAUNCH();
  return D3D_OK;
}
