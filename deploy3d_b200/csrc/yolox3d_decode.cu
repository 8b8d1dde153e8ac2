// YoloX3dDecode: per (batch row, class) the K best BEV cells by class score, decoded into boxes.
//
// Replaces decoder::YoloX3dDecodePlugin of the reference (trt/decoder/yolox3d_decode.cu:147-412): there a
// segmented radix sort of all B*C*Y*X scores (cub, :341-355) followed by one decode launch per class (:357-367).
// Only the first K entries of every sorted segment are ever read, so here one CTA per (class, batch row) selects
// them directly: a 4-pass radix select finds the K-th largest key, the cells above it (and, among equal scores,
// the lowest positions, which is what the stable sort of the reference yields) are collected in shared memory,
// sorted there, and decoded in the same kernel.  No workspace, one launch for all classes.
#include <cuda_fp16.h>
#include <string.h>

#include "common.cuh"

namespace d3d {
namespace {

constexpr int kThreads = 1024;
constexpr int kMaxTopK = 4096;  // candidates are sorted in shared memory

// Order-preserving map of a float to an unsigned key (larger score = larger key); -0 and +0 share a key.
__device__ __forceinline__ uint32_t score_key(float f) {
  uint32_t u = __float_as_uint(f);
  if ((u << 1) == 0u) u = 0u;
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
template <class T> __device__ __forceinline__ float load_f32(const T* p);
template <> __device__ __forceinline__ float load_f32<float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float load_f32<__half>(const __half* p) { return __half2float(__ldg(p)); }

struct DecodeArgs {
  const void* cls_scores;  // [B, C, Y, X]
  const void* bbox_preds;  // [B, 9 + a, Y, X]
  const float* pillar_config;
  int num_class, size_y, size_x, box_in_params, topk;
  int stride;
  int class_ids[8];
  int32_t* out_ids[8];  // [B, K]
  float* out_scores[8];  // [B, K]
  float* out_boxes[8];   // [B, K, 7 + a]
};

// Box of BEV cell `pos` (trt/decoder/yolox3d_decode.cu:46-125, same arithmetic in the same precision).
template <class T>
__device__ __forceinline__ void decode_cell(const DecodeArgs& a, const T* preds_b, int pos, float score, int32_t* id_out,
                                            float* score_out, float* box_out, int cls) {
  const int n = a.size_y * a.size_x;
  const float x_min = a.pillar_config[0], y_min = a.pillar_config[1];
  const float feat_stride = static_cast<float>(a.stride) * a.pillar_config[3];
  const float x_base = static_cast<float>(pos % a.size_x), y_base = static_cast<float>(pos / a.size_x);
  const T* pred = preds_b + pos;
  float cx = load_f32(pred) + x_base;
  const bool cx_valid = (cx <= a.size_x && cx >= 0);
  cx = x_min + feat_stride * cx;
  float cy = load_f32(pred + n) + y_base;
  const bool cy_valid = (cy <= a.size_y && cy >= 0);
  cy = y_min + feat_stride * cy;
  float cz = load_f32(pred + 2 * n);
  float dx = feat_stride * expf(load_f32(pred + 3 * n));
  float dy = feat_stride * expf(load_f32(pred + 4 * n));
  float dz = expf(load_f32(pred + 5 * n));
  float yaw = load_f32(pred + 6 * n);
  const float dir_sine = load_f32(pred + 7 * n), dir_cosine = load_f32(pred + 8 * n);
  const float dir = atan2f(dir_sine, dir_cosine);
  const bool yaw_valid = (dir_sine != 0) || (dir_cosine != 0);
  if (!(isfinite(cx) && isfinite(cy) && isfinite(cz) && isfinite(dx) && isfinite(dy) && isfinite(dz) && isfinite(yaw) &&
        dx > 0 && dy > 0 && dz > 0 && yaw_valid && cx_valid && cy_valid)) {
    score = -1.0f;
    cx = cy = cz = 10000.0f;
    dx = dy = dz = 1.f;
    yaw = 0.f;
  } else if (0.9f * dx < dy && dy < 1.11f * dx) {  // nearly square: the direction head decides the heading
    yaw = dir;
    const float t = fmaxf(dx, dy);
    dx = t, dy = t;
  } else {  // elongated: yaw, flipped to the half-plane of the direction head
    if (dy > dx) {
      yaw += M_PI_2;
      const float t = dy;
      dy = dx, dx = t;
    }
    yaw += floorf((dir - yaw) / M_PI + 0.5) * M_PI;
    yaw -= floorf(yaw / (2 * M_PI) + 0.5) * (2 * M_PI);
  }
  *id_out = cls;
  *score_out = score;
  box_out[0] = cx, box_out[1] = cy, box_out[2] = cz, box_out[3] = dx, box_out[4] = dy, box_out[5] = dz, box_out[6] = yaw;
  for (int e = 9; e < a.box_in_params; ++e) box_out[e - 2] = load_f32(pred + (int64_t)e * n);
}

template <class T>
__global__ void __launch_bounds__(kThreads)
topk_decode_kernel(const DecodeArgs a) {
  extern __shared__ unsigned long long cand[];  // [padded K] (key << 32) | ~position: descending = the output order
  __shared__ int hist[256];
  __shared__ int scratch[40];
  __shared__ uint32_t sel_prefix, sel_mask;
  __shared__ int sel_need, n_greater;
  const int c = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  const int n = a.size_y * a.size_x, k_out = a.topk;
  const T* scores = reinterpret_cast<const T*>(a.cls_scores) + ((int64_t)b * a.num_class + c) * n;
  const T* preds_b = reinterpret_cast<const T*>(a.bbox_preds) + (int64_t)b * a.box_in_params * n;
  if (tid == 0) sel_prefix = 0u, sel_mask = 0u, sel_need = k_out, n_greater = 0;
  // ---- radix select: after the four passes sel_prefix is the K-th largest key, sel_need how many cells with
  // exactly that key belong to the top K
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int d = tid; d < 256; d += kThreads) hist[d] = 0;
    __syncthreads();
    const uint32_t prefix = sel_prefix, mask = sel_mask;
    for (int i = tid; i < n; i += kThreads) {
      const uint32_t key = score_key(load_f32(scores + i));
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int need = sel_need, d = 255;
      for (; d > 0 && hist[d] < need; --d) need -= hist[d];
      sel_need = need;
      sel_prefix = prefix | ((uint32_t)d << shift);
      sel_mask = mask | (255u << shift);
    }
    __syncthreads();
  }
  const uint32_t threshold = sel_prefix;
  const int need = sel_need, greater = k_out - need;
  // ---- collect: everything above the threshold (any order), then the `need` lowest positions at the threshold
  int tie_base = 0;
  for (int base = 0; base < n; base += kThreads) {
    const int i = base + tid;
    uint32_t key = 0u;
    bool tie = false;
    if (i < n) {
      key = score_key(load_f32(scores + i));
      tie = key == threshold;
      if (key > threshold) cand[atomicAdd(&n_greater, 1)] = ((unsigned long long)key << 32) | (0xFFFFFFFFu - (uint32_t)i);
    }
    int total;
    const int rank = tie_base + block_exclusive_scan(tie ? 1 : 0, scratch, &total);
    if (tie && rank < need) cand[greater + rank] = ((unsigned long long)key << 32) | (0xFFFFFFFFu - (uint32_t)i);
    tie_base += total;
  }
  int padded = 1;
  while (padded < k_out) padded <<= 1;
  for (int i = k_out + tid; i < padded; i += kThreads) cand[i] = 0ull;
  __syncthreads();
  // ---- bitonic sort, descending
  for (int size = 2; size <= padded; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = tid; t < (padded >> 1); t += kThreads) {
        const int lo = 2 * t - (t & (stride - 1)), hi = lo + stride;
        const bool descending = (lo & size) == 0;
        const unsigned long long x = cand[lo], y = cand[hi];
        if ((x < y) == descending) cand[lo] = y, cand[hi] = x;
      }
      __syncthreads();
    }
  }
  // ---- decode
  for (int r = tid; r < k_out; r += kThreads) {
    const int pos = (int)(0xFFFFFFFFu - (uint32_t)cand[r]);
    const int64_t o = (int64_t)b * k_out + r;
    decode_cell<T>(a, preds_b, pos, load_f32(scores + pos), a.out_ids[c] + o, a.out_scores[c] + o,
                   a.out_boxes[c] + o * (a.box_in_params - 2), a.class_ids[c]);
  }
}

int num_classes(const d3d_yolox3d_decode_params* p) {
  for (int i = 0; i < 8; ++i)
    if (p->class_ids[i] < 0) return i;
  return 8;
}

}  // namespace
}  // namespace d3d

using namespace d3d;

extern "C" int d3d_yolox3d_decode_parse(const void* data_s, size_t len, d3d_yolox3d_decode_params* p) {
  D3D_REQUIRE(p && (data_s || len == 0), D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(len >= sizeof(int32_t) * 10, D3D_ERR_BAD_BLOB);
  const unsigned char* s = reinterpret_cast<const unsigned char*>(data_s);
  memcpy(&p->stride, s, 4);
  memcpy(&p->topk, s + 4, 4);
  memcpy(p->class_ids, s + 8, 32);
  D3D_REQUIRE(p->stride >= 1 && p->topk >= 1, D3D_ERR_BAD_BLOB);
  return D3D_OK;
}

extern "C" int d3d_yolox3d_decode_num_outputs(const d3d_yolox3d_decode_params* p) {
  return p ? 3 * num_classes(p) : D3D_ERR_INVALID_ARGUMENT;
}

static int decode_dims(const d3d_yolox3d_decode_params* p, const d3d_tensor_desc* in, int n_in, int* b, int* c, int* y,
                       int* x, int* box_in, int* k) {
  D3D_REQUIRE(p && in && n_in >= 3 && in[0].nb_dims == 4 && in[1].nb_dims == 4 && in[2].nb_dims == 1,
              D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE((in[0].dtype == D3D_FLOAT || in[0].dtype == D3D_HALF) && in[1].dtype == in[0].dtype &&
                  in[2].dtype == D3D_FLOAT,
              D3D_ERR_UNSUPPORTED_DTYPE);
  *b = (int)in[0].dims[0], *c = (int)in[0].dims[1], *y = (int)in[0].dims[2], *x = (int)in[0].dims[3];
  *box_in = (int)in[1].dims[1];
  D3D_REQUIRE(in[1].dims[0] == *b && in[1].dims[2] == *y && in[1].dims[3] == *x && *box_in >= 9 && in[2].dims[0] >= 4,
              D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(*c >= 0 && *c <= num_classes(p), D3D_ERR_INVALID_ARGUMENT);
  const int64_t n = (int64_t)*y * *x;
  D3D_REQUIRE(n < (1ll << 31) && *b <= 65535, D3D_ERR_TOO_LARGE);
  *k = (int)(n < p->topk ? n : p->topk);
  return D3D_OK;
}

extern "C" int d3d_yolox3d_decode_output_desc(const d3d_yolox3d_decode_params* p, const d3d_tensor_desc* in, int n_in,
                                              int index, d3d_tensor_desc* out) {
  D3D_REQUIRE(out && index >= 0, D3D_ERR_INVALID_ARGUMENT);
  int b, c, y, x, box_in, k;
  int rc = decode_dims(p, in, n_in, &b, &c, &y, &x, &box_in, &k);
  if (rc != D3D_OK) return rc;
  D3D_REQUIRE(index < 3 * num_classes(p), D3D_ERR_INVALID_ARGUMENT);
  memset(out, 0, sizeof(*out));
  out->dtype = index % 3 == 0 ? D3D_INT32 : D3D_FLOAT;
  out->nb_dims = index % 3 == 2 ? 3 : 2;
  out->dims[0] = b, out->dims[1] = k;
  if (index % 3 == 2) out->dims[2] = box_in - 2;
  return D3D_OK;
}

extern "C" int d3d_yolox3d_decode_workspace(const d3d_yolox3d_decode_params* p, const d3d_tensor_desc* in, int n_in,
                                            size_t* bytes) {
  D3D_REQUIRE(p && bytes, D3D_ERR_INVALID_ARGUMENT);
  (void)in, (void)n_in;
  *bytes = 0;  // the reference needs the radix-sort scratch (yolox3d_decode.cu:255-298); the top-K select needs none
  return D3D_OK;
}

extern "C" int d3d_yolox3d_decode_enqueue(const d3d_yolox3d_decode_params* p, const d3d_tensor_desc* in, int n_in,
                                          const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                                          void* const* outputs, void* workspace, size_t workspace_bytes,
                                          void* stream) {
  D3D_NVTX_RANGE("d3d_yolox3d_decode_enqueue");
  (void)workspace, (void)workspace_bytes;
  D3D_REQUIRE(out && inputs && outputs, D3D_ERR_INVALID_ARGUMENT);
  int b, c, y, x, box_in, k;
  int rc = decode_dims(p, in, n_in, &b, &c, &y, &x, &box_in, &k);
  if (rc != D3D_OK) return rc;
  D3D_REQUIRE(n_out >= 3 * c, D3D_ERR_INVALID_ARGUMENT);
  if (b == 0 || c == 0 || k == 0) return D3D_OK;
  D3D_REQUIRE(k <= kMaxTopK, D3D_ERR_TOO_LARGE);
  DecodeArgs a;
  a.cls_scores = inputs[0], a.bbox_preds = inputs[1], a.pillar_config = reinterpret_cast<const float*>(inputs[2]);
  a.num_class = c, a.size_y = y, a.size_x = x, a.box_in_params = box_in, a.topk = k, a.stride = p->stride;
  for (int i = 0; i < 8; ++i) {
    a.class_ids[i] = p->class_ids[i];
    a.out_ids[i] = i < c ? reinterpret_cast<int32_t*>(outputs[3 * i]) : nullptr;
    a.out_scores[i] = i < c ? reinterpret_cast<float*>(outputs[3 * i + 1]) : nullptr;
    a.out_boxes[i] = i < c ? reinterpret_cast<float*>(outputs[3 * i + 2]) : nullptr;
    D3D_REQUIRE(i >= c || (a.out_ids[i] && a.out_scores[i] && a.out_boxes[i]), D3D_ERR_INVALID_ARGUMENT);
  }
  int padded = 1;
  while (padded < k) padded <<= 1;
  const size_t smem = (size_t)padded * sizeof(unsigned long long);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (in[0].dtype == D3D_FLOAT)
    topk_decode_kernel<float><<<dim3(c, b), kThreads, smem, st>>>(a);
  else
    topk_decode_kernel<__half><<<dim3(c, b), kThreads, smem, st>>>(a);
  D3D_CHECK_LAUNCH();
  return D3D_OK;
}
