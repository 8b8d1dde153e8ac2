// NMS3d: rotated-BEV non-maximum suppression.
//
// Replaces decoder::NMS3dPlugin (trt/decoder/nms3d.cu:58-127, :200-236) with the IoU arithmetic of
// trt/decoder/iou_rotated.cuh:36-234 restated operation by operation (this file is compiled with -fmad=false so
// that no multiply-add is fused and the keep-set is bit-identical to a strict IEEE-754 evaluation).
//
// Two kernels:
//   overlap mask : 64 x 64 box blocks of the upper triangle; 256 threads per block, each thread owns one row box
//                  and a quarter of the columns; a bounding-circle test rejects far-apart pairs before the exact
//                  polygon clipping (for such pairs the clipped area is exactly zero, so the result is unchanged
//                  whenever the threshold is positive).
//   suppression  : one warp per batch row.  Inside a 64-box block the greedy scan runs on register-resident
//                  diagonal words exchanged by warp shuffles; the rows of the kept boxes are then OR-ed into the
//                  remaining words lane-parallel.  The reference runs this step on a single thread per row
//                  (nms3d.cu:106-127, launched <<<B, 1>>>).
#include <math.h>

#include <atomic>

#include "common.cuh"

namespace d3d {
namespace {

struct Pt {
  float x, y;
};
__device__ __forceinline__ Pt sub(Pt a, Pt b) { return Pt{a.x - b.x, a.y - b.y}; }
__device__ __forceinline__ float cross2(Pt a, Pt b) { return a.x * b.y - b.x * a.y; }
__device__ __forceinline__ float dot2(Pt a, Pt b) { return a.x * b.x + a.y * b.y; }

struct Box {
  Pt p[4];     // corners (iou_rotated.cuh:30-49)
  float area;  // dx * dy
  float cx, cy, rad;
};

__device__ __forceinline__ Box make_box(const float* b) {
  Box r;
  float cx = b[0], cy = b[1], w = b[3], h = b[4];
  double theta = b[6];
  float c2 = (float)cos(theta) * 0.5f;
  float s2 = (float)sin(theta) * 0.5f;
  r.p[0].x = cx - s2 * h - c2 * w;
  r.p[0].y = cy + c2 * h - s2 * w;
  r.p[1].x = cx + s2 * h - c2 * w;
  r.p[1].y = cy - c2 * h - s2 * w;
  r.p[2].x = 2 * cx - r.p[0].x;
  r.p[2].y = 2 * cy - r.p[0].y;
  r.p[3].x = 2 * cx - r.p[1].x;
  r.p[3].y = 2 * cy - r.p[1].y;
  r.area = w * h;
  r.cx = cx, r.cy = cy;
  r.rad = 0.5f * sqrtf(w * w + h * h);
  return r;
}

// Area of the intersection polygon (iou_rotated.cuh:51-234).
__device__ float clipped_area(const Box& A, const Box& B) {
  Pt ea[4], eb[4], pts[24], q[24];
  float dist[24];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    ea[i] = sub(A.p[(i + 1) & 3], A.p[i]);
    eb[i] = sub(B.p[(i + 1) & 3], B.p[i]);
  }
  int num = 0;
  for (int i = 0; i < 4; ++i) {
    for (int j = 0; j < 4; ++j) {
      float det = cross2(eb[j], ea[i]);
      if (fabs((double)det) <= 1e-14) continue;
      Pt d = sub(B.p[j], A.p[i]);
      float t1 = cross2(eb[j], d) / det;
      float t2 = cross2(ea[i], d) / det;
      if (t1 >= 0.0f && t1 <= 1.0f && t2 >= 0.0f && t2 <= 1.0f) {
        pts[num].x = A.p[i].x + ea[i].x * t1;
        pts[num].y = A.p[i].y + ea[i].y * t1;
        ++num;
      }
    }
  }
  {
    Pt ab = eb[0], da = eb[3];
    float abab = dot2(ab, ab), adad = dot2(da, da);
    for (int i = 0; i < 4; ++i) {
      Pt ap = sub(A.p[i], B.p[0]);
      float apab = dot2(ap, ab), apad = -dot2(ap, da);
      if (apab >= 0 && apad >= 0 && apab <= abab && apad <= adad) pts[num++] = A.p[i];
    }
  }
  {
    Pt ab = ea[0], da = ea[3];
    float abab = dot2(ab, ab), adad = dot2(da, da);
    for (int i = 0; i < 4; ++i) {
      Pt ap = sub(B.p[i], A.p[0]);
      float apab = dot2(ap, ab), apad = -dot2(ap, da);
      if (apab >= 0 && apad >= 0 && apab <= abab && apad <= adad) pts[num++] = B.p[i];
    }
  }
  if (num <= 2) return 0.0f;
  // Graham scan around the lowest point (iou_rotated.cuh:124-199)
  int t = 0;
  for (int i = 1; i < num; ++i)
    if (pts[i].y < pts[t].y || (pts[i].y == pts[t].y && pts[i].x < pts[t].x)) t = i;
  Pt start = pts[t];
  for (int i = 0; i < num; ++i) q[i] = sub(pts[i], start);
  Pt tmp = q[0];
  q[0] = q[t];
  q[t] = tmp;
  for (int i = 0; i < num; ++i) dist[i] = dot2(q[i], q[i]);
  for (int i = 1; i < num - 1; ++i) {
    for (int j = i + 1; j < num; ++j) {
      float cr = cross2(q[i], q[j]);
      if (((double)cr < -1e-6) || (fabs((double)cr) < 1e-6 && dist[i] > dist[j])) {
        Pt qt = q[i];
        q[i] = q[j];
        q[j] = qt;
        float dt = dist[i];
        dist[i] = dist[j];
        dist[j] = dt;
      }
    }
  }
  int k;
  for (k = 1; k < num; ++k)
    if ((double)dist[k] > 1e-8) break;
  if (k == num) return 0.0f;  // a single point
  q[1] = q[k];
  int m = 2;
  for (int i = k + 1; i < num; ++i) {
    while (m > 1 && cross2(sub(q[i], q[m - 2]), sub(q[m - 1], q[m - 2])) >= 0) --m;
    q[m++] = q[i];
  }
  if (m <= 2) return 0.0f;
  float area = 0;
  for (int i = 1; i < m - 1; ++i) area += (float)fabs((double)cross2(sub(q[i], q[0]), sub(q[i + 1], q[0])));
  return (float)((double)area / 2.0);
}

// nms3d.cu:42-56: BEV IoU, z ignored.  Two boxes whose bounding circles are disjoint cannot overlap (their clipped
// area is exactly 0, and 0 >= thr fails for thr > 0): such pairs never reach the polygon clipping.
__device__ __forceinline__ bool circles_touch(const Box& a, const Box& b) {
  float dx = a.cx - b.cx, dy = a.cy - b.cy, r = a.rad + b.rad;
  return !(dx * dx + dy * dy > r * r * 1.0001f + 1e-6f);
}
__device__ __forceinline__ bool iou_reaches(const Box& a, const Box& b, float thr) {
  float ov = clipped_area(a, b);
  return ov / fmaxf(a.area + b.area - ov, 1e-8f) >= thr;
}

constexpr int kNmsBlock = 64;

// grid (col block, row block, batch); upper triangle only.  mask[b][row][col block] bit j = row suppresses col*64+j.
// Two passes over the 64 x 64 pairs of a CTA: the bounding-circle test for every pair (cheap, uniform), then the
// polygon clipping for the pairs that passed, dealt out evenly over the 256 threads -- taken pair by pair inside the
// first loop, the few survivors would each hold up their whole warp.
__global__ void __launch_bounds__(256)
overlap_mask_kernel(const float* __restrict__ boxes, int k, int box_dim, float thr, int nw,
                    unsigned long long* __restrict__ mask) {
  const int cb = blockIdx.x, rb = blockIdx.y, b = blockIdx.z;
  if (rb > cb) return;
  __shared__ Box cols[kNmsBlock], rows[kNmsBlock];
  __shared__ unsigned int part[kNmsBlock][4];       // 16 columns per word
  __shared__ unsigned short cand[kNmsBlock * kNmsBlock];  // row << 8 | column of a pair to clip
  __shared__ int warp_base[9];
  const float* bx = boxes + (int64_t)b * k * box_dim;
  const int tid = threadIdx.x, r = tid & 63, quarter = tid >> 6;
  if (tid < kNmsBlock) {
    int c = cb * kNmsBlock + tid;
    if (c < k) cols[tid] = make_box(bx + (int64_t)c * box_dim);
  } else if (tid < 2 * kNmsBlock) {
    int rr = rb * kNmsBlock + tid - kNmsBlock;
    if (rr < k) rows[tid - kNmsBlock] = make_box(bx + (int64_t)rr * box_dim);
  }
  part[r][quarter] = 0u;
  __syncthreads();
  const int row = rb * kNmsBlock + r;
  const int ncol = min(k - cb * kNmsBlock, kNmsBlock);
  unsigned int near = 0;  // bit j - 16 * quarter: column j passed the circle test
  if (row < k) {
    int j0 = quarter * 16, j1 = min(j0 + 16, ncol);
    if (rb == cb) j0 = max(j0, r + 1);
    for (int j = j0; j < j1; ++j)
      if (thr <= 0.f || circles_touch(rows[r], cols[j])) near |= 1u << (j - quarter * 16);
  }
  // positions of this thread's pairs in the CTA's list: warp scan, then the eight warp totals
  const int lane = tid & 31, warp = tid >> 5;
  const int mine = __popc(near);
  int inc = mine;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += t;
  }
  if (lane == 31) warp_base[warp + 1] = inc;
  __syncthreads();
  if (tid == 0) {
    warp_base[0] = 0;
    for (int w = 1; w <= 8; ++w) warp_base[w] += warp_base[w - 1];
  }
  __syncthreads();
  int pos = warp_base[warp] + inc - mine;
  for (unsigned int m = near; m; m &= m - 1) cand[pos++] = (unsigned short)((r << 8) | (quarter * 16 + __ffs(m) - 1));
  __syncthreads();
  const int total = warp_base[8];
  for (int i = tid; i < total; i += 256) {
    const int pr = cand[i] >> 8, pj = cand[i] & 255;
    if (iou_reaches(rows[pr], cols[pj], thr)) atomicOr(&part[pr][pj >> 4], 1u << (pj & 15));
  }
  __syncthreads();
  if (tid < kNmsBlock && row < k) {
    unsigned long long w = (unsigned long long)part[r][0] | ((unsigned long long)part[r][1] << 16) |
                           ((unsigned long long)part[r][2] << 32) | ((unsigned long long)part[r][3] << 48);
    mask[((int64_t)b * k + row) * nw + cb] = w;
  }
}

// One warp per batch row (nms3d.cu:106-127).  remv words are lane-distributed: lane l owns words l, l+32, ...
constexpr int kMaxWordsPerLane = 8;  // K <= 64 * 32 * 8 = 16384 boxes per row

__global__ void __launch_bounds__(32)
suppress_kernel(const unsigned long long* __restrict__ mask, const float* __restrict__ in_scores, int k, int nw,
                float* __restrict__ out_scores) {
  const int b = blockIdx.x, lane = threadIdx.x;
  const unsigned long long* mk = mask + (int64_t)b * k * nw;
  unsigned long long remv[kMaxWordsPerLane];
#pragma unroll
  for (int s = 0; s < kMaxWordsPerLane; ++s) remv[s] = 0ull;
  for (int blk = 0; blk < nw; ++blk) {
    const int base = blk * kNmsBlock;
    const int nbox = min(k - base, kNmsBlock);
    // diagonal words of the 64 boxes of this block: lane holds boxes lane and lane + 32
    unsigned long long d0 = lane < nbox ? mk[(int64_t)(base + lane) * nw + blk] : 0ull;
    unsigned long long d1 = lane + 32 < nbox ? mk[(int64_t)(base + lane + 32) * nw + blk] : 0ull;
    unsigned long long cur = 0ull;
#pragma unroll
    for (int s = 0; s < kMaxWordsPerLane; ++s)
      if ((blk >> 5) == s) cur = remv[s];
    cur = __shfl_sync(0xffffffffu, cur, blk & 31);
    for (int i = 0; i < nbox; ++i) {
      unsigned long long di = __shfl_sync(0xffffffffu, i < 32 ? d0 : d1, i & 31);
      if (!((cur >> i) & 1ull)) cur |= di;
    }
    unsigned long long valid = nbox == 64 ? ~0ull : ((1ull << nbox) - 1ull);
    unsigned long long kept = ~cur & valid;
    // scores of this block
    for (int i = lane; i < nbox; i += 32) {
      float s = in_scores[(int64_t)b * k + base + i];
      out_scores[(int64_t)b * k + base + i] = ((cur >> i) & 1ull) ? -1.0f : s;
    }
    // OR the rows of the kept boxes into the words behind this block
    while (kept) {
      int i = __ffsll((long long)kept) - 1;
      kept &= kept - 1;
      const unsigned long long* row = mk + (int64_t)(base + i) * nw;
#pragma unroll
      for (int s = 0; s < kMaxWordsPerLane; ++s) {
        int w = s * 32 + lane;
        if (w > blk && w < nw) remv[s] |= row[w];
      }
    }
  }
}

// Same sweep for K <= 2048 boxes (nw <= 32: lane w owns mask word w).  The mask rows of the 64 boxes of a block
// are first staged in shared memory with independent, coalesced loads; the serial part then touches shared memory
// only, instead of waiting for one global load per kept box.
constexpr int kStagedMaxWords = 32;

constexpr int kStagedThreads = 128;  // four warps load the rows of a block, the first one sweeps them

__global__ void __launch_bounds__(kStagedThreads)
suppress_staged_kernel(const unsigned long long* __restrict__ mask, const float* __restrict__ in_scores, int k, int nw,
                       float* __restrict__ out_scores) {
  __shared__ unsigned long long rows[kNmsBlock * kStagedMaxWords];
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31;
  const bool sweeper = tid < 32;
  const unsigned long long* mk = mask + (int64_t)b * k * nw;
  unsigned long long remv = 0ull;  // word `lane` of the removed set (first warp)
  for (int blk = 0; blk < nw; ++blk) {
    const int base = blk * kNmsBlock;
    const int nbox = min(k - base, kNmsBlock);
    const unsigned long long* src = mk + (int64_t)base * nw;  // nbox consecutive rows of nw words
    const int words = nbox * nw;
    __syncthreads();  // the previous block's rows are no longer needed
#pragma unroll 4
    for (int f = tid; f < words; f += kStagedThreads) rows[f] = __ldg(src + f);
    __syncthreads();
    if (!sweeper) continue;
    const unsigned long long d0 = lane < nbox ? rows[lane * nw + blk] : 0ull;
    const unsigned long long d1 = lane + 32 < nbox ? rows[(lane + 32) * nw + blk] : 0ull;
    unsigned long long cur = __shfl_sync(0xffffffffu, remv, blk);
    for (int i = 0; i < nbox; ++i) {
      const unsigned long long di = __shfl_sync(0xffffffffu, i < 32 ? d0 : d1, i & 31);
      if (!((cur >> i) & 1ull)) cur |= di;
    }
    const unsigned long long valid = nbox == 64 ? ~0ull : ((1ull << nbox) - 1ull);
    unsigned long long kept = ~cur & valid;
    for (int i = lane; i < nbox; i += 32) {
      const float s = in_scores[(int64_t)b * k + base + i];
      out_scores[(int64_t)b * k + base + i] = ((cur >> i) & 1ull) ? -1.0f : s;
    }
    // OR the rows of the kept boxes into the words behind this block
    if (lane > blk && lane < nw) {
      while (kept) {
        const int i = __ffsll((long long)kept) - 1;
        kept &= kept - 1;
        remv |= rows[i * nw + lane];
      }
    }
  }
}

}  // namespace
}  // namespace d3d

using namespace d3d;

extern "C" int d3d_nms3d_parse(const void* data_s, size_t len, d3d_nms3d_params* p) {
  (void)data_s, (void)len;  // the reference plugin carries no parameters (nms3d.cu:143-144)
  D3D_REQUIRE(p, D3D_ERR_INVALID_ARGUMENT);
  p->iou_threshold = 0.1f;  // nms3d.cu:138
  return D3D_OK;
}

static int nms_dims(const d3d_tensor_desc* in, int n_in, int* b, int* k, int* box_dim) {
  D3D_REQUIRE(in && n_in >= 2 && in[0].nb_dims == 2 && in[1].nb_dims == 3, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(in[0].dtype == D3D_FLOAT && in[1].dtype == D3D_FLOAT, D3D_ERR_UNSUPPORTED_DTYPE);
  *b = (int)in[1].dims[0], *k = (int)in[1].dims[1], *box_dim = (int)in[1].dims[2];
  D3D_REQUIRE(in[0].dims[0] == *b && in[0].dims[1] == *k && *box_dim >= 7, D3D_ERR_INVALID_ARGUMENT);
  D3D_REQUIRE(*k <= kNmsBlock * 32 * kMaxWordsPerLane && *b <= 65535, D3D_ERR_TOO_LARGE);
  return D3D_OK;
}

extern "C" int d3d_nms3d_workspace(const d3d_nms3d_params* p, const d3d_tensor_desc* in, int n_in, size_t* bytes) {
  D3D_REQUIRE(p && bytes, D3D_ERR_INVALID_ARGUMENT);
  int b, k, bd;
  int rc = nms_dims(in, n_in, &b, &k, &bd);
  if (rc != D3D_OK) return rc;
  *bytes = align_up((size_t)b * k * ceil_div(k, kNmsBlock) * sizeof(unsigned long long), 256);
  return D3D_OK;
}

// The two launches of an NMS3d call over a mask scratch of b * k * nw words.  Neither sweep reads a word the mask
// kernel did not write in the same call (the diagonal word and the words behind it; the staged sweep copies whole
// rows into shared memory but uses the same words), so the scratch needs no initialisation.
static int launch_nms(const d3d_nms3d_params* p, int b, int k, int bd, int nw, const void* const* inputs,
                      void* const* outputs, unsigned long long* mask, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  overlap_mask_kernel<<<dim3(nw, nw, b), 256, 0, st>>>(reinterpret_cast<const float*>(inputs[1]), k, bd,
                                                       p->iou_threshold, nw, mask);
  if (nw <= kStagedMaxWords)
    suppress_staged_kernel<<<b, kStagedThreads, 0, st>>>(mask, reinterpret_cast<const float*>(inputs[0]), k, nw,
                                                         reinterpret_cast<float*>(outputs[0]));
  else
    suppress_kernel<<<b, 32, 0, st>>>(mask, reinterpret_cast<const float*>(inputs[0]), k, nw,
                                      reinterpret_cast<float*>(outputs[0]));
  D3D_CHECK_LAUNCH();
  return D3D_OK;
}

extern "C" int d3d_nms3d_enqueue(const d3d_nms3d_params* p, const d3d_tensor_desc* in, int n_in,
                                 const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                                 void* const* outputs, void* workspace, size_t workspace_bytes, void* stream) {
  D3D_NVTX_RANGE("d3d_nms3d_enqueue");
  D3D_REQUIRE(p && out && inputs && outputs && n_out >= 1, D3D_ERR_INVALID_ARGUMENT);
  int b, k, bd;
  int rc = nms_dims(in, n_in, &b, &k, &bd);
  if (rc != D3D_OK) return rc;
  if (b == 0 || k == 0) return D3D_OK;
  const int nw = (int)ceil_div(k, kNmsBlock);
  D3D_REQUIRE(workspace && workspace_bytes >= (size_t)b * k * nw * sizeof(unsigned long long),
              D3D_ERR_WORKSPACE_TOO_SMALL);
  return launch_nms(p, b, k, bd, nw, inputs, outputs, reinterpret_cast<unsigned long long*>(workspace), stream);
}

// ---------------------------------------------------------------------------------------------
// NMS3d without a caller-provided workspace.
//
// Some hosts of this library hand a plugin nothing but its input and output pointers and a stream, and are not
// allowed to obtain device memory themselves: a real-time perception loop that bans allocator calls once it is
// running, an engine that was built before the plugin asked for workspace, a thin C caller that owns no memory
// pool.  For them the overlap-mask scratch of NMS3d lives in the library image itself: a file-scope device
// array of fixed size.  Every GPU that loads the library keeps those 2 MiB until the process exits.
//
// `g_nms_static_mask` below is, in host code, only a handle for the symbol -- not a device address.  The address
// a kernel can use is looked up once per device with cudaGetSymbolAddress (with that device current) and cached;
// that look-up happens inside the first call on a device, which therefore should be made before any stream
// capture is started.  Nothing in the array has to start at zero: the mask kernel overwrites every word the
// suppression kernel reads, so stale contents of an earlier call are harmless.  All calls on one GPU share the
// one array: two calls that overlap on the GPU (different streams, or different threads) race on it.
// ---------------------------------------------------------------------------------------------
// D3D_NMS3D_STATIC_MAX_WORDS (include/deploy3d_b200.h): 256 Ki 64-bit mask words = 2 MiB; 10 x 1000 boxes need 160 000
static __device__ __align__(256) unsigned long long g_nms_static_mask[D3D_NMS3D_STATIC_MAX_WORDS];

namespace {
constexpr int kMaxStaticDevices = 64;
// per-device address of g_nms_static_mask, null = not yet known; atomic because any host thread may be the first
std::atomic<unsigned long long*> g_nms_static_ptr[kMaxStaticDevices];
}  // namespace

extern "C" int d3d_nms3d_enqueue_static(const d3d_nms3d_params* p, const d3d_tensor_desc* in, int n_in,
                                        const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                                        void* const* outputs, void* stream) {
  D3D_NVTX_RANGE("d3d_nms3d_enqueue_static");
  D3D_REQUIRE(p && out && inputs && outputs && n_out >= 1, D3D_ERR_INVALID_ARGUMENT);
  int b, k, bd;
  int rc = nms_dims(in, n_in, &b, &k, &bd);
  if (rc != D3D_OK) return rc;
  if (b == 0 || k == 0) return D3D_OK;
  const int nw = (int)ceil_div(k, kNmsBlock);
  // the scratch is fixed: larger problems are refused, never truncated
  D3D_REQUIRE((size_t)b * k * nw <= (size_t)D3D_NMS3D_STATIC_MAX_WORDS, D3D_ERR_TOO_LARGE);
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxStaticDevices) return D3D_ERR_CUDA;
  unsigned long long* mask = g_nms_static_ptr[dev].load(std::memory_order_acquire);
  if (!mask) {
    void* addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_nms_static_mask) != cudaSuccess || !addr) return D3D_ERR_CUDA;
    mask = reinterpret_cast<unsigned long long*>(addr);
    g_nms_static_ptr[dev].store(mask, std::memory_order_release);  // the same value whichever thread stores it
  }
  // the same launches as the workspace variant, over the built-in scratch
  return launch_nms(p, b, k, bd, nw, inputs, outputs, mask, stream);
}
