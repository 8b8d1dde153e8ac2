/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of deploy3d's sparse-convolution hot path.
 *
 * This file is the checker for the CUDA library, never a product path: only the test-suite,
 * the smoke check and the CPU-baseline leg of the benchmark may load it.  Every function
 * restates, in plain scalar C, what the reference's CUDA code computes and cites the
 * reference file:line it follows (paths are relative to the reference project root).
 *
 * Where the reference's result depends on a race between GPU threads (order of output
 * voxels of a strided convolution, order of voxels of the encoders, order of float
 * atomics) this file reproduces the result of ONE legal schedule: threads run one after
 * the other in ascending index order.  Comparisons against it are therefore made after
 * canonicalisation (see oracle.py).
 *
 * Parity pins: the rotated-IoU arithmetic is checked bit-for-bit against the reference's
 * own trt/decoder/iou_rotated.cuh compiled for the host (oracle/_ref); rulebooks and the
 * convolution are checked against golden vectors the reference's own GPU code (trt/spconv/index.cu,
 * trt/spconv/mm.h compiled for sm_100a) wrote on a B200 (tests/golden/spconv_ref_gpu.npz), and every
 * operator against the reference's plugin classes run on the GPU (tests/test_gpu_reference.py);
 * beside those, the properties the reference's tests assert (tests/spconv/test_spconv.py:72-124)
 * and a brute-force dictionary model of the rulebook.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_MAX_NDIM 4
#define ORC_SEGMENT 128 /* trt/spconv/index.cu:21 TBSegment */

/* ---------------------------------------------------------------------------------------
 * Hash table of the reference: trt/include/common/hash32.h:21-85
 * int32 keys, EMPTY = INT32_MAX, Murmur3 finaliser, linear probing.
 * ------------------------------------------------------------------------------------- */
static inline uint32_t orc_murmur(uint32_t k) { /* hash32.h:23-33 */
  k ^= k >> 16;
  k *= 0x85ebca6bu;
  k ^= k >> 13;
  k *= 0xc2b2ae35u;
  k ^= k >> 16;
  return k;
}

typedef struct {
  int32_t* keys;
  int32_t* vals;
  size_t size;
} orc_hash;

static void orc_hash_reset(orc_hash* h) { /* index.cu:184-186 */
  for (size_t i = 0; i < h->size; i++) h->keys[i] = INT32_MAX;
}

static size_t orc_hash_insert(orc_hash* h, int32_t key, int32_t val) { /* hash32.h:59-71 */
  size_t slot = (size_t)orc_murmur((uint32_t)key) % h->size;
  for (size_t i = 0; i < h->size; i++) {
    if (h->keys[slot] == INT32_MAX || h->keys[slot] == key) {
      h->keys[slot] = key;
      h->vals[slot] = val;
      return slot;
    }
    slot = (slot + 1) % h->size;
  }
  return (size_t)-1;
}

static int orc_hash_lookup(const orc_hash* h, int32_t key, int32_t* val) { /* hash32.h:73-85 */
  size_t slot = (size_t)orc_murmur((uint32_t)key) % h->size;
  for (size_t i = 0; i < h->size; i++) {
    int32_t found = h->keys[slot];
    if (found == key) {
      *val = h->vals[slot];
      return 1;
    }
    if (found == INT32_MAX) return 0;
    slot = (slot + 1) % h->size;
  }
  return 0;
}

static size_t orc_pow2(size_t x) { /* index.cu:209-213 getMinPower2 */
  size_t y = 1;
  while (y < x) y <<= 1;
  return y;
}

/* ---------------------------------------------------------------------------------------
 * Geometry: trt/spconv/geometry.h and trt/include/common/refnd.h
 * ------------------------------------------------------------------------------------- */

/* refnd.h:29-36 is_valid, :48-54 offset; shape[0] is the batch extent. */
static int orc_coor_valid(const int32_t* c, const int64_t* shape, int rank) {
  for (int i = 0; i < rank; i++)
    if (c[i] < 0 || c[i] > shape[i] - 1) return 0;
  return 1;
}
static int64_t orc_coor_offset(const int32_t* c, const int64_t* shape, int rank) {
  int64_t off = c[0];
  for (int i = 1; i < rank; i++) off = off * shape[i] + c[i];
  return off;
}
static void orc_coor_decode(int32_t* c, int64_t off, const int64_t* shape, int rank) { /* refnd.h:56-64 */
  for (int i = rank - 1; i >= 0; i--) {
    c[i] = (int32_t)(off % shape[i]);
    off /= shape[i];
  }
}

/* geometry.h:118-169: spatial extent of the output of a (transposed) convolution.
 * in_shape / out_shape hold [B, D0, .., D(ndim-1)]. */
void orc_out_shape(int ndim, const int64_t* in_shape, const int32_t* ksize, const int32_t* stride,
                   const int32_t* pad, const int32_t* dil, const int32_t* out_pad, int transpose,
                   int64_t* out_shape) {
  out_shape[0] = in_shape[0];
  for (int i = 0; i < ndim; i++) {
    if (transpose) { /* geometry.h:150-153 */
      out_shape[i + 1] =
          (in_shape[i + 1] - 1) * stride[i] - 2 * pad[i] + (ksize[i] - 1) * dil[i] + out_pad[i] + 1;
    } else { /* geometry.h:128-133 */
      int64_t size = (in_shape[i + 1] + 2 * pad[i] - dil[i] * (ksize[i] - 1) - 1) / stride[i] + 1;
      out_shape[i + 1] = ksize[i] == -1 ? 1 : size;
    }
  }
}

/* Callback-free enumeration of geometry.h:28-116 getOutPosLoop: for input voxel `cin`
 * visit every kernel offset k (last dimension fastest) and produce the output coordinate.
 * Returns the number of candidates written; cand_k[j] is the offset id and cand_c[j*(ndim+1)..]
 * the coordinate (not yet bounds-checked). */
static int orc_out_positions(int ndim, const int32_t* cin, const int32_t* ksize, const int32_t* stride,
                             const int32_t* pad, const int32_t* dil, int transpose, int32_t* cand_k,
                             int32_t* cand_c) {
  int kvol = 1;
  for (int i = 0; i < ndim; i++) kvol *= ksize[i];
  int n = 0;
  for (int k = 0; k < kvol; k++) {
    int rem = k, ok = 1;
    int32_t c[ORC_MAX_NDIM + 1];
    c[0] = cin[0];
    for (int i = ndim - 1; i >= 0; i--) {
      int ki = rem % ksize[i];
      rem /= ksize[i];
      if (transpose) { /* geometry.h:66-72 */
        c[i + 1] = cin[i + 1] * stride[i] - pad[i] + ki * dil[i];
      } else { /* geometry.h:41-49 */
        int32_t dc = cin[i + 1] + pad[i] - ki * dil[i];
        if (dc % stride[i] != 0) {
          ok = 0;
          break;
        }
        c[i + 1] = dc / stride[i];
      }
    }
    if (!ok) continue;
    cand_k[n] = k;
    memcpy(cand_c + (size_t)n * (ndim + 1), c, sizeof(int32_t) * (ndim + 1));
    n++;
  }
  return n;
}

/* trt/spconv/index.cu:123-156 (+ the scans at :355-366 / :462-474): turn the table
 * pair_out[k][i] (output id or -1) into the three index rows.  Segments of ascending k,
 * each starting at a multiple of 128, ascending input index inside, -1 everywhere else.
 * index points to [3][row_len]; returns numIndex. */
static int32_t orc_compact_pairs(const int32_t* pair_out, int kvol, int64_t n, int32_t* index, int64_t row_len) {
  int32_t* gather = index;
  int32_t* scatter = index + row_len;
  int32_t* koff = index + 2 * row_len;
  for (int64_t p = 0; p < 3 * row_len; p++) index[p] = -1; /* index.cu:352-354 */
  int64_t pos = 0;
  for (int k = 0; k < kvol; k++) {
    for (int64_t i = 0; i < n; i++) {
      int32_t o = pair_out[(int64_t)k * n + i];
      if (o >= 0) {
        gather[pos] = (int32_t)i;
        scatter[pos] = o;
        koff[pos] = k;
        pos++;
      }
    }
    pos = (pos + ORC_SEGMENT - 1) / ORC_SEGMENT * ORC_SEGMENT; /* index.cu:148-156 */
  }
  return (int32_t)pos; /* index.cu:139-144 */
}

/* trt/spconv/index.cu:400-476 createSparseSubMIndex.
 * coors: [n][ndim+1] (batch first).  shape: [B, D..].  index: [3][row_len] int32.
 * Returns 0, or -1 when the rulebook would not fit row_len. */
int orc_rulebook_subm(int ndim, const int32_t* coors, int64_t n, const int64_t* shape, const int32_t* ksize,
                      const int32_t* stride, const int32_t* pad, const int32_t* dil, int32_t* index,
                      int64_t row_len, int32_t* num_index) {
  int rank = ndim + 1, kvol = 1;
  for (int i = 0; i < ndim; i++) kvol *= ksize[i];
  if (n == 0) { /* index.cu:413-417: only numIndex is written */
    *num_index = 0;
    return 0;
  }
  orc_hash h;
  h.size = orc_pow2((size_t)n * 2); /* index.cu:423 */
  h.keys = (int32_t*)malloc(sizeof(int32_t) * h.size);
  h.vals = (int32_t*)malloc(sizeof(int32_t) * h.size);
  orc_hash_reset(&h);
  for (int64_t i = 0; i < n; i++) /* index.cu:174-182 */
    orc_hash_insert(&h, (int32_t)orc_coor_offset(coors + i * rank, shape, rank), (int32_t)i);
  int32_t* pair_out = (int32_t*)malloc(sizeof(int32_t) * (size_t)kvol * n);
  memset(pair_out, 0xFF, sizeof(int32_t) * (size_t)kvol * n); /* index.cu:449 */
  int32_t* ck = (int32_t*)malloc(sizeof(int32_t) * kvol);
  int32_t* cc = (int32_t*)malloc(sizeof(int32_t) * (size_t)kvol * rank);
  for (int64_t i = 0; i < n; i++) { /* index.cu:69-84, :48-67 */
    int m = orc_out_positions(ndim, coors + i * rank, ksize, stride, pad, dil, 0, ck, cc);
    for (int j = 0; j < m; j++) {
      const int32_t* c = cc + (size_t)j * rank;
      if (!orc_coor_valid(c, shape, rank)) continue;
      int32_t o;
      if (orc_hash_lookup(&h, (int32_t)orc_coor_offset(c, shape, rank), &o)) pair_out[(int64_t)ck[j] * n + i] = o;
    }
  }
  int64_t need = 0;
  for (int k = 0; k < kvol; k++) {
    int64_t c = 0;
    for (int64_t i = 0; i < n; i++) c += pair_out[(int64_t)k * n + i] >= 0;
    need += (c + ORC_SEGMENT - 1) / ORC_SEGMENT * ORC_SEGMENT;
  }
  int rc = 0;
  if (need > row_len) rc = -1;
  else *num_index = orc_compact_pairs(pair_out, kvol, n, index, row_len);
  free(cc), free(ck), free(pair_out), free(h.keys), free(h.vals);
  return rc;
}

/* trt/spconv/index.cu:253-368 createSparseConvIndex (strided and transposed).
 * out_shape: [B, D'..] as given by orc_out_shape.  out_coors: [max_out][ndim+1].
 * Output voxel ids follow the reference: rank of the hash slot among occupied slots
 * (index.cu:330-331), ids >= max_out are dropped (index.cu:158-172). */
int orc_rulebook_conv(int ndim, const int32_t* coors, int64_t n, const int64_t* out_shape, const int32_t* ksize,
                      const int32_t* stride, const int32_t* pad, const int32_t* dil, int transpose,
                      int32_t max_out, int32_t* index, int64_t row_len, int32_t* num_index, int32_t* out_coors,
                      int32_t* num_out) {
  int rank = ndim + 1, kvol = 1;
  for (int i = 0; i < ndim; i++) kvol *= ksize[i];
  if (n == 0) { /* index.cu:270-274 */
    *num_index = 0;
    *num_out = 0;
    return 0;
  }
  orc_hash h;
  h.size = orc_pow2((size_t)kvol * n * 2); /* index.cu:281 */
  h.keys = (int32_t*)malloc(sizeof(int32_t) * h.size);
  h.vals = (int32_t*)calloc(h.size, sizeof(int32_t)); /* index.cu:310 */
  orc_hash_reset(&h);
  uint32_t* slot_of = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)kvol * n);
  memset(slot_of, 0xFF, sizeof(uint32_t) * (size_t)kvol * n); /* index.cu:309 */
  int32_t* ck = (int32_t*)malloc(sizeof(int32_t) * kvol);
  int32_t* cc = (int32_t*)malloc(sizeof(int32_t) * (size_t)kvol * rank);
  for (int64_t i = 0; i < n; i++) { /* index.cu:86-102, :28-46 */
    int m = orc_out_positions(ndim, coors + i * rank, ksize, stride, pad, dil, transpose, ck, cc);
    for (int j = 0; j < m; j++) {
      const int32_t* c = cc + (size_t)j * rank;
      if (!orc_coor_valid(c, out_shape, rank)) continue;
      slot_of[(int64_t)ck[j] * n + i] = (uint32_t)orc_hash_insert(&h, (int32_t)orc_coor_offset(c, out_shape, rank), 1);
    }
  }
  /* index.cu:330-331 exclusive scan of the occupancy flags, :104-121 coordinates */
  int32_t* uid = (int32_t*)malloc(sizeof(int32_t) * h.size);
  int32_t run = 0;
  for (size_t s = 0; s < h.size; s++) {
    uid[s] = run;
    if (h.keys[s] != INT32_MAX) {
      if (run < max_out) orc_coor_decode(out_coors + (size_t)run * rank, h.keys[s], out_shape, rank);
      run += h.vals[s];
    }
  }
  *num_out = run < max_out ? run : max_out; /* index.cu:119 */
  /* index.cu:158-172 slot -> output id, dropping ids beyond max_out */
  int32_t* pair_out = (int32_t*)malloc(sizeof(int32_t) * (size_t)kvol * n);
  for (int64_t e = 0; e < (int64_t)kvol * n; e++) {
    uint32_t s = slot_of[e];
    pair_out[e] = (s < h.size && uid[s] < max_out) ? uid[s] : -1;
  }
  int64_t need = 0;
  for (int k = 0; k < kvol; k++) {
    int64_t c = 0;
    for (int64_t i = 0; i < n; i++) c += pair_out[(int64_t)k * n + i] >= 0;
    need += (c + ORC_SEGMENT - 1) / ORC_SEGMENT * ORC_SEGMENT;
  }
  int rc = 0;
  if (need > row_len) rc = -1;
  else *num_index = orc_compact_pairs(pair_out, kvol, n, index, row_len);
  free(pair_out), free(uid), free(cc), free(ck), free(slot_of), free(h.keys), free(h.vals);
  return rc;
}

/* ---------------------------------------------------------------------------------------
 * Feature computation.  trt/spconv/mm.h:35-71 (bias initialisation then accumulate) with
 * the arithmetic the reference's test uses as ground truth, tests/spconv/test_spconv.py:152-161:
 *   out[:] = bias;  out[scatter[p]] += in[gather[p]] . W[koff[p]]   for p < numIndex, koff[p] >= 0
 * `inverse` swaps the gather and scatter rows (trt/spconv/mm_trt.cu:174-177).
 * Weights: [kvol][cin][cout], cout fastest (tests/cylinder/test_cylinder3d.py:32-36).
 * All arrays are fp32; callers round inputs/weights to fp16 or bf16 beforehand when they
 * model the half-precision plugin path (mm_trt.cu:131-139).  Accumulation is fp32 in pair order.
 * ------------------------------------------------------------------------------------- */
void orc_spconv_mm(const float* in_feats, const float* weight, const float* bias, const int32_t* index,
                   int64_t row_len, int32_t num_index, int inverse, int cin, int cout, float* out_feats,
                   int64_t max_out) {
  const int32_t* gather = index;
  const int32_t* scatter = index + row_len;
  const int32_t* koff = index + 2 * row_len;
  if (inverse) {
    const int32_t* t = gather;
    gather = scatter;
    scatter = t;
  }
  for (int64_t o = 0; o < max_out; o++) /* mm.h:18-25, :51-56 */
    for (int c = 0; c < cout; c++) out_feats[o * cout + c] = bias ? bias[c] : 0.0f;
  for (int32_t p = 0; p < num_index; p++) {
    int32_t k = koff[p];
    if (k < 0) continue; /* padding rows: mm/kernel.h:99-101, input_iterator.h:513-514 */
    int32_t g = gather[p], s = scatter[p];
    if (g < 0 || s < 0 || s >= max_out) continue;
    const float* x = in_feats + (int64_t)g * cin;
    const float* w = weight + (int64_t)k * cin * cout;
    float* y = out_feats + (int64_t)s * cout;
    for (int ci = 0; ci < cin; ci++) {
      float xv = x[ci];
      const float* wr = w + (int64_t)ci * cout;
      for (int c = 0; c < cout; c++) y[c] += xv * wr[c];
    }
  }
}

/* trt/spconv/bev_densify_trt.cu:23-35, :160-163: zero, then out[b][c][z][y][x] = feat[i][c]. */
void orc_bev_densify(const float* feats, const int32_t* coors, int32_t n, int c, int64_t b, int64_t z, int64_t y,
                     int64_t x, float* out) {
  memset(out, 0, sizeof(float) * (size_t)(b * c * z * y * x));
  for (int32_t i = 0; i < n; i++) {
    const int32_t* co = coors + (size_t)i * 4;
    for (int ch = 0; ch < c; ch++)
      out[((((int64_t)co[0] * c + ch) * z + co[1]) * y + co[2]) * x + co[3]] = feats[(size_t)i * c + ch];
  }
}

/* ---------------------------------------------------------------------------------------
 * Voxel encoders.
 * ------------------------------------------------------------------------------------- */
static int orc_all_finite(const float* p, int c) { /* simple_mean_trt.cu:39-41 */
  for (int i = 0; i < c; i++)
    if (!isfinite(p[i])) return 0;
  return 1;
}

/* trt/voxel_encoder/simple_mean_trt.cu:121-168 with kernels :28-102.
 * pts [n][c], batch [n]; cfg = (xmin,ymin,zmin,dx,dy,dz); shape = (B,Z,Y,X).
 * Voxel ids are the rank of the hash slot (table of 2n slots, :133, :157-158); the float sums
 * are taken in point order; voxels beyond max_out are dropped (:75) and the count is clamped (:89). */
void orc_simple_mean(const float* pts, const int32_t* batch, int64_t n, int c, const float* cfg,
                     const int64_t* shape, int64_t max_out, float* out_feats, int32_t* out_coors,
                     int32_t* num_out) {
  memset(out_feats, 0, sizeof(float) * (size_t)max_out * c); /* :148 */
  if (n == 0) {
    *num_out = 0;
    return;
  }
  orc_hash h;
  h.size = (size_t)n * 2;
  h.keys = (int32_t*)malloc(sizeof(int32_t) * h.size);
  h.vals = (int32_t*)calloc(h.size, sizeof(int32_t));
  orc_hash_reset(&h);
  int64_t* slot = (int64_t*)malloc(sizeof(int64_t) * n);
  for (int64_t i = 0; i < n; i++) { /* :28-60 */
    const float* p = pts + i * c;
    slot[i] = -1;
    if (!orc_all_finite(p, c)) continue;
    int32_t co[4];
    co[0] = batch[i];
    if (co[0] < 0) continue;
    co[3] = (int32_t)((p[0] - cfg[0]) / cfg[3]); /* truncation toward zero, :51-53 */
    co[2] = (int32_t)((p[1] - cfg[1]) / cfg[4]);
    co[1] = (int32_t)((p[2] - cfg[2]) / cfg[5]);
    if (!orc_coor_valid(co, shape, 4)) continue;
    slot[i] = (int64_t)orc_hash_insert(&h, (int32_t)orc_coor_offset(co, shape, 4), 1);
  }
  int32_t* rank = (int32_t*)malloc(sizeof(int32_t) * h.size); /* inclusive scan - 1, :157-158, :74 */
  int32_t run = 0;
  for (size_t s = 0; s < h.size; s++) {
    run += h.vals[s];
    rank[s] = run - 1;
  }
  int32_t* count = (int32_t*)calloc((size_t)max_out > 0 ? (size_t)max_out : 1, sizeof(int32_t));
  for (int64_t i = 0; i < n; i++) { /* :62-91 */
    if (slot[i] < 0) continue;
    int32_t v = rank[slot[i]];
    if (v >= max_out) continue;
    if (count[v]++ == 0) orc_coor_decode(out_coors + (size_t)v * 4, h.keys[slot[i]], shape, 4);
    for (int f = 0; f < c; f++) out_feats[(size_t)v * c + f] += pts[i * c + f];
  }
  *num_out = run > max_out ? (int32_t)max_out : run;
  for (int32_t v = 0; v < *num_out; v++) /* :93-102 */
    for (int f = 0; f < c; f++) out_feats[(size_t)v * c + f] = out_feats[(size_t)v * c + f] / (float)count[v];
  free(count), free(rank), free(slot), free(h.keys), free(h.vals);
}

/* trt/voxel_encoder/cylinder_trt.cu:130-174 with kernels :28-111.
 * cfg = (zmin,phimin,rhomin,zmax,phimax,rhomax); shape = (B,RHO,PHI,Z).
 * aug [n][c+5] (zero for dropped points, :162), scatter_to [n] (-1 for dropped, :160),
 * scatter_count [max_out], out_coors [max_out][4] = (b,rho,phi,z). */
void orc_cylinder(const float* pts, const int32_t* batch, int64_t n, int c, const float* cfg, const int64_t* shape,
                  int64_t max_out, float* aug, int32_t* scatter_to, int32_t* scatter_count, int32_t* out_coors,
                  int32_t* num_out) {
  int ca = c + 5;
  memset(aug, 0, sizeof(float) * (size_t)n * ca);
  memset(scatter_count, 0, sizeof(int32_t) * (size_t)max_out);
  for (int64_t i = 0; i < n; i++) scatter_to[i] = -1;
  if (n == 0) {
    *num_out = 0;
    return;
  }
  orc_hash h;
  h.size = (size_t)n * 2;
  h.keys = (int32_t*)malloc(sizeof(int32_t) * h.size);
  h.vals = (int32_t*)calloc(h.size, sizeof(int32_t));
  orc_hash_reset(&h);
  int64_t* slot = (int64_t*)malloc(sizeof(int64_t) * n);
  for (int64_t i = 0; i < n; i++) { /* :28-85 */
    const float* p = pts + i * c;
    float* a = aug + i * ca;
    slot[i] = -1;
    if (!orc_all_finite(p, c)) continue;
    int32_t b = batch[i];
    float x = p[0], y = p[1], z = p[2];
    float rho = sqrtf(x * x + y * y);
    float phi = atan2f(y, x);
    if (b < 0) continue;
    float zmin = cfg[0], phimin = cfg[1], rhomin = cfg[2];
    int64_t rdim = shape[1], pdim = shape[2], zdim = shape[3];
    float zs = (cfg[3] - cfg[0]) / zdim;
    float ps = (cfg[4] - cfg[1]) / pdim;
    float rs = (cfg[5] - cfg[2]) / rdim;
    int32_t zc = (int32_t)((z - zmin) / zs);
    int32_t pc = (int32_t)((phi - phimin) / ps);
    int32_t rc = (int32_t)((rho - rhomin) / rs);
    if (!(pc >= 0 && pc < pdim && rc >= 0 && rc < rdim)) continue;
    zc = zc < 0 ? 0 : zc; /* :64-66 z is clamped, not dropped */
    zc = zc >= zdim ? (int32_t)(zdim - 1) : zc;
    int32_t co[4] = {b, rc, pc, zc};
    slot[i] = (int64_t)orc_hash_insert(&h, (int32_t)orc_coor_offset(co, shape, 4), 1);
    a[0] = z; /* :72-80 */
    a[1] = phi;
    a[2] = rho;
    a[3] = z - ((zc + 0.5f) * zs + zmin);
    a[4] = phi - ((pc + 0.5f) * ps + phimin);
    a[5] = rho - ((rc + 0.5f) * rs + rhomin);
    a[6] = x;
    a[7] = y;
    for (int f = 3; f < c; f++) a[f + 5] = p[f];
  }
  int32_t* rank = (int32_t*)malloc(sizeof(int32_t) * h.size);
  int32_t run = 0;
  for (size_t s = 0; s < h.size; s++) {
    run += h.vals[s];
    rank[s] = run - 1;
  }
  for (int64_t i = 0; i < n; i++) { /* :87-111 */
    if (slot[i] < 0) continue;
    int32_t v = rank[slot[i]];
    if (v >= max_out) continue;
    scatter_to[i] = v;
    if (scatter_count[v]++ == 0) orc_coor_decode(out_coors + (size_t)v * 4, h.keys[slot[i]], shape, 4);
  }
  *num_out = run > max_out ? (int32_t)max_out : run;
  free(rank), free(slot), free(h.keys), free(h.vals);
}

/* trt/point_voxel_mapping/scatter_to.cu:83-103 with kernels :45-79.
 * reduce_type 0: max, initialised to the lowest float (:92-94); otherwise mean as the sum of
 * x / count in point order (:61-75).  All max_out rows are initialised. */
void orc_scatter_to(const float* in_feats, const int32_t* scatter_to, const int32_t* scatter_count, int64_t n, int c,
                    int64_t max_out, int reduce_type, float* out) {
  if (reduce_type == 0) {
    for (int64_t e = 0; e < max_out * c; e++) out[e] = -3.402823466e+38f; /* numeric_limits<float>::lowest() */
    for (int64_t i = 0; i < n; i++) {
      int32_t v = scatter_to[i];
      if (v < 0) continue;
      for (int f = 0; f < c; f++) {
        float x = in_feats[i * c + f];
        if (x > out[(int64_t)v * c + f]) out[(int64_t)v * c + f] = x;
      }
    }
  } else {
    memset(out, 0, sizeof(float) * (size_t)max_out * c);
    for (int64_t i = 0; i < n; i++) {
      int32_t v = scatter_to[i];
      if (v < 0) continue;
      for (int f = 0; f < c; f++) out[(int64_t)v * c + f] += in_feats[i * c + f] / (float)scatter_count[v];
    }
  }
}

/* trt/point_voxel_mapping/gather_back.cu:28-47: out[p] = in[idx[p]]; rows with idx < 0 are
 * written only when `fill` is set (otherwise left untouched). */
void orc_gather_back(const float* in_feats, const int32_t* scatter_to, int64_t n, int64_t c, int fill, float fill_val,
                     float* out) {
  for (int64_t i = 0; i < n; i++) {
    int32_t v = scatter_to[i];
    for (int64_t f = 0; f < c; f++) {
      if (v < 0) {
        if (fill) out[i * c + f] = fill_val;
      } else {
        out[i * c + f] = in_feats[(int64_t)v * c + f];
      }
    }
  }
}

/* ---------------------------------------------------------------------------------------
 * Rotated-BEV NMS.  Intersection area of two rotated rectangles restated from
 * trt/decoder/iou_rotated.cuh:36-234 (same operations in the same order, fp32, trig in
 * double precision as at :39-41); IoU and suppression from trt/decoder/nms3d.cu:32-127.
 * Compile with -ffp-contract=off so no multiply-add is fused.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  float x, y;
} orc_pt;

static inline float orc_cross(orc_pt a, orc_pt b) { return a.x * b.y - b.x * a.y; } /* iou_rotated.cuh:26-28 */
static inline float orc_dot(orc_pt a, orc_pt b) { return a.x * b.x + a.y * b.y; }   /* :22-24 */
static inline orc_pt orc_sub(orc_pt a, orc_pt b) {
  orc_pt r = {a.x - b.x, a.y - b.y};
  return r;
}

static void orc_corners(float cx, float cy, float w, float hgt, float ang, orc_pt* p) { /* :30-49 */
  double theta = ang;
  float c2 = (float)cos(theta) * 0.5f;
  float s2 = (float)sin(theta) * 0.5f;
  p[0].x = cx - s2 * hgt - c2 * w;
  p[0].y = cy + c2 * hgt - s2 * w;
  p[1].x = cx + s2 * hgt - c2 * w;
  p[1].y = cy - c2 * hgt - s2 * w;
  p[2].x = 2 * cx - p[0].x;
  p[2].y = 2 * cy - p[0].y;
  p[3].x = 2 * cx - p[1].x;
  p[3].y = 2 * cy - p[1].y;
}

static int orc_clip_points(const orc_pt* a, const orc_pt* b, orc_pt* out) { /* :51-122 */
  orc_pt ea[4], eb[4];
  for (int i = 0; i < 4; i++) {
    ea[i] = orc_sub(a[(i + 1) % 4], a[i]);
    eb[i] = orc_sub(b[(i + 1) % 4], b[i]);
  }
  int num = 0;
  for (int i = 0; i < 4; i++) { /* edge-edge crossings, :63-81 */
    for (int j = 0; j < 4; j++) {
      float det = orc_cross(eb[j], ea[i]);
      if (fabs((double)det) <= 1e-14) continue;
      orc_pt d = orc_sub(b[j], a[i]);
      float t1 = orc_cross(eb[j], d) / det;
      float t2 = orc_cross(ea[i], d) / det;
      if (t1 >= 0.0f && t1 <= 1.0f && t2 >= 0.0f && t2 <= 1.0f) {
        out[num].x = a[i].x + ea[i].x * t1;
        out[num].y = a[i].y + ea[i].y * t1;
        num++;
      }
    }
  }
  { /* corners of a inside b, :84-103 */
    orc_pt ab = eb[0], da = eb[3];
    float abab = orc_dot(ab, ab), adad = orc_dot(da, da);
    for (int i = 0; i < 4; i++) {
      orc_pt ap = orc_sub(a[i], b[0]);
      float apab = orc_dot(ap, ab), apad = -orc_dot(ap, da);
      if (apab >= 0 && apad >= 0 && apab <= abab && apad <= adad) out[num++] = a[i];
    }
  }
  { /* corners of b inside a, :106-119 */
    orc_pt ab = ea[0], da = ea[3];
    float abab = orc_dot(ab, ab), adad = orc_dot(da, da);
    for (int i = 0; i < 4; i++) {
      orc_pt ap = orc_sub(b[i], a[0]);
      float apab = orc_dot(ap, ab), apad = -orc_dot(ap, da);
      if (apab >= 0 && apad >= 0 && apab <= abab && apad <= adad) out[num++] = b[i];
    }
  }
  return num;
}

static int orc_hull(const orc_pt* p, int n, orc_pt* q) { /* :124-199, shift_to_zero = true */
  int t = 0;
  for (int i = 1; i < n; i++)
    if (p[i].y < p[t].y || (p[i].y == p[t].y && p[i].x < p[t].x)) t = i;
  orc_pt start = p[t];
  for (int i = 0; i < n; i++) q[i] = orc_sub(p[i], start);
  orc_pt tmp = q[0];
  q[0] = q[t];
  q[t] = tmp;
  float dist[24];
  for (int i = 0; i < n; i++) dist[i] = orc_dot(q[i], q[i]);
  for (int i = 1; i < n - 1; i++) { /* exchange sort by polar angle, :152-165 */
    for (int j = i + 1; j < n; j++) {
      float cr = orc_cross(q[i], q[j]);
      if (((double)cr < -1e-6) || (fabs((double)cr) < 1e-6 && dist[i] > dist[j])) {
        orc_pt qt = q[i];
        q[i] = q[j];
        q[j] = qt;
        float dt = dist[i];
        dist[i] = dist[j];
        dist[j] = dt;
      }
    }
  }
  int k;
  for (k = 1; k < n; k++)
    if ((double)dist[k] > 1e-8) break;
  if (k == n) {
    q[0] = p[t];
    return 1;
  }
  q[1] = q[k];
  int m = 2;
  for (int i = k + 1; i < n; i++) { /* Graham scan, :185-188 */
    while (m > 1 && orc_cross(orc_sub(q[i], q[m - 2]), orc_sub(q[m - 1], q[m - 2])) >= 0) m--;
    q[m++] = q[i];
  }
  return m;
}

/* iou_rotated.cuh:215-234 */
float orc_rotated_intersection(float cx1, float cy1, float w1, float h1, float a1, float cx2, float cy2, float w2,
                               float h2, float a2) {
  orc_pt pa[4], pb[4], pts[24], hull[24];
  orc_corners(cx1, cy1, w1, h1, a1, pa);
  orc_corners(cx2, cy2, w2, h2, a2, pb);
  int n = orc_clip_points(pa, pb, pts);
  if (n <= 2) return 0.0f;
  int m = orc_hull(pts, n, hull);
  if (m <= 2) return 0.0f; /* :201-203 */
  float area = 0;
  for (int i = 1; i < m - 1; i++) /* :205-208 */
    area += (float)fabs((double)orc_cross(orc_sub(hull[i], hull[0]), orc_sub(hull[i + 1], hull[0])));
  return (float)((double)area / 2.0);
}

/* nms3d.cu:32-56: BEV IoU of boxes [cx,cy,cz,dx,dy,dz,yaw,...]; z extent ignored. */
float orc_bev_iou(const float* a, const float* b) {
  float va = a[3] * a[4], vb = b[3] * b[4];
  float ov = orc_rotated_intersection(a[0], a[1], a[3], a[4], a[6], b[0], b[1], b[3], b[4], b[6]);
  return ov / fmaxf(va + vb - ov, 1e-8f);
}

/* nms3d.cu:58-127, :200-236: scores [b][k] pre-sorted descending, boxes [b][k][box_dim].
 * A box is suppressed (score := -1) when an earlier kept box overlaps it with IoU >= thr. */
void orc_nms3d(const float* scores, const float* boxes, int nb, int k, int box_dim, float thr, float* out_scores) {
  uint8_t* dead = (uint8_t*)malloc((size_t)k > 0 ? (size_t)k : 1);
  for (int b = 0; b < nb; b++) {
    const float* bx = boxes + (size_t)b * k * box_dim;
    memset(dead, 0, (size_t)k);
    for (int i = 0; i < k; i++) {
      out_scores[(size_t)b * k + i] = scores[(size_t)b * k + i];
      if (dead[i]) {
        out_scores[(size_t)b * k + i] = -1.0f;
        continue;
      }
      for (int j = i + 1; j < k; j++)
        if (!dead[j] && orc_bev_iou(bx + (size_t)i * box_dim, bx + (size_t)j * box_dim) >= thr) dead[j] = 1;
    }
  }
  free(dead);
}
