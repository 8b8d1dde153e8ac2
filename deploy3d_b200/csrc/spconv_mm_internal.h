// Internal contract between the SPConvMM host code (spconv_mm.cu) and its two kernels:
// the SIMT fp32-FMA kernel (any dtype, any channel count) and the tcgen05/TMEM kernel
// (fp16 / bf16, channel counts that are multiples of 16).
#pragma once
#include <stdint.h>
#include <vector>

#include "../../include/deploy3d_b200.h"

struct d3d_spconv_mm_s {
  d3d_spconv_mm_params p;
  std::vector<float> wb;     // host copy: weights [kVol][Cin][Cout] then bias [Cout] (as in the data_s blob)
  int dtype = -1;            // dtype of the device copy, -1 before configure
  int device = -1;
  void* w_dev = nullptr;     // [kVol][Cin][Cout] in `dtype` (reference layout; SIMT kernel)
  void* wt_dev = nullptr;    // [kVol][Cout][Cin] in `dtype` (K-major B operand of the tcgen05 kernel)
  float* b_dev = nullptr;    // bias in fp32 (zeros when the blob has no bias)
  int kernel_choice = 0;     // 0 auto, 1 SIMT, 2 tcgen05
  int dependent_launch = 0;  // tcgen05 path: launch with the programmatic stream-serialisation attribute
  void* tc_state = nullptr;  // tensor map of the tcgen05 path (owned by spconv_mm_tc.cu, created by configure)
};

namespace d3d {

struct MmLaunch {
  const d3d_spconv_mm_s* h;
  int dtype;
  const void* in_feats;
  int64_t max_num_act_in;
  const int32_t* num_act_out;
  // [tiles][kVol][128] input row per (output tile, offset, row in tile); tiles = ceil(max_num_act_out / 128); then
  // one offset mask per tile; then the row masks [tiles][kVol][4] (bit r of word q: row 32 q + r has an input; an id
  // whose bit is clear is unspecified); then the output row of every tile row, int32 [tiles][128] (-1 = none)
  const int32_t* table;
  void* out_feats;
  int relu;
  const void* residual;
  int regrouped;  // hint: the table's outputs were regrouped (few offsets per tile)
  void* stream;
};

// Bytes of the id part of the neighbour table; the per-tile offset masks (one uint32 per tile) start right after.
inline size_t table_ids_bytes(int kernel_vol, int64_t max_num_act_out) {
  const size_t pitch = (size_t)((max_num_act_out + 127) / 128 * 128);
  return ((size_t)kernel_vol * pitch * sizeof(int32_t) + 255) / 256 * 256;
}

// Bytes of the per-tile offset masks; the row masks (four words per (tile, offset)) follow them.
inline size_t table_mask_bytes(int64_t max_num_act_out) {
  const size_t tiles = (size_t)((max_num_act_out + 127) / 128);
  return (tiles * sizeof(uint32_t) + 255) / 256 * 256;
}
inline size_t table_rows_bytes(int kernel_vol, int64_t max_num_act_out) {
  const size_t tiles = (size_t)((max_num_act_out + 127) / 128);
  return (tiles * (size_t)kernel_vol * 4 * sizeof(uint32_t) + 255) / 256 * 256;
}

// The parts of a neighbour table.
struct TableParts {
  int32_t* ids;
  uint32_t* tile_mask;
  uint32_t* row_masks;
  int32_t* perm;
  int64_t tiles;
};
inline TableParts table_parts(void* table, int kernel_vol, int64_t max_num_act_out) {
  TableParts t;
  unsigned char* b = reinterpret_cast<unsigned char*>(table);
  t.tiles = (max_num_act_out + 127) / 128;
  t.ids = reinterpret_cast<int32_t*>(b);
  b += table_ids_bytes(kernel_vol, max_num_act_out);
  t.tile_mask = reinterpret_cast<uint32_t*>(b);
  b += table_mask_bytes(max_num_act_out);
  t.row_masks = reinterpret_cast<uint32_t*>(b);
  b += table_rows_bytes(kernel_vol, max_num_act_out);
  t.perm = reinterpret_cast<int32_t*>(b);
  return t;
}
inline size_t table_perm_bytes(int64_t max_num_act_out) {
  const size_t tiles = (size_t)((max_num_act_out + 127) / 128);
  return (tiles * 128 * sizeof(int32_t) + 255) / 256 * 256;
}

int launch_spconv_mm_simt(const MmLaunch& a);
// Returns D3D_ERR_INVALID_ARGUMENT when the shape/dtype is not eligible for the tensor-core path.
bool spconv_mm_tc_eligible(const d3d_spconv_mm_s* h, int dtype);
int launch_spconv_mm_tc(const MmLaunch& a);
// Per-handle state of the tensor-core path: created while configuring (device weights exist), freed with them.
int spconv_mm_tc_prepare(d3d_spconv_mm_s* h, int dtype);
void spconv_mm_tc_release(d3d_spconv_mm_s* h);

}  // namespace d3d
