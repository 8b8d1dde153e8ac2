// getOutputDimensions / getOutputDataType of the plugins whose outputs are plain functions of the input
// descriptors, with concrete dims: one source for the TensorRT shells (which state the same rules as symbolic
// expressions) and for the Python plugin objects.  Host code only.
#include <string.h>

#include "common.cuh"
#include "spconv_mm_internal.h"

using namespace d3d;

namespace {
void set_desc(d3d_tensor_desc* out, int dtype, int nb, int64_t d0, int64_t d1 = 0, int64_t d2 = 0, int64_t d3 = 0) {
  memset(out, 0, sizeof(*out));
  out->dtype = dtype, out->nb_dims = nb;
  out->dims[0] = d0, out->dims[1] = d1, out->dims[2] = d2, out->dims[3] = d3;
}
}  // namespace

// SPConvMM: [maxNumActOut, outChannels] in the dtype of inFeats (trt/spconv/mm_trt.cu:96-105).
extern "C" int d3d_spconv_mm_output_desc(d3d_spconv_mm_t h, const d3d_tensor_desc* in, int n_in, int index,
                                         d3d_tensor_desc* out) {
  D3D_REQUIRE(h && in && out && n_in >= 1 && index == 0, D3D_ERR_INVALID_ARGUMENT);
  set_desc(out, in[0].dtype, 2, h->p.max_num_act_out, h->p.out_channels);
  return D3D_OK;
}

// BEVDensify: [B, outChannels, Y, X] from inSpatialShape [B, 0, Z, Y, X], dtype of inFeats
// (trt/spconv/bev_densify_trt.cu:93-108).
extern "C" int d3d_bev_densify_output_desc(const d3d_bev_densify_params* p, const d3d_tensor_desc* in, int n_in,
                                           int index, d3d_tensor_desc* out) {
  D3D_REQUIRE(p && in && out && n_in >= 4 && index == 0 && in[3].nb_dims >= 5, D3D_ERR_INVALID_ARGUMENT);
  set_desc(out, in[0].dtype, 4, in[3].dims[0], p->out_channels, in[3].dims[3], in[3].dims[4]);
  return D3D_OK;
}

// SimpleMeanEncoder: outFeats = input shape with dim 0 = maxNumActOut, outCoors [maxNumActOut, 4], numActOut [1]
// (trt/voxel_encoder/simple_mean_trt.cu:220-245).
extern "C" int d3d_simple_mean_encoder_output_desc(const d3d_voxel_encoder_params* p, const d3d_tensor_desc* in,
                                                   int n_in, int index, d3d_tensor_desc* out) {
  D3D_REQUIRE(p && in && out && n_in >= 1, D3D_ERR_INVALID_ARGUMENT);
  switch (index) {
    case 0:
      *out = in[0];
      out->dims[0] = p->max_num_act_out;
      return D3D_OK;
    case 1: set_desc(out, D3D_INT32, 2, p->max_num_act_out, 4); return D3D_OK;
    case 2: set_desc(out, D3D_INT32, 1, 1); return D3D_OK;
    default: return D3D_ERR_INVALID_ARGUMENT;
  }
}

// CylinderEncoder: outFeats [N, C + 5], scatterTo [N], scatterCount [maxNumActOut], outCoors [maxNumActOut, 4],
// numActOut [1] (trt/voxel_encoder/cylinder_trt.cu:226-259).
extern "C" int d3d_cylinder_encoder_output_desc(const d3d_voxel_encoder_params* p, const d3d_tensor_desc* in, int n_in,
                                                int index, d3d_tensor_desc* out) {
  D3D_REQUIRE(p && in && out && n_in >= 1 && in[0].nb_dims >= 2, D3D_ERR_INVALID_ARGUMENT);
  switch (index) {
    case 0: set_desc(out, in[0].dtype, 2, in[0].dims[0], in[0].dims[1] + 5); return D3D_OK;
    case 1: set_desc(out, D3D_INT32, 1, in[0].dims[0]); return D3D_OK;
    case 2: set_desc(out, D3D_INT32, 1, p->max_num_act_out); return D3D_OK;
    case 3: set_desc(out, D3D_INT32, 2, p->max_num_act_out, 4); return D3D_OK;
    case 4: set_desc(out, D3D_INT32, 1, 1); return D3D_OK;
    default: return D3D_ERR_INVALID_ARGUMENT;
  }
}

// ScatterTo: [M, C] with M from scatterCount, C from batchPointFeats (trt/point_voxel_mapping/scatter_to.cu:152-160).
extern "C" int d3d_scatter_to_output_desc(const d3d_scatter_to_params* p, const d3d_tensor_desc* in, int n_in,
                                          int index, d3d_tensor_desc* out) {
  D3D_REQUIRE(p && in && out && n_in >= 3 && index == 0 && in[0].nb_dims >= 2, D3D_ERR_INVALID_ARGUMENT);
  set_desc(out, in[0].dtype, 2, in[2].dims[0], in[0].dims[1]);
  return D3D_OK;
}

// GatherBack: reducedFeats' shape with dim 0 = N of scatterTo (trt/point_voxel_mapping/gather_back.cu:110-120).
extern "C" int d3d_gather_back_output_desc(const d3d_gather_back_params* p, const d3d_tensor_desc* in, int n_in,
                                           int index, d3d_tensor_desc* out) {
  D3D_REQUIRE(p && in && out && n_in >= 2 && index == 0, D3D_ERR_INVALID_ARGUMENT);
  *out = in[0];
  out->dims[0] = in[1].dims[0];
  return D3D_OK;
}

// NMS3d: outScores has the shape of inScores, float (trt/decoder/nms3d.cu:166-176).
extern "C" int d3d_nms3d_output_desc(const d3d_nms3d_params* p, const d3d_tensor_desc* in, int n_in, int index,
                                     d3d_tensor_desc* out) {
  D3D_REQUIRE(p && in && out && n_in >= 1 && index == 0, D3D_ERR_INVALID_ARGUMENT);
  *out = in[0];
  out->dtype = D3D_FLOAT;
  return D3D_OK;
}
