/*
 * deploy3d_b200 -- C ABI of the B200-native sparse-convolution hot path.
 *
 * Every entry point is what a TensorRT plugin shell (IPluginV2DynamicExt) of the reference
 * project would bind for the corresponding plugin: <op>_parse  <-> the deserialising
 * constructor, <op>_workspace <-> getWorkspaceSize, <op>_enqueue <-> enqueue.  Tensors are
 * plain device pointers described by d3d_tensor_desc (dtype + dims, dense row-major), in the
 * same order and with the same shapes the reference plugins use.  Citations are
 * file:line inside the reference project (zhanggefan/deploy3d).
 *
 * Conventions
 *   - all functions return D3D_OK (0) or a negative d3d_status;
 *   - no entry point synchronises the stream or reads device memory on the host;
 *     voxel counts stay on the device (the reference blocks on a D2H copy,
 *     trt/spconv/index_trt.cu:207-209, trt/spconv/bev_densify_trt.cu:152-155);
 *   - `stream` is a cudaStream_t passed as void*;
 *   - spatial shapes travel as the dims of zero-element tensors [B, 0, D0, D1, ...]
 *     exactly as in the reference (trt/spconv/index_trt.cu:216-226).
 */
#ifndef DEPLOY3D_B200_H_
#define DEPLOY3D_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define D3D_MAX_DIMS 8
#define D3D_MAX_NDIM 4 /* SPConvIdx1d..4d, trt/spconv/index_trt.cu:279-290 */

typedef enum {
  D3D_OK = 0,
  D3D_ERR_INVALID_ARGUMENT = -1,
  D3D_ERR_UNSUPPORTED_DTYPE = -2, /* enqueue of the reference returns -1 (trt/spconv/mm_trt.cu:204) */
  D3D_ERR_WORKSPACE_TOO_SMALL = -3,
  D3D_ERR_CUDA = -4,
  D3D_ERR_BAD_BLOB = -5, /* truncated data_s; the reference only prints (trt/include/common/refnd.h:279-283) */
  D3D_ERR_TOO_LARGE = -6
} d3d_status;

/* Soft failures: a kernel that has to drop work ORs one of these bits into the device word the caller passed in the
 * `status` field of an extras struct (never a trap, never a host synchronisation; the caller reads and clears the
 * word when it likes).  The reference is silent in both cases: an insert into a full table returns "no slot"
 * (trt/include/common/hash32.h:70) and outputs beyond maxNumActOut are dropped (trt/spconv/index.cu:163-168). */
#define D3D_STATUS_HASH_FULL 1       /* a key found no free slot: its pairs / points were dropped */
#define D3D_STATUS_OUTPUT_OVERFLOW 2 /* more output voxels than maxNumActOut: the surplus was dropped */

/* Values follow nvinfer1::DataType so a plugin shell can pass PluginTensorDesc::type through. */
typedef enum {
  D3D_FLOAT = 0,
  D3D_HALF = 1,
  D3D_INT8 = 2,
  D3D_INT32 = 3,
  D3D_BOOL = 4,
  D3D_BF16 = 7
} d3d_dtype;

/* Mirror of the fields of nvinfer1::PluginTensorDesc the reference reads (format is always kLINEAR). */
typedef struct {
  int32_t dtype;
  int32_t nb_dims;
  int64_t dims[D3D_MAX_DIMS];
} d3d_tensor_desc;

const char* d3d_version(void);
const char* d3d_status_string(int status);
/* Debug aid (no reference counterpart; the reference only prints CUDA errors, trt/include/common/macros.h:14-34):
 * synchronises the device, returns in *code the error word a kernel of this library raised when one of its bounded
 * waits expired (0 = none) and clears it.  The word is one per process: a wait of the tensor-core SPConvMM kernel
 * gives up after about one second of wall clock (far beyond any hand-over of a running kernel; a context that is
 * time-sliced away for longer would trip it too), the CTA then drains, part of the output stays unwritten, and the
 * asynchronous enqueue that launched it has long returned D3D_OK.  Not thread-safe. */
int d3d_debug_take_kernel_error(int* code);
/* Debug aid (no reference counterpart).  A checked build of the library (-DDEPLOY3D_BOUNDS_CHECK) range-checks every
 * row id, table entry and coordinate its kernels index with, skips an access that is out of range and records it:
 * this call synchronises the device, copies {violations seen, site, value, limit of the first} to record[0..3] and
 * clears them.  Sites: 1 / 2 neighbour id in SPConvMM (tensor-core / SIMT kernel), 3 rulebook entry while the
 * neighbour table is built, 4 BEVDensify coordinate, 5 ScatterTo id, 6 GatherBack id, 7 a centre-offset rulebook
 * entry that does not map a row to itself although d3d_spconv_mm_prepare was given the mirror hint (value = gather
 * index, limit = scatter index + 1).  The regular build checks nothing of the kind and returns
 * D3D_ERR_INVALID_ARGUMENT. */
int d3d_debug_take_bounds_violation(int32_t* record);
/* Tuning aid (no reference counterpart): overrides the pipeline plan of the tensor-core SPConvMM kernel for every
 * later launch of the process: kernel offsets per pipeline stage, maximum number of stages, producer warps (4 or 8);
 * 0 = automatic.  Not thread-safe; results do not depend on the plan. */
int d3d_debug_set_tc_plan(int group, int max_stages, int prod_warps);

/* ---------------------------------------------------------------------------------------------
 * SPConvIdx{1,2,3,4}d -- rulebook generation.
 * Replaces spconv::SPConvIdxPlugin<NDim> (trt/spconv/index_trt.cu:52-249) and
 * spconv::func::createSparse{SubM,Conv}Index (trt/spconv/index.cu:253-476).
 * data_s layout (trt/spconv/index_trt.cu:39-50, written by deploy3d/symfun/ops/spconv/spconv_index.py:94-101):
 *   int32 kernelSize[NDim], stride[NDim], padding[NDim], dilation[NDim], outPadding[NDim];
 *   int32 maxNumActOut; bool subM; bool transpose      (packed, 66 bytes for NDim = 3)
 * Inputs : 0 inCoors int32 [maxNumActIn, NDim+1] (b, d0, ...), 1 numActIn int32 [1],
 *          2 inSpatialShape [B, 0, D0, ...] (shape only)
 * Outputs: 0 index int32 [3, kVol*(maxNumActIn+128)] rows gatherIn | scatterOut | kernelOffset,
 *          1 numIndex int32 [1]; when !subM also 2 outCoors int32 [maxNumActOut, NDim+1],
 *          3 numActOut int32 [1], 4 outSpatialShape [B, 0, D0', ...] (shape only).
 * Layout of `index` is bit-identical to the reference: segments of ascending kernel offset, each
 * starting at a multiple of 128, ascending input index inside, every other entry -1.
 * Output voxels of a strided/transposed rulebook are numbered by first touch (smallest
 * inputIndex*kVol + kernelOffset that produces them); the reference's order is hash-slot order.
 * ------------------------------------------------------------------------------------------- */
typedef struct {
  int32_t ndim;
  int32_t kernel_size[D3D_MAX_NDIM];
  int32_t stride[D3D_MAX_NDIM];
  int32_t padding[D3D_MAX_NDIM];
  int32_t dilation[D3D_MAX_NDIM];
  int32_t out_padding[D3D_MAX_NDIM];
  int32_t max_num_act_out;
  int32_t subm;
  int32_t transpose;
} d3d_spconv_index_params;

int d3d_spconv_index_parse(int ndim, const void* data_s, size_t len, d3d_spconv_index_params* p);
/* getNbOutputs (index_trt.cu:97-100) */
int d3d_spconv_index_num_outputs(const d3d_spconv_index_params* p);
/* getOutputDimensions (index_trt.cu:101-152) with concrete dims */
int d3d_spconv_index_output_desc(const d3d_spconv_index_params* p, const d3d_tensor_desc* in, int n_in,
                                 int out_index, d3d_tensor_desc* out);
/* getWorkspaceSize (index_trt.cu:174-187) */
int d3d_spconv_index_workspace(const d3d_spconv_index_params* p, const d3d_tensor_desc* in, int n_in,
                               size_t* bytes);
/* enqueue (index_trt.cu:188-248) */
int d3d_spconv_index_enqueue(const d3d_spconv_index_params* p, const d3d_tensor_desc* in, int n_in,
                             const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                             void* const* outputs, void* workspace, size_t workspace_bytes, void* stream);

/* Optional extras for callers that own their buffers across calls (no reference counterpart; TensorRT owns and
 * reuses a plugin's tensors, so the shells never pass them).
 *  persistent_buffers  the `index` output and the workspace are the same memory as in the previous call with this
 *                      flag and nobody else wrote them in between: the -1 padding beyond the previous rulebook is
 *                      still in place, so only [numIndex, previous numIndex) is refilled instead of the whole tail
 *                      of the three rows.  The bytes of `index` are the same as without the flag.
 *  first_call          with persistent_buffers: nothing is known about the buffers yet (do the full fill).
 *  subm_table          when non-null, a buffer of d3d_spconv_mm_table_bytes(kVol, maxNumActIn) bytes that receives
 *                      the neighbour table d3d_spconv_mm_prepare(kVol, 0, maxNumActIn, index, ..) would build from
 *                      this rulebook, written by the probe kernel itself.  Only for rulebooks for which
 *                      d3d_spconv_index_subm_table_ok() returns 1 (3-D SubM, odd kernel, stride 1, padding =
 *                      dilation * (k - 1) / 2 on every axis: offsets k and kVol-1-k mirror each other,
 *                      tests/spconv/test_spconv.py:101-108) and input coordinates without duplicates. */
typedef struct {
  int32_t persistent_buffers;
  int32_t first_call;
  void* subm_table;
  int32_t* status; /* optional device word that receives D3D_STATUS_* bits (see below), or NULL */
} d3d_spconv_index_extras;
int d3d_spconv_index_subm_table_ok(const d3d_spconv_index_params* p);
int d3d_spconv_index_enqueue_ex(const d3d_spconv_index_params* p, const d3d_tensor_desc* in, int n_in,
                                const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                                void* const* outputs, void* workspace, size_t workspace_bytes, void* stream,
                                const d3d_spconv_index_extras* extras);

/* ---------------------------------------------------------------------------------------------
 * SPConvMM -- gather / GEMM / scatter over the rulebook.
 * Replaces spconv::SPConvMMPlugin (trt/spconv/mm_trt.cu:39-206) and
 * spconv::func::indexedSpConv (trt/spconv/mm.h:35-71).
 * data_s layout (mm_trt.cu:27-37, deploy3d/symfun/ops/spconv/spconv_mm.py:54-63):
 *   int32 kernelVol, inChannels, outChannels, maxNumActOut; bool subM, inverse, withBias;
 *   float weight[kernelVol][inChannels][outChannels]; float bias[outChannels] (if withBias)
 * Inputs : 0 inFeats [maxNumActIn, Cin] half | bf16 | float, 1 numActIn int32[1], 2 numActOut int32[1],
 *          3 index int32 [3, L], 4 numIndex int32[1]
 * Output : 0 outFeats [maxNumActOut, Cout], same dtype as inFeats.
 * The handle owns the host copy of the weights (the plugin object of the reference) and, after
 * d3d_spconv_mm_configure, their device copy in the compute dtype (configurePlugin, mm_trt.cu:127-142).
 * Accumulation is fp32 for every dtype (the reference accumulates in fp16, mm/config_tensorop.h:77).
 * ------------------------------------------------------------------------------------------- */
typedef struct d3d_spconv_mm_s* d3d_spconv_mm_t;

typedef struct {
  int32_t kernel_vol;
  int32_t in_channels;
  int32_t out_channels;
  int32_t max_num_act_out;
  int32_t subm; /* deprecated in the reference, kept for the round trip */
  int32_t inverse;
  int32_t with_bias;
} d3d_spconv_mm_params;

/* Epilogue fused after bias; all zero == the reference plugin (activation is a separate graph op there,
 * tests/cylinder/test_cylinder3d.py:91-92).  `residual` (same dtype/shape as outFeats) is added to the result.
 * relu: 0 none; 1 ReLU after the residual add (residual block); 2 ReLU before it (sum of two activated branches,
 * tests/cylinder/test_cylinder3d.py:113-124).
 * regrouped: a hint, nonzero when `table` went through d3d_spconv_mm_regroup: the kernel then packs the few offsets a
 * tile has left into its pipeline stages instead of walking fixed windows of offsets.  Results do not depend on it. */
typedef struct {
  int32_t relu;
  const void* residual;
  int32_t regrouped;
} d3d_spconv_mm_epilogue;

int d3d_spconv_mm_create(const void* data_s, size_t len, d3d_spconv_mm_t* handle);
int d3d_spconv_mm_get_params(d3d_spconv_mm_t handle, d3d_spconv_mm_params* p);
/* serialize (mm_trt.cu:71-74): writes the blob back; *len receives the size (buffer may be NULL). */
int d3d_spconv_mm_serialize(d3d_spconv_mm_t handle, void* buffer, size_t* len);
/* configurePlugin: convert weights to `dtype` and upload them to the current device (allocates). */
int d3d_spconv_mm_configure(d3d_spconv_mm_t handle, int dtype);
int d3d_spconv_mm_destroy(d3d_spconv_mm_t handle);
/* getOutputDimensions / getOutputDataType (mm_trt.cu:96-105) with concrete dims */
int d3d_spconv_mm_output_desc(d3d_spconv_mm_t handle, const d3d_tensor_desc* in, int n_in, int index,
                              d3d_tensor_desc* out);
/* The reference needs no workspace (mm_trt.cu:143-148); this implementation keeps an
 * output-stationary neighbour table [ceil(maxNumActOut/128), kVol, 128] there. */
int d3d_spconv_mm_workspace(d3d_spconv_mm_t handle, const d3d_tensor_desc* in, int n_in, size_t* bytes);
/* enqueue (mm_trt.cu:149-205) == prepare + run below with the table in `workspace`. */
int d3d_spconv_mm_enqueue(d3d_spconv_mm_t handle, const d3d_tensor_desc* in, int n_in,
                          const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                          void* const* outputs, void* workspace, size_t workspace_bytes, void* stream);
/* Two-step form for callers that run several SPConvMM layers over one rulebook (the reference
 * shares rulebooks through an indice_key dictionary, tests/cylinder/test_cylinder3d.py:52-75):
 * prepare builds the neighbour table once, run consumes it.  `table` must hold
 * d3d_spconv_mm_table_bytes(kVol, maxNumActOut) bytes.
 * `mode`: bit 0 = inverse (swap the gather and scatter rows, trt/spconv/mm_trt.cu:174-177); bit 1 = the caller
 * asserts that the rulebook is a mirror-symmetric SubM rulebook (odd kernel, padding = dilation * (k - 1) / 2 on
 * every axis, so that offset k and kVol-1-k hold each other's pairs with the roles swapped -- the property the
 * reference's test checks, tests/spconv/test_spconv.py:101-108); the table is then written in gather order, which
 * is faster.  The result is the same table.  Precondition the library does not verify: the input coordinates are
 * unique and inside the grid (with duplicates the rulebook is not symmetric and the mirrored build writes a wrong
 * table; the checked build records it, site 7 of d3d_debug_take_bounds_violation).  The plugin-level
 * d3d_spconv_mm_enqueue never sets bit 1. */
size_t d3d_spconv_mm_table_bytes(int kernel_vol, int64_t max_num_act_out);
/* Optional step between prepare and run (no reference counterpart): rebuilds a neighbour table with its outputs
 * grouped by offset mask.  The convolution kernel works on tiles of 128 outputs and spends a pipeline slot, a weight
 * block and its MMAs on every kernel offset that feeds at least one output of the tile; in voxel order that is nearly
 * every offset for every tile.  Sorted by which offsets feed them, outputs with like masks share tiles and most
 * (tile, offset) blocks disappear (LiDAR frames: 27 -> 4..19 per tile).  `table_in` is a table as d3d_spconv_mm_prepare
 * or the SubM probe kernel wrote it, `table_out` a second buffer of d3d_spconv_mm_table_bytes bytes, `scratch`
 * d3d_spconv_mm_regroup_scratch_bytes bytes.  The regrouped table records the output row of every tile row, run writes
 * every row where it belongs and accumulates every output's offsets in the same order: results are bit-identical to
 * those of the plain table.  Worth its three kernels (keys, a radix sort, a gather) when several layers share the
 * rulebook or the rulebook is very sparse.  kernel_vol <= 32. */
size_t d3d_spconv_mm_regroup_scratch_bytes(int kernel_vol, int64_t max_num_act_out);
int d3d_spconv_mm_regroup(int kernel_vol, int64_t max_num_act_out, const void* table_in, void* table_out,
                          void* scratch, size_t scratch_bytes, void* stream);
int d3d_spconv_mm_prepare(int kernel_vol, int mode, int64_t max_num_act_out, const int32_t* index,
                          int64_t index_row_len, const int32_t* num_index, void* table, void* stream);
int d3d_spconv_mm_run(d3d_spconv_mm_t handle, int dtype, const void* in_feats, int64_t max_num_act_in,
                      const int32_t* num_act_out, const void* table, void* out_feats,
                      const d3d_spconv_mm_epilogue* epilogue, void* stream);
/* Kernel choice for tests and profiling: 0 = automatic, 1 = SIMT fp32-FMA path, 2 = tcgen05 tensor-core path (what
 * "automatic" picks for eligible shapes), 3 = tcgen05 path restricted to one CTA per SM (layers of at most 64 input
 * channels otherwise run two half-size CTAs per SM).  2 and 3 fail with D3D_ERR_INVALID_ARGUMENT at run time when
 * the shape is not eligible. */
int d3d_spconv_mm_set_kernel(d3d_spconv_mm_t handle, int which);
/* Opt-in for callers that enqueue layers back to back on ONE stream (as TensorRT does): the tensor-core kernel is
 * launched with the programmatic stream-serialisation attribute, so that its prologue overlaps the tail of the
 * preceding kernel of the stream; it waits for that kernel before reading or writing any tensor.  Results are
 * unchanged.  Off by default: where other streams run kernels beside the layers, those fill the tails better.
 * No reference counterpart. */
int d3d_spconv_mm_set_dependent_launch(d3d_spconv_mm_t handle, int enable);

/* ---------------------------------------------------------------------------------------------
 * BEVDensify.  Replaces spconv::BEVDensifyPlugin (trt/spconv/bev_densify_trt.cu:52-178).
 * data_s: int32 outChannels (= Cin * Z).
 * Inputs : 0 inFeats [maxNumActIn, C] float | half | bf16, 1 inCoors int32 [maxNumActIn, 4] (b,z,y,x),
 *          2 numActIn int32[1], 3 inSpatialShape [B, 0, Z, Y, X]
 * Output : 0 outFeatMaps [B, C*Z, Y, X]
 * ------------------------------------------------------------------------------------------- */
typedef struct {
  int32_t out_channels;
} d3d_bev_densify_params;
int d3d_bev_densify_parse(const void* data_s, size_t len, d3d_bev_densify_params* p);
/* getOutputDimensions / getOutputDataType (bev_densify_trt.cu:93-108) */
int d3d_bev_densify_output_desc(const d3d_bev_densify_params* p, const d3d_tensor_desc* in, int n_in, int index,
                                d3d_tensor_desc* out);
int d3d_bev_densify_workspace(const d3d_bev_densify_params* p, const d3d_tensor_desc* in, int n_in, size_t* bytes);
int d3d_bev_densify_enqueue(const d3d_bev_densify_params* p, const d3d_tensor_desc* in, int n_in,
                            const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                            void* const* outputs, void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * SimpleMeanEncoder.  Replaces voxel_encoder::SimpleMeanEncoderPlugin
 * (trt/voxel_encoder/simple_mean_trt.cu:121-168, :181-314).  data_s: int32 maxNumActOut.
 * Inputs : 0 batchPointFeats float [N, C], 1 batchIndices int32 [N] (<0: ignore point),
 *          2 voxelConfig float [6] = (xmin,ymin,zmin,dx,dy,dz), 3 inSpatialShape [B, 0, Z, Y, X]
 * Outputs: 0 outFeats float [maxNumActOut, C], 1 outCoors int32 [maxNumActOut, 4] (b,z,y,x), 2 numActOut int32[1]
 * Voxels are numbered by first touch (smallest point index); the reference uses hash-slot order.
 * ------------------------------------------------------------------------------------------- */
typedef struct {
  int32_t max_num_act_out;
} d3d_voxel_encoder_params;
int d3d_simple_mean_encoder_parse(const void* data_s, size_t len, d3d_voxel_encoder_params* p);
/* getOutputDimensions / getOutputDataType (simple_mean_trt.cu:220-245) */
int d3d_simple_mean_encoder_output_desc(const d3d_voxel_encoder_params* p, const d3d_tensor_desc* in, int n_in,
                                        int index, d3d_tensor_desc* out);
int d3d_simple_mean_encoder_workspace(const d3d_voxel_encoder_params* p, const d3d_tensor_desc* in, int n_in,
                                      size_t* bytes);
int d3d_simple_mean_encoder_enqueue(const d3d_voxel_encoder_params* p, const d3d_tensor_desc* in, int n_in,
                                    const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                                    void* const* outputs, void* workspace, size_t workspace_bytes, void* stream);
/* Optional extra output (no reference counterpart; in the reference's graph TensorRT inserts a reformat layer
 * between the fp32 encoder and the fp16 convolutions): the voxel means also in half / bfloat16, in rows of
 * lp_channels >= C channels (the additional channels zero), for the live voxels -- the tensor the first SPConvMM
 * reads.  Rows beyond numActOut are left untouched. */
typedef struct {
  void* lp_feats;      /* [maxNumActOut, lp_channels], or NULL */
  int32_t lp_dtype;    /* D3D_HALF or D3D_BF16 */
  int32_t lp_channels; /* >= C */
  int32_t* status;     /* optional device word that receives D3D_STATUS_* bits, or NULL */
} d3d_mean_encoder_extras;
int d3d_simple_mean_encoder_enqueue_ex(const d3d_voxel_encoder_params* p, const d3d_tensor_desc* in, int n_in,
                                       const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                                       void* const* outputs, void* workspace, size_t workspace_bytes, void* stream,
                                       const d3d_mean_encoder_extras* extras);

/* ---------------------------------------------------------------------------------------------
 * CylinderEncoder.  Replaces voxel_encoder::CylinderEncoderPlugin
 * (trt/voxel_encoder/cylinder_trt.cu:130-174, :187-333).  data_s: int32 maxNumActOut.
 * Inputs : 0 batchPointFeats float [N, C], 1 batchIndices int32 [N],
 *          2 cylinderConfig float [6] = (zmin,phimin,rhomin,zmax,phimax,rhomax), 3 inSpatialShape [B, 0, RHO, PHI, Z]
 * Outputs: 0 outFeats float [N, C+5], 1 scatterTo int32 [N], 2 scatterCount int32 [maxNumActOut],
 *          3 outCoors int32 [maxNumActOut, 4] (b,rho,phi,z), 4 numActOut int32[1]
 * ------------------------------------------------------------------------------------------- */
int d3d_cylinder_encoder_parse(const void* data_s, size_t len, d3d_voxel_encoder_params* p);
/* getOutputDimensions / getOutputDataType (cylinder_trt.cu:226-259) */
int d3d_cylinder_encoder_output_desc(const d3d_voxel_encoder_params* p, const d3d_tensor_desc* in, int n_in, int index,
                                     d3d_tensor_desc* out);
int d3d_cylinder_encoder_workspace(const d3d_voxel_encoder_params* p, const d3d_tensor_desc* in, int n_in,
                                   size_t* bytes);
int d3d_cylinder_encoder_enqueue(const d3d_voxel_encoder_params* p, const d3d_tensor_desc* in, int n_in,
                                 const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                                 void* const* outputs, void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * ScatterTo / GatherBack.  Replace point_voxel_mapping::ScatterToPlugin
 * (trt/point_voxel_mapping/scatter_to.cu:83-103, :120-214) and GatherBackPlugin
 * (trt/point_voxel_mapping/gather_back.cu:51-62, :77-184).  Both honour `stream`
 * (the reference launches them on the default stream, scatter_to.cu:212, gather_back.cu:173).
 * ScatterTo  data_s: int8 reduceType (0 max, otherwise mean).
 *   Inputs : 0 batchPointFeats float [N, C], 1 scatterTo int32 [N], 2 scatterCount int32 [M]
 *   Output : 0 reducedFeats float [M, C]
 * GatherBack data_s: bool fill; float fillVal.
 *   Inputs : 0 reducedFeats float [M, ...], 1 scatterTo int32 [N]
 *   Output : 0 batchPointFeats float [N, ...]
 *   Beyond the reference (float only, gather_back.cu:146-150): reducedFeats may be half / bf16, as a
 *   half-precision network writes them; the output is then of the same type (what output_desc reports) or,
 *   when the caller's output descriptor says float, widened while gathering.
 * ------------------------------------------------------------------------------------------- */
typedef struct {
  int32_t reduce_type;
} d3d_scatter_to_params;
typedef struct {
  int32_t fill;
  float fill_val;
} d3d_gather_back_params;
int d3d_scatter_to_parse(const void* data_s, size_t len, d3d_scatter_to_params* p);
/* getOutputDimensions / getOutputDataType (scatter_to.cu:152-160, gather_back.cu:110-120) */
int d3d_scatter_to_output_desc(const d3d_scatter_to_params* p, const d3d_tensor_desc* in, int n_in, int index,
                               d3d_tensor_desc* out);
int d3d_gather_back_output_desc(const d3d_gather_back_params* p, const d3d_tensor_desc* in, int n_in, int index,
                                d3d_tensor_desc* out);
int d3d_scatter_to_enqueue(const d3d_scatter_to_params* p, const d3d_tensor_desc* in, int n_in,
                           const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                           void* const* outputs, void* workspace, size_t workspace_bytes, void* stream);
int d3d_gather_back_parse(const void* data_s, size_t len, d3d_gather_back_params* p);
int d3d_gather_back_enqueue(const d3d_gather_back_params* p, const d3d_tensor_desc* in, int n_in,
                            const d3d_tensor_desc* out, int n_out, const void* const* inputs,
                            void* const* outputs, void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * NMS3d -- rotated-BEV non-maximum suppression.  Replaces decoder::NMS3dPlugin
 * (trt/decoder/nms3d.cu:58-127, :135-236).  The reference has no data_s and hard-codes the
 * IoU threshold 0.1 (nms3d.cu:138); a plugin shell passes iou_threshold = 0.1f.
 * Inputs : 0 inScores float [B, K] sorted descending per row, 1 boxes float [B, K, 7+a] (cx,cy,cz,dx,dy,dz,yaw,..)
 * Output : 0 outScores float [B, K], suppressed entries set to -1.
 * Workspace: B*K*ceil(K/64) 64-bit mask words (same as the reference, nms3d.cu:195-199).
 * ------------------------------------------------------------------------------------------- */
typedef struct {
  float iou_threshold;
} d3d_nms3d_params;
int d3d_nms3d_parse(const void* data_s, size_t len, d3d_nms3d_params* p);
/* getOutputDimensions / getOutputDataType (nms3d.cu:166-176) */
int d3d_nms3d_output_desc(const d3d_nms3d_params* p, const d3d_tensor_desc* in, int n_in, int index,
                          d3d_tensor_desc* out);
int d3d_nms3d_workspace(const d3d_nms3d_params* p, const d3d_tensor_desc* in, int n_in, size_t* bytes);
int d3d_nms3d_enqueue(const d3d_nms3d_params* p, const d3d_tensor_desc* in, int n_in, const d3d_tensor_desc* out,
                      int n_out, const void* const* inputs, void* const* outputs, void* workspace,
                      size_t workspace_bytes, void* stream);
/* NMS3d for callers that cannot supply a workspace and may not allocate device memory (a control loop that forbids
 * allocator calls after start-up, an engine built without plugin workspace, a bare C host with no memory pool).
 * This entry point has no counterpart in the reference.  Same inputs, outputs and results as d3d_nms3d_enqueue; the
 * overlap-mask scratch is a fixed 2 MiB array inside the library (held by every GPU that loads it), so
 * B*K*ceil(K/64) must not exceed D3D_NMS3D_STATIC_MAX_WORDS or the call returns D3D_ERR_TOO_LARGE.  The call
 * performs no device allocation.  The first call on a device resolves the array's device address; make that call
 * before starting a stream capture.  All calls on a GPU share the array: calls that overlap on the GPU race. */
#define D3D_NMS3D_STATIC_MAX_WORDS (256 * 1024)
int d3d_nms3d_enqueue_static(const d3d_nms3d_params* p, const d3d_tensor_desc* in, int n_in,
                             const d3d_tensor_desc* out, int n_out, const void* const* inputs, void* const* outputs,
                             void* stream);

/* ---------------------------------------------------------------------------------------------
 * YoloX3dDecode -- per class, the topK BEV cells by class score, decoded into boxes; the step before NMS3d.
 * Replaces decoder::YoloX3dDecodePlugin (trt/decoder/yolox3d_decode.cu:139-412).
 * data_s (pack(1), :139-145): int32 stride, int32 topk, int32 classIds[8] (unused entries -1).
 * Inputs : 0 cls_scores float/half [B, C, Y, X], 1 bbox_preds same dtype [B, 9+a, Y, X]
 *          (dx, dy, z, log w, log l, log h, yaw, sin, cos, extras), 2 voxel_config float [6] (x_min, y_min, z_min,
 *          voxel size, ..).
 * Outputs: for class i < C: 3i topk_class_ids int32 [B, K], 3i+1 topk_scores float [B, K] (descending; equal scores
 *          in ascending cell order, as the reference's stable sort leaves them; -1 for an invalid box),
 *          3i+2 topk_boxes float [B, K, 7+a]; K = min(topk, Y*X) (:192-206).
 * Workspace: none (the reference sorts all B*C*Y*X scores and needs the cub scratch, :255-298).
 * K above 4096 is refused with D3D_ERR_TOO_LARGE.
 * ------------------------------------------------------------------------------------------- */
typedef struct {
  int32_t stride;
  int32_t topk;
  int32_t class_ids[8];
} d3d_yolox3d_decode_params;
int d3d_yolox3d_decode_parse(const void* data_s, size_t len, d3d_yolox3d_decode_params* p);
int d3d_yolox3d_decode_num_outputs(const d3d_yolox3d_decode_params* p);
int d3d_yolox3d_decode_output_desc(const d3d_yolox3d_decode_params* p, const d3d_tensor_desc* in, int n_in, int index,
                                   d3d_tensor_desc* out);
int d3d_yolox3d_decode_workspace(const d3d_yolox3d_decode_params* p, const d3d_tensor_desc* in, int n_in,
                                 size_t* bytes);
int d3d_yolox3d_decode_enqueue(const d3d_yolox3d_decode_params* p, const d3d_tensor_desc* in, int n_in,
                               const d3d_tensor_desc* out, int n_out, const void* const* inputs, void* const* outputs,
                               void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DEPLOY3D_B200_H_ */
