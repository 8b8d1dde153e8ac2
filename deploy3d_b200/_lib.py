"""ctypes binding of ``libs/libdeploy3d_b200.so`` (the C ABI declared in ``include/deploy3d_b200.h``).

The reference loads its plugin library the same way: every ``deploy3d/libs/*.so`` through
``ctypes.CDLL`` (deploy3d/symfun/trt_utils/trt_module.py:58-64).  There is no fallback: when the
library is missing or a symbol cannot be resolved, importing code gets an exception.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# DEPLOY3D_B200_CHECKED=1 selects the checked build (python -m deploy3d_b200.build --checked): same entry points,
# every id range-checked before use, first violation recorded (d3d_debug_take_bounds_violation)
LIB_PATH = os.path.join(_HERE, "libs", "libdeploy3d_b200_checked.so" if os.environ.get("DEPLOY3D_B200_CHECKED") == "1"
                        else "libdeploy3d_b200.so")

D3D_MAX_DIMS = 8
D3D_MAX_NDIM = 4

D3D_FLOAT, D3D_HALF, D3D_INT8, D3D_INT32, D3D_BOOL, D3D_BF16 = 0, 1, 2, 3, 4, 7
D3D_STATUS_HASH_FULL, D3D_STATUS_OUTPUT_OVERFLOW = 1, 2


class TensorDesc(ctypes.Structure):
    _fields_ = [("dtype", ctypes.c_int32), ("nb_dims", ctypes.c_int32), ("dims", ctypes.c_int64 * D3D_MAX_DIMS)]


class SpconvIndexParams(ctypes.Structure):
    _fields_ = [("ndim", ctypes.c_int32),
                ("kernel_size", ctypes.c_int32 * D3D_MAX_NDIM),
                ("stride", ctypes.c_int32 * D3D_MAX_NDIM),
                ("padding", ctypes.c_int32 * D3D_MAX_NDIM),
                ("dilation", ctypes.c_int32 * D3D_MAX_NDIM),
                ("out_padding", ctypes.c_int32 * D3D_MAX_NDIM),
                ("max_num_act_out", ctypes.c_int32),
                ("subm", ctypes.c_int32),
                ("transpose", ctypes.c_int32)]


class SpconvIndexExtras(ctypes.Structure):
    _fields_ = [("persistent_buffers", ctypes.c_int32), ("first_call", ctypes.c_int32),
                ("subm_table", ctypes.c_void_p), ("status", ctypes.c_void_p)]


class MeanEncoderExtras(ctypes.Structure):
    _fields_ = [("lp_feats", ctypes.c_void_p), ("lp_dtype", ctypes.c_int32), ("lp_channels", ctypes.c_int32),
                ("status", ctypes.c_void_p)]


class SpconvMMParams(ctypes.Structure):
    _fields_ = [("kernel_vol", ctypes.c_int32), ("in_channels", ctypes.c_int32), ("out_channels", ctypes.c_int32),
                ("max_num_act_out", ctypes.c_int32), ("subm", ctypes.c_int32), ("inverse", ctypes.c_int32),
                ("with_bias", ctypes.c_int32)]


class SpconvMMEpilogue(ctypes.Structure):
    _fields_ = [("relu", ctypes.c_int32), ("residual", ctypes.c_void_p), ("regrouped", ctypes.c_int32)]


class BevDensifyParams(ctypes.Structure):
    _fields_ = [("out_channels", ctypes.c_int32)]


class VoxelEncoderParams(ctypes.Structure):
    _fields_ = [("max_num_act_out", ctypes.c_int32)]


class ScatterToParams(ctypes.Structure):
    _fields_ = [("reduce_type", ctypes.c_int32)]


class GatherBackParams(ctypes.Structure):
    _fields_ = [("fill", ctypes.c_int32), ("fill_val", ctypes.c_float)]


class Nms3dParams(ctypes.Structure):
    _fields_ = [("iou_threshold", ctypes.c_float)]


class YoloX3dDecodeParams(ctypes.Structure):
    _fields_ = [("stride", ctypes.c_int32), ("topk", ctypes.c_int32), ("class_ids", ctypes.c_int32 * 8)]


_vp = ctypes.c_void_p
_sz = ctypes.c_size_t
_descp = ctypes.POINTER(TensorDesc)
_vpp = ctypes.POINTER(ctypes.c_void_p)
_szp = ctypes.POINTER(ctypes.c_size_t)


def _enqueue_sig(params_t):
    return [params_t, _descp, ctypes.c_int, _descp, ctypes.c_int, _vpp, _vpp, _vp, _sz, _vp]


def _workspace_sig(params_t):
    return [params_t, _descp, ctypes.c_int, _szp]


# name -> (restype, argtypes); every function include/deploy3d_b200.h declares
SIGNATURES = {
    "d3d_version": (ctypes.c_char_p, []),
    "d3d_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "d3d_debug_take_kernel_error": (ctypes.c_int, [ctypes.POINTER(ctypes.c_int)]),
    "d3d_spconv_mm_regroup_scratch_bytes": (ctypes.c_size_t, [ctypes.c_int, ctypes.c_int64]),
    "d3d_spconv_mm_regroup": (ctypes.c_int, [ctypes.c_int, ctypes.c_int64, _vp, _vp, _vp, ctypes.c_size_t, _vp]),
    "d3d_debug_take_bounds_violation": (ctypes.c_int, [ctypes.POINTER(ctypes.c_int32)]),
    "d3d_debug_set_tc_plan": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int]),
    "d3d_spconv_index_parse": (ctypes.c_int, [ctypes.c_int, _vp, _sz, ctypes.POINTER(SpconvIndexParams)]),
    "d3d_spconv_index_num_outputs": (ctypes.c_int, [ctypes.POINTER(SpconvIndexParams)]),
    "d3d_spconv_index_output_desc": (ctypes.c_int, [ctypes.POINTER(SpconvIndexParams), _descp, ctypes.c_int,
                                                     ctypes.c_int, _descp]),
    "d3d_spconv_index_workspace": (ctypes.c_int, _workspace_sig(ctypes.POINTER(SpconvIndexParams))),
    "d3d_spconv_index_enqueue": (ctypes.c_int, _enqueue_sig(ctypes.POINTER(SpconvIndexParams))),
    "d3d_spconv_index_subm_table_ok": (ctypes.c_int, [ctypes.POINTER(SpconvIndexParams)]),
    "d3d_spconv_index_enqueue_ex": (ctypes.c_int, _enqueue_sig(ctypes.POINTER(SpconvIndexParams)) +
                                    [ctypes.POINTER(SpconvIndexExtras)]),
    "d3d_spconv_mm_create": (ctypes.c_int, [_vp, _sz, ctypes.POINTER(_vp)]),
    "d3d_spconv_mm_get_params": (ctypes.c_int, [_vp, ctypes.POINTER(SpconvMMParams)]),
    "d3d_spconv_mm_serialize": (ctypes.c_int, [_vp, _vp, _szp]),
    "d3d_spconv_mm_configure": (ctypes.c_int, [_vp, ctypes.c_int]),
    "d3d_spconv_mm_destroy": (ctypes.c_int, [_vp]),
    "d3d_spconv_mm_output_desc": (ctypes.c_int, [_vp, _descp, ctypes.c_int, ctypes.c_int, _descp]),
    "d3d_spconv_mm_workspace": (ctypes.c_int, _workspace_sig(_vp)),
    "d3d_spconv_mm_enqueue": (ctypes.c_int, _enqueue_sig(_vp)),
    "d3d_spconv_mm_table_bytes": (_sz, [ctypes.c_int, ctypes.c_int64]),
    "d3d_spconv_mm_prepare": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int64, _vp, ctypes.c_int64, _vp,
                                              _vp, _vp]),
    "d3d_spconv_mm_run": (ctypes.c_int, [_vp, ctypes.c_int, _vp, ctypes.c_int64, _vp, _vp, _vp,
                                          ctypes.POINTER(SpconvMMEpilogue), _vp]),
    "d3d_spconv_mm_set_kernel": (ctypes.c_int, [_vp, ctypes.c_int]),
    "d3d_spconv_mm_set_dependent_launch": (ctypes.c_int, [_vp, ctypes.c_int]),
    "d3d_bev_densify_parse": (ctypes.c_int, [_vp, _sz, ctypes.POINTER(BevDensifyParams)]),
    "d3d_bev_densify_output_desc": (ctypes.c_int, [ctypes.POINTER(BevDensifyParams), _descp, ctypes.c_int, ctypes.c_int, _descp]),
    "d3d_bev_densify_workspace": (ctypes.c_int, _workspace_sig(ctypes.POINTER(BevDensifyParams))),
    "d3d_bev_densify_enqueue": (ctypes.c_int, _enqueue_sig(ctypes.POINTER(BevDensifyParams))),
    "d3d_simple_mean_encoder_parse": (ctypes.c_int, [_vp, _sz, ctypes.POINTER(VoxelEncoderParams)]),
    "d3d_simple_mean_encoder_output_desc": (ctypes.c_int, [ctypes.POINTER(VoxelEncoderParams), _descp, ctypes.c_int, ctypes.c_int, _descp]),
    "d3d_simple_mean_encoder_workspace": (ctypes.c_int, _workspace_sig(ctypes.POINTER(VoxelEncoderParams))),
    "d3d_simple_mean_encoder_enqueue": (ctypes.c_int, _enqueue_sig(ctypes.POINTER(VoxelEncoderParams))),
    "d3d_simple_mean_encoder_enqueue_ex": (ctypes.c_int, _enqueue_sig(ctypes.POINTER(VoxelEncoderParams)) +
                                           [ctypes.POINTER(MeanEncoderExtras)]),
    "d3d_cylinder_encoder_parse": (ctypes.c_int, [_vp, _sz, ctypes.POINTER(VoxelEncoderParams)]),
    "d3d_cylinder_encoder_output_desc": (ctypes.c_int, [ctypes.POINTER(VoxelEncoderParams), _descp, ctypes.c_int, ctypes.c_int, _descp]),
    "d3d_cylinder_encoder_workspace": (ctypes.c_int, _workspace_sig(ctypes.POINTER(VoxelEncoderParams))),
    "d3d_cylinder_encoder_enqueue": (ctypes.c_int, _enqueue_sig(ctypes.POINTER(VoxelEncoderParams))),
    "d3d_scatter_to_parse": (ctypes.c_int, [_vp, _sz, ctypes.POINTER(ScatterToParams)]),
    "d3d_scatter_to_output_desc": (ctypes.c_int, [ctypes.POINTER(ScatterToParams), _descp, ctypes.c_int, ctypes.c_int, _descp]),
    "d3d_scatter_to_enqueue": (ctypes.c_int, _enqueue_sig(ctypes.POINTER(ScatterToParams))),
    "d3d_gather_back_parse": (ctypes.c_int, [_vp, _sz, ctypes.POINTER(GatherBackParams)]),
    "d3d_gather_back_output_desc": (ctypes.c_int, [ctypes.POINTER(GatherBackParams), _descp, ctypes.c_int, ctypes.c_int, _descp]),
    "d3d_gather_back_enqueue": (ctypes.c_int, _enqueue_sig(ctypes.POINTER(GatherBackParams))),
    "d3d_nms3d_parse": (ctypes.c_int, [_vp, _sz, ctypes.POINTER(Nms3dParams)]),
    "d3d_nms3d_output_desc": (ctypes.c_int, [ctypes.POINTER(Nms3dParams), _descp, ctypes.c_int, ctypes.c_int, _descp]),
    "d3d_nms3d_workspace": (ctypes.c_int, _workspace_sig(ctypes.POINTER(Nms3dParams))),
    "d3d_nms3d_enqueue": (ctypes.c_int, _enqueue_sig(ctypes.POINTER(Nms3dParams))),
    "d3d_yolox3d_decode_parse": (ctypes.c_int, [_vp, _sz, ctypes.POINTER(YoloX3dDecodeParams)]),
    "d3d_yolox3d_decode_num_outputs": (ctypes.c_int, [ctypes.POINTER(YoloX3dDecodeParams)]),
    "d3d_yolox3d_decode_output_desc": (ctypes.c_int, [ctypes.POINTER(YoloX3dDecodeParams), _descp, ctypes.c_int,
                                                      ctypes.c_int, _descp]),
    "d3d_yolox3d_decode_workspace": (ctypes.c_int, _workspace_sig(ctypes.POINTER(YoloX3dDecodeParams))),
    "d3d_yolox3d_decode_enqueue": (ctypes.c_int, _enqueue_sig(ctypes.POINTER(YoloX3dDecodeParams))),
    "d3d_nms3d_enqueue_static": (ctypes.c_int, [ctypes.POINTER(Nms3dParams), _descp, ctypes.c_int, _descp,
                                                 ctypes.c_int, _vpp, _vpp, _vp]),
}

_LIB = None


class D3DError(RuntimeError):
    def __init__(self, fn, status):
        self.status = status
        msg = lib().d3d_status_string(status).decode() if _LIB is not None else str(status)
        super().__init__("%s failed: %s (%d)" % (fn, msg, status))


def lib():
    """The loaded library; raises when it has not been built (``python -m deploy3d_b200.build``)."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("%s is missing: build it with `python -m deploy3d_b200.build`; "
                               "there is no CPU fallback" % LIB_PATH)
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError when the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _LIB = handle
    return _LIB


def use_tuning_build(name):
    """Load ``libs/libdeploy3d_b200_<name>.so`` (``python -m deploy3d_b200.build --tuning <name> ...``) instead of the
    regular library; must be called before anything else touches the library.  For microbench.py only."""
    global LIB_PATH
    if _LIB is not None:
        raise RuntimeError("the library is already loaded")
    LIB_PATH = os.path.join(_HERE, "libs", "libdeploy3d_b200_%s.so" % name)


def check(fn_name, status):
    if status != 0:
        raise D3DError(fn_name, status)


def make_desc(dtype, dims):
    d = TensorDesc()
    d.dtype = dtype
    d.nb_dims = len(dims)
    for i, v in enumerate(dims):
        d.dims[i] = int(v)
    return d


def desc_array(descs):
    return (TensorDesc * max(len(descs), 1))(*descs)


def ptr_array(ptrs):
    return (ctypes.c_void_p * max(len(ptrs), 1))(*[ctypes.c_void_p(p) for p in ptrs])
