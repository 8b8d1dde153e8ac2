"""Plugin objects: the host-side mirror of the reference's TensorRT plugin classes, over the C ABI.

Each class corresponds to one ``IPluginV2DynamicExt`` of the reference, is created the only way the
reference creates plugins -- from the plugin name and the serialized ``data_s`` blob
(``IPluginCreator::deserializePlugin``, e.g. trt/spconv/index_trt.cu:270-275) -- and exposes
``output_descs`` (getOutputDimensions / getOutputDataType), ``workspace_size`` (getWorkspaceSize) and
``enqueue``.  Tensors are torch CUDA tensors used purely as device buffers; the work happens in
``libdeploy3d_b200.so``.  TensorRT itself is not involved, so these objects double as the test harness
the reference implements with ``TRTPluginModule`` (deploy3d/symfun/trt_utils/trt_module.py:99-140).
"""
import ctypes

import numpy as np
import torch

from . import _lib
from ._lib import (D3D_BF16, D3D_FLOAT, D3D_HALF, D3D_INT32, check, desc_array, lib, make_desc, ptr_array)

PLUGIN_VERSION = "2.0"  # e.g. trt/spconv/index_trt.cu:24

_TORCH2D3D = {torch.float32: D3D_FLOAT, torch.float16: D3D_HALF, torch.int32: D3D_INT32, torch.bfloat16: D3D_BF16,
              torch.int8: _lib.D3D_INT8, torch.bool: _lib.D3D_BOOL}
_D3D2TORCH = {v: k for k, v in _TORCH2D3D.items()}


def _desc_of(t):
    if t.dtype not in _TORCH2D3D:
        raise TypeError("unsupported tensor dtype %s" % t.dtype)
    return make_desc(_TORCH2D3D[t.dtype], tuple(t.shape))


def _stream_ptr(stream):
    if stream is None:
        stream = torch.cuda.current_stream()
    return ctypes.c_void_p(stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream))


class _Plugin:
    """Common enqueue plumbing: descriptors, output allocation, workspace, status check."""
    name = None
    version = PLUGIN_VERSION
    _prefix = None

    def __init__(self):
        self._workspace = None

    # -- to be provided by subclasses
    def _params_ref(self):
        raise NotImplementedError

    num_outputs = 1

    def output_descs(self, in_descs):
        """getOutputDimensions / getOutputDataType, from the library (one source with the TensorRT shells)."""
        fn = getattr(lib(), self._prefix + "_output_desc")
        outs = []
        for i in range(self.num_outputs):
            d = _lib.TensorDesc()
            check(self._prefix + "_output_desc", fn(self._params_ref(), desc_array(in_descs), len(in_descs), i,
                                                    ctypes.byref(d)))
            outs.append(d)
        return outs

    def workspace_size(self, in_descs):
        fn = getattr(lib(), self._prefix + "_workspace", None)
        if fn is None:
            return 0
        n = ctypes.c_size_t(0)
        check(self._prefix + "_workspace", fn(self._params_ref(), desc_array(in_descs), len(in_descs),
                                              ctypes.byref(n)))
        return int(n.value)

    def _get_workspace(self, nbytes, device):
        if nbytes == 0:
            return None
        if self._workspace is None or self._workspace.numel() < nbytes or self._workspace.device != device:
            self._workspace = torch.empty(nbytes, dtype=torch.uint8, device=device)
        return self._workspace

    def enqueue(self, *inputs, outputs=None, stream=None):
        """Runs the plugin on the current (or given) CUDA stream and returns the tuple of output tensors."""
        if not inputs or not inputs[0].is_cuda:
            raise RuntimeError("%s: inputs must be CUDA tensors; this library has no CPU path" % self.name)
        inputs = [t if t.is_contiguous() else t.contiguous() for t in inputs]
        device = inputs[0].device
        in_descs = [_desc_of(t) for t in inputs]
        out_descs = self.output_descs(in_descs)
        if outputs is None:
            outputs = [torch.empty(tuple(d.dims[:d.nb_dims]), dtype=_D3D2TORCH[d.dtype], device=device)
                       for d in out_descs]
        else:  # the caller's buffers say which of the accepted output types it wants (GatherBack can widen)
            for d, t in zip(out_descs, outputs):
                d.dtype = _TORCH2D3D[t.dtype]
        ws_bytes = self.workspace_size(in_descs)
        ws = self._get_workspace(ws_bytes, device)
        fn = getattr(lib(), self._prefix + "_enqueue")
        with torch.cuda.device(device):
            status = fn(self._params_ref(), desc_array(in_descs), len(in_descs), desc_array(out_descs),
                        len(out_descs), ptr_array([t.data_ptr() for t in inputs]),
                        ptr_array([t.data_ptr() for t in outputs]),
                        ctypes.c_void_p(ws.data_ptr() if ws is not None else 0), ctypes.c_size_t(ws_bytes),
                        _stream_ptr(stream))
        check(self._prefix + "_enqueue", status)
        return tuple(outputs)


class SPConvIdxPlugin(_Plugin):
    """``SPConvIdx{1,2,3,4}d`` (trt/spconv/index_trt.cu:52-249)."""
    _prefix = "d3d_spconv_index"

    def __init__(self, name, data_s):
        super().__init__()
        self.name = name
        ndim = int(name[len("SPConvIdx")])
        self.p = _lib.SpconvIndexParams()
        buf = ctypes.create_string_buffer(bytes(data_s), len(data_s))
        check("d3d_spconv_index_parse", lib().d3d_spconv_index_parse(ndim, buf, len(data_s), ctypes.byref(self.p)))

    def _params_ref(self):
        return ctypes.byref(self.p)

    def output_descs(self, in_descs):
        n = lib().d3d_spconv_index_num_outputs(ctypes.byref(self.p))
        outs = []
        for i in range(n):
            d = _lib.TensorDesc()
            check("d3d_spconv_index_output_desc",
                  lib().d3d_spconv_index_output_desc(ctypes.byref(self.p), desc_array(in_descs), len(in_descs), i,
                                                     ctypes.byref(d)))
            outs.append(d)
        return outs


    def subm_table_ok(self):
        """True when enqueue_ex can write SPConvMM's neighbour table itself (mirror-symmetric 3-D SubM rulebook)."""
        return bool(lib().d3d_spconv_index_subm_table_ok(ctypes.byref(self.p)))

    def enqueue_ex(self, *inputs, outputs, persistent=False, first_call=True, subm_table=None, status=None,
                   stream=None):
        """enqueue for a caller that owns its buffers across calls: `persistent` refills only the stale part of the
        -1 padding (same bytes in `index`), `subm_table` receives the neighbour table of a mirror-symmetric SubM
        rulebook straight from the probe kernel.  `outputs` must be given (they are the persistent buffers)."""
        inputs = [t if t.is_contiguous() else t.contiguous() for t in inputs]
        device = inputs[0].device
        in_descs = [_desc_of(t) for t in inputs]
        out_descs = self.output_descs(in_descs)
        ws_bytes = self.workspace_size(in_descs)
        ws = self._get_workspace(ws_bytes, device)
        extras = _lib.SpconvIndexExtras(int(bool(persistent)), int(bool(first_call)),
                                        subm_table.data_ptr() if subm_table is not None else None,
                                        status.data_ptr() if status is not None else None)
        with torch.cuda.device(device):
            status = lib().d3d_spconv_index_enqueue_ex(
                ctypes.byref(self.p), desc_array(in_descs), len(in_descs), desc_array(out_descs), len(out_descs),
                ptr_array([t.data_ptr() for t in inputs]), ptr_array([t.data_ptr() for t in outputs]),
                ctypes.c_void_p(ws.data_ptr() if ws is not None else 0), ctypes.c_size_t(ws_bytes),
                _stream_ptr(stream), ctypes.byref(extras))
        check("d3d_spconv_index_enqueue_ex", status)
        return tuple(outputs)


class SPConvMMPlugin(_Plugin):
    """``SPConvMM`` (trt/spconv/mm_trt.cu:39-206); owns the weight handle."""
    name = "SPConvMM"
    _prefix = "d3d_spconv_mm"

    def __init__(self, name, data_s):
        super().__init__()
        self.handle = ctypes.c_void_p(0)
        buf = ctypes.create_string_buffer(bytes(data_s), len(data_s))
        check("d3d_spconv_mm_create", lib().d3d_spconv_mm_create(buf, len(data_s), ctypes.byref(self.handle)))
        self.p = _lib.SpconvMMParams()
        check("d3d_spconv_mm_get_params", lib().d3d_spconv_mm_get_params(self.handle, ctypes.byref(self.p)))

    def __del__(self):
        try:
            if getattr(self, "handle", None) and self.handle.value:
                lib().d3d_spconv_mm_destroy(self.handle)
                self.handle = ctypes.c_void_p(0)
        except Exception:
            pass

    def _params_ref(self):
        return self.handle

    def serialize(self):
        n = ctypes.c_size_t(0)
        check("d3d_spconv_mm_serialize", lib().d3d_spconv_mm_serialize(self.handle, None, ctypes.byref(n)))
        buf = ctypes.create_string_buffer(n.value)
        check("d3d_spconv_mm_serialize", lib().d3d_spconv_mm_serialize(self.handle, buf, ctypes.byref(n)))
        return buf.raw

    def enqueue(self, *inputs, outputs=None, stream=None):
        """configurePlugin for the dtype of ``inFeats`` (a no-op when already done), then enqueue: the C entry
        point itself refuses a handle that was not configured, as it may not allocate."""
        with torch.cuda.device(inputs[0].device):
            self.configure(inputs[0].dtype)
        return super().enqueue(*inputs, outputs=outputs, stream=stream)

    def configure(self, torch_dtype):
        """configurePlugin: upload the weights in the compute dtype (trt/spconv/mm_trt.cu:127-142)."""
        check("d3d_spconv_mm_configure", lib().d3d_spconv_mm_configure(self.handle, _TORCH2D3D[torch_dtype]))

    def set_kernel(self, which):
        """0 automatic, 1 SIMT, 2 tcgen05, 3 tcgen05 with one CTA per SM."""
        check("d3d_spconv_mm_set_kernel", lib().d3d_spconv_mm_set_kernel(self.handle, int(which)))

    def set_dependent_launch(self, enable):
        """Programmatic dependent launch of the tensor-core kernel, for layers enqueued back to back on one stream."""
        check("d3d_spconv_mm_set_dependent_launch",
              lib().d3d_spconv_mm_set_dependent_launch(self.handle, int(bool(enable))))

    # two-step form: one neighbour table shared by all layers over the same rulebook
    @staticmethod
    def table_bytes(kernel_vol, max_num_act_out):
        return int(lib().d3d_spconv_mm_table_bytes(int(kernel_vol), int(max_num_act_out)))

    @staticmethod
    def prepare(kernel_vol, inverse, max_num_act_out, index, num_index, table=None, stream=None, mirror=False):
        """`mirror`: the rulebook is a mirror-symmetric SubM rulebook (same table, faster build)."""
        nbytes = SPConvMMPlugin.table_bytes(kernel_vol, max_num_act_out)
        if table is None:
            table = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=index.device)
        assert table.numel() >= nbytes
        with torch.cuda.device(index.device):
            check("d3d_spconv_mm_prepare",
                  lib().d3d_spconv_mm_prepare(int(kernel_vol), int(bool(inverse)) | (2 if mirror else 0),
                                              int(max_num_act_out),
                                              ctypes.c_void_p(index.data_ptr()), int(index.shape[1]),
                                              ctypes.c_void_p(num_index.data_ptr()),
                                              ctypes.c_void_p(table.data_ptr()), _stream_ptr(stream)))
        return table

    @staticmethod
    def regroup_scratch_bytes(kernel_vol, max_num_act_out):
        return int(lib().d3d_spconv_mm_regroup_scratch_bytes(int(kernel_vol), int(max_num_act_out)))

    @staticmethod
    def regroup(kernel_vol, max_num_act_out, table_in, table_out=None, scratch=None, stream=None):
        """The table with its outputs grouped by offset mask (d3d_spconv_mm_regroup): same results from `run`, fewer
        (tile, offset) blocks for it to walk.  Returns table_out."""
        nbytes = SPConvMMPlugin.table_bytes(kernel_vol, max_num_act_out)
        sbytes = SPConvMMPlugin.regroup_scratch_bytes(kernel_vol, max_num_act_out)
        if table_out is None:
            table_out = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=table_in.device)
        if scratch is None:
            scratch = torch.empty(max(sbytes, 16), dtype=torch.uint8, device=table_in.device)
        assert table_in.numel() >= nbytes and table_out.numel() >= nbytes and scratch.numel() >= sbytes
        with torch.cuda.device(table_in.device):
            check("d3d_spconv_mm_regroup",
                  lib().d3d_spconv_mm_regroup(int(kernel_vol), int(max_num_act_out),
                                              ctypes.c_void_p(table_in.data_ptr()),
                                              ctypes.c_void_p(table_out.data_ptr()),
                                              ctypes.c_void_p(scratch.data_ptr()), int(scratch.numel()),
                                              _stream_ptr(stream)))
        return table_out

    def run(self, in_feats, num_act_out, table, out=None, relu=False, residual=None, stream=None, regrouped=False):
        """`regrouped`: hint that `table` came from `regroup` (same results either way)."""
        if out is None:
            out = torch.empty((self.p.max_num_act_out, self.p.out_channels), dtype=in_feats.dtype,
                              device=in_feats.device)
        epi = _lib.SpconvMMEpilogue(int(relu), residual.data_ptr() if residual is not None else None,  # relu: 0 / 1 / 2
                                    int(bool(regrouped)))
        with torch.cuda.device(in_feats.device):
            check("d3d_spconv_mm_run",
                  lib().d3d_spconv_mm_run(self.handle, _TORCH2D3D[in_feats.dtype],
                                          ctypes.c_void_p(in_feats.data_ptr()), int(in_feats.shape[0]),
                                          ctypes.c_void_p(num_act_out.data_ptr()),
                                          ctypes.c_void_p(table.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                          ctypes.byref(epi), _stream_ptr(stream)))
        return out


class _PodPlugin(_Plugin):
    _params_t = None

    def __init__(self, name, data_s):
        super().__init__()
        self.p = self._params_t()
        buf = ctypes.create_string_buffer(bytes(data_s), max(len(data_s), 1))
        fn = getattr(lib(), self._prefix + "_parse")
        check(self._prefix + "_parse", fn(buf, len(data_s), ctypes.byref(self.p)))

    def _params_ref(self):
        return ctypes.byref(self.p)


class BEVDensifyPlugin(_PodPlugin):
    """``BEVDensify`` (trt/spconv/bev_densify_trt.cu:52-178)."""
    name = "BEVDensify"
    _prefix = "d3d_bev_densify"
    _params_t = _lib.BevDensifyParams


class SimpleMeanEncoderPlugin(_PodPlugin):
    """``SimpleMeanEncoder`` (trt/voxel_encoder/simple_mean_trt.cu:181-314)."""
    name = "SimpleMeanEncoder"
    _prefix = "d3d_simple_mean_encoder"
    _params_t = _lib.VoxelEncoderParams
    num_outputs = 3


    def enqueue_lp(self, *inputs, outputs, lp_feats=None, status=None, stream=None):
        """enqueue that also writes the voxel means in half / bfloat16, zero-padded to lp_feats.shape[1] channels,
        and / or reports soft failures (D3D_STATUS_* bits) in the int32 device tensor `status`."""
        inputs = [t if t.is_contiguous() else t.contiguous() for t in inputs]
        device = inputs[0].device
        in_descs = [_desc_of(t) for t in inputs]
        out_descs = self.output_descs(in_descs)
        ws_bytes = self.workspace_size(in_descs)
        ws = self._get_workspace(ws_bytes, device)
        extras = _lib.MeanEncoderExtras(lp_feats.data_ptr() if lp_feats is not None else None,
                                        _TORCH2D3D[lp_feats.dtype] if lp_feats is not None else 0,
                                        int(lp_feats.shape[1]) if lp_feats is not None else 0,
                                        status.data_ptr() if status is not None else None)
        with torch.cuda.device(device):
            status = lib().d3d_simple_mean_encoder_enqueue_ex(
                ctypes.byref(self.p), desc_array(in_descs), len(in_descs), desc_array(out_descs), len(out_descs),
                ptr_array([t.data_ptr() for t in inputs]), ptr_array([t.data_ptr() for t in outputs]),
                ctypes.c_void_p(ws.data_ptr() if ws is not None else 0), ctypes.c_size_t(ws_bytes),
                _stream_ptr(stream), ctypes.byref(extras))
        check("d3d_simple_mean_encoder_enqueue_ex", status)
        return tuple(outputs)


class CylinderEncoderPlugin(_PodPlugin):
    """``CylinderEncoder`` (trt/voxel_encoder/cylinder_trt.cu:187-333)."""
    name = "CylinderEncoder"
    _prefix = "d3d_cylinder_encoder"
    _params_t = _lib.VoxelEncoderParams
    num_outputs = 5


class ScatterToPlugin(_PodPlugin):
    """``ScatterTo`` (trt/point_voxel_mapping/scatter_to.cu:120-214)."""
    name = "ScatterTo"
    _prefix = "d3d_scatter_to"
    _params_t = _lib.ScatterToParams


class GatherBackPlugin(_PodPlugin):
    """``GatherBack`` (trt/point_voxel_mapping/gather_back.cu:77-184).  Besides the reference's float features it
    takes half / bfloat16 ones and writes them as they are or, into a float `outputs` tensor, widened."""
    name = "GatherBack"
    _prefix = "d3d_gather_back"
    _params_t = _lib.GatherBackParams


class NMS3dPlugin(_PodPlugin):
    """``NMS3d`` (trt/decoder/nms3d.cu:135-236).  ``iou_threshold`` is fixed to 0.1 by the reference."""
    name = "NMS3d"
    _prefix = "d3d_nms3d"
    _params_t = _lib.Nms3dParams


class YoloX3dDecodePlugin(_PodPlugin):
    """``YoloX3dDecode`` (trt/decoder/yolox3d_decode.cu:147-412): three outputs per class id of the blob."""
    name = "YoloX3dDecode"
    _prefix = "d3d_yolox3d_decode"
    _params_t = _lib.YoloX3dDecodeParams

    def output_descs(self, d):
        n = lib().d3d_yolox3d_decode_num_outputs(ctypes.byref(self.p))
        out = []
        for i in range(n):
            desc = _lib.TensorDesc()
            check("d3d_yolox3d_decode_output_desc",
                  lib().d3d_yolox3d_decode_output_desc(ctypes.byref(self.p), desc_array(d), len(d), i,
                                                       ctypes.byref(desc)))
            out.append(desc)
        return out


_REGISTRY = {
    "SPConvIdx1d": SPConvIdxPlugin, "SPConvIdx2d": SPConvIdxPlugin, "SPConvIdx3d": SPConvIdxPlugin,
    "SPConvIdx4d": SPConvIdxPlugin, "SPConvMM": SPConvMMPlugin, "BEVDensify": BEVDensifyPlugin,
    "SimpleMeanEncoder": SimpleMeanEncoderPlugin, "CylinderEncoder": CylinderEncoderPlugin,
    "ScatterTo": ScatterToPlugin, "GatherBack": GatherBackPlugin, "NMS3d": NMS3dPlugin,
    "YoloX3dDecode": YoloX3dDecodePlugin,
}


def registered_plugins():
    """Names under which the reference registers its creators (REGISTER_TENSORRT_PLUGIN)."""
    return sorted(_REGISTRY)


def deserialize_plugin(name, data_s, version=PLUGIN_VERSION):
    """``IPluginCreator::deserializePlugin(name, serialData, serialLength)``."""
    if version != PLUGIN_VERSION:
        raise KeyError("plugin version %r is not registered (only %r)" % (version, PLUGIN_VERSION))
    if name not in _REGISTRY:
        raise KeyError("plugin %r is not registered" % name)
    return _REGISTRY[name](name, bytes(data_s))
