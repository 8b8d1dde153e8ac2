"""TEST INFRASTRUCTURE ONLY -- the reference's own GPU code: rulebook builders, indexed convolution, and its other
plugins (voxel encoders, point <-> voxel mapping, BEV densify, NMS, box decode) through their plugin classes.

``oracle/_ref/libref_spconv.so`` is compiled by ``make -C oracle ref_spconv`` from the reference's
trt/spconv/index.cu and trt/spconv/mm.h where those sources lie (wrappers: ``oracle/ref_spconv.cu``); it is a
build product that is kept out of the history.  The functions here call it the way the reference's plugins do
(trt/spconv/index_trt.cu:189-248, trt/spconv/mm_trt.cu:146-205), on torch CUDA tensors.  The other plugins are one
library each (``oracle/_ref/libref_<name>.so``, wrapper ``oracle/ref_plugin.cu``): the reference's plugin class is
constructed from its serialised parameters and its own configurePlugin / getWorkspaceSize / enqueue run.

Only the GPU parity tests and ``oracle/ref_gpu_timing.py`` may import this module; the product package never does.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

_i32p = ctypes.POINTER(ctypes.c_int32)
_i64p = ctypes.POINTER(ctypes.c_int64)


def lib():
    """The library, or None when it was never built (no reference checkout where the repository was built)."""
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "_ref", "libref_spconv.so")
        if not os.path.exists(path):
            return None
        L = ctypes.CDLL(path)
        L.ref_spconv_index_workspace.restype = ctypes.c_size_t
        L.ref_spconv_index_workspace.argtypes = [ctypes.c_int, ctypes.c_int32, _i32p]
        L.ref_spconv_index_run.restype = ctypes.c_int
        L.ref_spconv_index_run.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int32, _i32p, _i32p,
                                           _i32p, _i32p, _i64p, ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p,
                                           ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                           ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
        L.has_mm = hasattr(L, "ref_spconv_mm_run")
        if L.has_mm:
            L.ref_spconv_mm_run.restype = ctypes.c_int
            L.ref_spconv_mm_run.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32,
                                            ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                            ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                            ctypes.c_int64, ctypes.c_int, ctypes.c_void_p]
        _LIB = L
    return _LIB


def _v3(v):
    a = np.ascontiguousarray(v, dtype=np.int32)
    assert a.shape == (3,), "the reference wrappers are instantiated for three spatial dimensions"
    return a, a.ctypes.data_as(_i32p)


def spconv_index(coors_t, n_max, out_shape_b, ksize, stride, pad, dil, max_num_act_out, subm, transpose,
                 sync=True):
    """Reference rulebook for the live rows of ``coors_t`` (int32 CUDA tensor [n, 4]).

    Returns (index [3, kVol * (n_max + 128)], num_index [1], out_coors [max_num_act_out, 4], num_act_out [1]) as
    CUDA tensors; for SubM the last two are None.  ``out_shape_b`` = (B, Z, Y, X) of the output grid."""
    import torch
    L = lib()
    n = int(coors_t.shape[0])
    kvol = int(np.prod(ksize))
    row_len = kvol * (n_max + 128)
    dev = coors_t.device
    # uninitialised on purpose (no extra kernels in a timed call): the reference fills `index` with -1 itself and
    # writes both counts; rows of out_coors beyond num_act_out stay undefined, as in the plugin
    index = torch.empty((3, row_len), dtype=torch.int32, device=dev)
    num_index = torch.empty(1, dtype=torch.int32, device=dev)
    out_coors = None if subm else torch.empty((max_num_act_out, 4), dtype=torch.int32, device=dev)
    num_act_out = None if subm else torch.empty(1, dtype=torch.int32, device=dev)
    ks, ksp = _v3(ksize)
    st, stp = _v3(stride)
    pd, pdp = _v3(pad)
    dl, dlp = _v3(dil)
    shape = np.ascontiguousarray(out_shape_b, dtype=np.int64)
    ws_bytes = int(L.ref_spconv_index_workspace(int(subm), n, ksp))
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
    coors_t = coors_t.contiguous()
    stream = torch.cuda.current_stream(dev).cuda_stream
    rc = L.ref_spconv_index_run(int(subm), int(transpose), coors_t.data_ptr(), n, ksp, stp, pdp, dlp,
                                shape.ctypes.data_as(_i64p), int(max_num_act_out), row_len, index.data_ptr(),
                                num_index.data_ptr(), 0 if subm else out_coors.data_ptr(),
                                0 if subm else num_act_out.data_ptr(), ws.data_ptr(), ws_bytes, int(sync), stream)
    if rc != 0:
        raise RuntimeError("reference rulebook: CUDA error %d" % rc)
    return index, num_index, out_coors, num_act_out


def spconv_mm(in_feats_t, weight_t, bias_t, index_t, num_index_t, inverse, max_num_act_out, sync=True):
    """Reference indexed convolution, fp16 only (trt/spconv/mm_trt.cu:111): out = bias; out[s] += in[g] @ W[k]
    with half-precision atomic adds.  weight_t [kVol, Cin, Cout], bias_t [Cout] or None."""
    import torch
    L = lib()
    assert L.has_mm and in_feats_t.dtype == torch.float16
    kvol, cin, cout = (int(x) for x in weight_t.shape)
    out = torch.empty((max_num_act_out, cout), dtype=torch.float16, device=in_feats_t.device)
    stream = torch.cuda.current_stream(in_feats_t.device).cuda_stream
    rc = L.ref_spconv_mm_run(in_feats_t.data_ptr(), int(in_feats_t.shape[0]), cin, cout, kvol, weight_t.data_ptr(),
                             0 if bias_t is None else bias_t.data_ptr(), index_t.data_ptr(), int(index_t.shape[1]),
                             int(bool(inverse)), num_index_t.data_ptr(), out.data_ptr(), int(max_num_act_out),
                             int(sync), stream)
    if rc != 0:
        raise RuntimeError("reference convolution: status %d" % rc)
    return out


# ---- the reference's other plugins, driven through their own plugin classes --------------------------------------
_PLUGIN_LIBS = {}


class _Desc(ctypes.Structure):
    _fields_ = [("dtype", ctypes.c_int32), ("nb_dims", ctypes.c_int32), ("dims", ctypes.c_int64 * 8)]


def plugin_lib(name):
    """oracle/_ref/libref_<name>.so (built by `make -C oracle ref_plugins`), or None when it was never built."""
    if name not in _PLUGIN_LIBS:
        path = os.path.join(_HERE, "_ref", "libref_%s.so" % name)
        L = None
        if os.path.exists(path):
            L = ctypes.CDLL(path)
            L.ref_plugin_num_outputs.restype = ctypes.c_int
            L.ref_plugin_num_outputs.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
            L.ref_plugin_run.restype = ctypes.c_int
            L.ref_plugin_run.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(_Desc), ctypes.c_int,
                                         ctypes.POINTER(_Desc), ctypes.c_int, ctypes.POINTER(ctypes.c_void_p),
                                         ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]
        _PLUGIN_LIBS[name] = L
    return _PLUGIN_LIBS[name]


def _descs(tensors):
    import torch
    code = {torch.float32: 0, torch.float16: 1, torch.int8: 2, torch.int32: 3, torch.bool: 4}
    arr = (_Desc * len(tensors))()
    ptrs = (ctypes.c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i].dtype, arr[i].nb_dims = code[t.dtype], t.dim()
        for d in range(t.dim()):
            arr[i].dims[d] = int(t.shape[d])
        ptrs[i] = t.data_ptr() if t.numel() else None
    return arr, ptrs


def run_plugin(name, data_s, inputs, outputs):
    """Runs the reference plugin `name` (library suffix, e.g. "simple_mean") built from the serialised parameters
    `data_s` on torch CUDA tensors; zero-element tensors carry shapes only, as in the reference.  `outputs` are
    written in place.  Synchronises the device before returning."""
    import torch
    L = plugin_lib(name)
    data_s = bytes(data_s)
    assert L.ref_plugin_num_outputs(data_s, len(data_s)) == len(outputs)
    inputs = [t.contiguous() for t in inputs]
    din, pin = _descs(inputs)
    dout, pout = _descs(outputs)
    stream = torch.cuda.current_stream(outputs[0].device).cuda_stream
    rc = L.ref_plugin_run(data_s, len(data_s), din, len(inputs), dout, len(outputs), pin, pout, stream)
    if rc != 0:
        raise RuntimeError("reference plugin %s: status %d" % (name, rc))
    return outputs
