"""The TensorRT plugin shells (deploy3d_b200/csrc/trt/deploy3d_trt_plugins.cpp), compiled against a stand-in for
<NvInfer.h> that carries the TensorRT 8 virtual signatures (tests/trt_stub/NvInfer.h) and driven the way TensorRT
drives a plugin: creators found by name, plugins made by deserializePlugin from the reference exporter's data_s
(tests/golden/plugin_blobs.npz), getNbOutputs / getOutputDimensions (symbolic, evaluated by a small IExprBuilder) /
getOutputDataType against the library's d3d_<op>_output_desc and the shapes the reference's shape-only forward()
allocates, supportsFormatCombination, serialize round trip, clone.  Not run under TensorRT itself: it is not installed
where this suite runs."""
import importlib.util
import os

import numpy as np
import pytest

from tests import _trt

HERE = os.path.join(os.path.dirname(__file__), "golden")


def _golden():
    spec = importlib.util.spec_from_file_location("make_golden_blobs", os.path.join(HERE, "make_golden_blobs.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    return gen, np.load(os.path.join(HERE, "plugin_blobs.npz"))


def test_twelve_creators_under_the_reference_names():
    from deploy3d_b200.plugins import registered_plugins
    h = _trt.harness()
    names = sorted(h.t_creator_name(i).decode() for i in range(h.t_num_creators()))
    assert names == registered_plugins() and len(names) == 12
    for i in range(h.t_num_creators()):
        assert h.t_creator_version(i) == b"2.0" and h.t_creator_namespace(i) == b""
        assert h.t_creator_refuses_fields(i) == 1  # only deserializePlugin creates plugins (index_trt.cu:262-275)


def test_shells_agree_with_the_library_and_the_exporter():
    from deploy3d_b200.plugins import _D3D2TORCH, _desc_of, deserialize_plugin
    gen, g = _golden()
    seen = set()
    for key, cls, _ in gen.CASES:
        blob = bytes(g[key + "_data"])
        shell = _trt.Shell(cls, blob)
        try:
            assert shell.h.t_type(shell.ptr).decode() == cls and shell.h.t_version(shell.ptr) == b"2.0"
            # serialize() gives the exporter's bytes back; a clone is the same plugin
            assert shell.serialize() == blob, "%s: serialize() changed the blob" % key
            twin = shell.clone()
            assert twin.serialize() == blob and twin.nb_outputs() == shell.nb_outputs()
            twin.close()
            assert shell.nb_outputs() == int(g[key + "_outputs"])
            plug = deserialize_plugin(cls, blob)
            in_descs = [_desc_of(t) for t in gen.make_inputs(cls)]
            lib_descs = plug.output_descs(in_descs)
            assert len(lib_descs) == shell.nb_outputs()
            for oi, d in enumerate(lib_descs):
                dtype, dims = shell.output_desc(oi, in_descs)
                assert dims == list(d.dims[:d.nb_dims]), "%s output %d: shell %s, library %s" % (
                    key, oi, dims, list(d.dims[:d.nb_dims]))
                assert dtype == d.dtype
                assert dims == [int(v) for v in g["%s_out%d_shape" % (key, oi)]]
                assert str(_D3D2TORCH[dtype]) == bytes(g["%s_out%d_dtype" % (key, oi)]).decode()
            # formats: the real combination is accepted at every position, a non-linear format never is
            inout = in_descs + lib_descs
            n_in, n_out = len(in_descs), len(lib_descs)
            for pos in range(n_in + n_out):
                assert shell.supports(pos, inout, n_in, n_out), "%s refuses position %d" % (key, pos)
                assert not shell.supports(pos, inout, n_in, n_out, non_linear=True)
            seen.add(cls)
        finally:
            shell.close()
    assert seen >= {"SPConvIdx3d", "SPConvMM", "BEVDensify", "SimpleMeanEncoder", "CylinderEncoder", "ScatterTo",
                    "GatherBack", "NMS3d", "YoloX3dDecode"}


def test_dtype_rules_follow_the_reference():
    from deploy3d_b200 import _lib, ops
    F, H, I = _lib.D3D_FLOAT, _lib.D3D_HALF, _lib.D3D_INT32
    w = np.zeros((27, 16, 16), np.float32)
    mm = _trt.Shell("SPConvMM", ops.data_s_spconv_mm((3, 3, 3), 16, 16, 1000, True, False, w, None))
    io = [(H, (900, 16)), (I, (1,)), (I, (1,)), (I, (3, 27 * 1028)), (I, (1,)), (H, (1000, 16))]
    assert all(mm.supports(p, io, 5, 1) for p in range(6))
    bad = list(io)
    bad[5] = (F, (1000, 16))  # output dtype must follow inFeats (mm_trt.cu:112)
    assert not mm.supports(5, bad, 5, 1)
    bad = list(io)
    bad[3] = (F, (3, 27 * 1028))  # the rulebook is int32
    assert not mm.supports(3, bad, 5, 1)
    assert mm.workspace(io[:5], io[5:]) >= 27 * 1024 * 4  # the neighbour table (the reference asks for none)
    mm.close()
    idx = _trt.Shell("SPConvIdx2d", ops.data_s_spconv_index((3, 3), (2, 2), (1, 1), (1, 1), (0, 0), 500, False, False))
    assert idx.nb_outputs() == 5
    dtype, dims = idx.output_desc(4, [(I, (300, 3)), (I, (1,)), (I, (2, 0, 40, 31))])
    assert dims == [2, 0, 20, 16] and dtype == I
    assert not idx.supports(0, [(F, (300, 3)), (I, (1,)), (I, (2, 0, 40, 31))] + [(I, (1,))] * 5, 3, 5)
    idx.close()
    enc = _trt.Shell("SimpleMeanEncoder", ops.data_s_voxel_encoder(777))
    io = [(F, (1000, 4)), (I, (1000,)), (F, (6,)), (I, (1, 0, 41, 160, 140)), (F, (777, 4)), (I, (777, 4)), (I, (1,))]
    assert all(enc.supports(p, io, 4, 3) for p in range(7))
    bad = list(io)
    bad[0] = (H, (1000, 4))  # the encoders are fp32 operators (simple_mean_trt.cu:250)
    assert not enc.supports(0, bad, 4, 3)
    enc.close()


def test_wrong_name_has_no_creator():
    with pytest.raises(AssertionError):
        _trt.Shell("Inspect", b"")  # emitted by the reference's exporter, never implemented in its C++ either
