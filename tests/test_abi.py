"""CPU tests of the drop-in boundary: the shared library loads without a GPU, exports every symbol the header
declares, and the host-only entry points (blob parsing, output shapes, workspace sizes, argument checks) behave."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(d3d):
    from deploy3d_b200 import _lib
    header = open(os.path.join(ROOT, "include", "deploy3d_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(d3d_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 30
    handle = ctypes.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(handle, name), "symbol %s declared in the header is not exported" % name
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)


def test_registry_matches_reference_names(d3d):
    from deploy3d_b200.plugins import deserialize_plugin, registered_plugins
    assert registered_plugins() == sorted(["SPConvIdx1d", "SPConvIdx2d", "SPConvIdx3d", "SPConvIdx4d", "SPConvMM",
                                           "BEVDensify", "SimpleMeanEncoder", "CylinderEncoder", "ScatterTo",
                                           "GatherBack", "NMS3d", "YoloX3dDecode"])
    with pytest.raises(KeyError):
        deserialize_plugin("NoSuchPlugin", b"")
    with pytest.raises(KeyError):
        deserialize_plugin("NMS3d", b"", version="1.0")


def test_yolox3d_decode_blob_round_trip(d3d):
    """The exporter's blob (deploy3d/symfun/ops/decoder/yolox3d_decode.py:43-50): stride, topk, 8 class ids."""
    from deploy3d_b200 import _lib
    from deploy3d_b200.plugins import deserialize_plugin
    blob = d3d.data_s_yolox3d_decode(8, (0, 3, 7), 500)
    assert len(blob) == 40
    plug = deserialize_plugin("YoloX3dDecode", blob)
    assert (plug.p.stride, plug.p.topk, list(plug.p.class_ids)) == (8, 500, [0, 3, 7, -1, -1, -1, -1, -1])
    assert _lib.lib().d3d_yolox3d_decode_num_outputs(plug._params_ref()) == 9
    with pytest.raises(_lib.D3DError):
        deserialize_plugin("YoloX3dDecode", blob[:39])


def test_spconv_index_blob_round_trip(d3d):
    from deploy3d_b200 import _lib
    from deploy3d_b200.plugins import deserialize_plugin
    blob = d3d.data_s_spconv_index((3, 1, 3), (2, 1, 2), (1, 0, 1), (1, 2, 1), (0, 1, 0), 4321, False, True)
    assert len(blob) == 66  # packed struct of the reference for NDim = 3
    p = deserialize_plugin("SPConvIdx3d", blob).p
    assert p.kernel_size[:3] == [3, 1, 3] and p.stride[:3] == [2, 1, 2] and p.padding[:3] == [1, 0, 1]
    assert p.dilation[:3] == [1, 2, 1] and p.out_padding[:3] == [0, 1, 0]
    assert (p.max_num_act_out, p.subm, p.transpose) == (4321, 0, 1)
    with pytest.raises(_lib.D3DError):
        deserialize_plugin("SPConvIdx3d", blob[:40])
    blob2 = d3d.data_s_spconv_index((3, 3), (1, 1), (1, 1), (1, 1), (0, 0), 10, True, False)
    assert len(blob2) == 46
    assert deserialize_plugin("SPConvIdx2d", blob2).p.subm == 1


def test_spconv_index_output_shapes_and_workspace(d3d):
    from deploy3d_b200 import _lib
    from deploy3d_b200.plugins import deserialize_plugin
    from oracle import oracle
    mk = _lib.make_desc
    ins = [mk(_lib.D3D_INT32, (40000, 4)), mk(_lib.D3D_INT32, (1,)), mk(_lib.D3D_INT32, (2, 0, 120, 90, 8))]
    for ks, st, pd, dl, op, tr in [((3, 3, 3), (2, 2, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), False),
                                   ((3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1), (1, 1, 1), True),
                                   ((3, 1, 1), (2, 1, 1), (0, 0, 0), (1, 1, 1), (0, 0, 0), False)]:
        plug = deserialize_plugin("SPConvIdx3d", d3d.data_s_spconv_index(ks, st, pd, dl, op, 50000, False, tr))
        outs = plug.output_descs(ins)
        assert len(outs) == 5
        assert list(outs[0].dims[:2]) == [3, int(np.prod(ks)) * (40000 + 128)]
        assert list(outs[2].dims[:2]) == [50000, 4]
        want = oracle.out_shape([2, 120, 90, 8], ks, st, pd, dl, op, tr)
        assert [outs[4].dims[0]] + list(outs[4].dims[2:5]) == want and outs[4].dims[1] == 0
        assert plug.workspace_size(ins) > 0
    subm = deserialize_plugin("SPConvIdx3d", d3d.data_s_spconv_index((3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1),
                                                                     (0, 0, 0), 0, True, False))
    assert len(subm.output_descs(ins)) == 2
    # a grid whose linear offsets do not fit 31 bits is refused, not wrapped around
    big = [ins[0], ins[1], mk(_lib.D3D_INT32, (64, 0, 41, 1600, 1408))]
    with pytest.raises(_lib.D3DError) as e:
        subm.workspace_size(big)
    assert e.value.status == -6


def test_spconv_mm_blob_round_trip(d3d):
    from deploy3d_b200 import _lib
    from deploy3d_b200.plugins import deserialize_plugin
    w = np.arange(27 * 4 * 8, dtype=np.float32).reshape(27, 4, 8)
    b = np.arange(8, dtype=np.float32)
    blob = d3d.data_s_spconv_mm((3, 3, 3), 4, 8, 1000, False, True, w, b)
    assert len(blob) == 19 + 4 * (27 * 4 * 8 + 8)
    plug = deserialize_plugin("SPConvMM", blob)
    assert (plug.p.kernel_vol, plug.p.in_channels, plug.p.out_channels, plug.p.max_num_act_out) == (27, 4, 8, 1000)
    assert (plug.p.inverse, plug.p.with_bias) == (1, 1)
    assert plug.serialize() == blob
    assert plug.workspace_size([_lib.make_desc(_lib.D3D_HALF, (500, 4))]) >= 27 * 1000 * 4
    with pytest.raises(_lib.D3DError):
        deserialize_plugin("SPConvMM", blob[:200])  # weights truncated
    nobias = deserialize_plugin("SPConvMM", d3d.data_s_spconv_mm((3, 3, 3), 4, 8, 1000, False, False, w, None))
    assert nobias.p.with_bias == 0


def test_small_blobs(d3d):
    from deploy3d_b200.plugins import deserialize_plugin
    assert deserialize_plugin("BEVDensify", d3d.data_s_bev_densify(256)).p.out_channels == 256
    assert deserialize_plugin("SimpleMeanEncoder", d3d.data_s_voxel_encoder(777)).p.max_num_act_out == 777
    assert deserialize_plugin("CylinderEncoder", d3d.data_s_voxel_encoder(5)).p.max_num_act_out == 5
    assert deserialize_plugin("ScatterTo", d3d.data_s_scatter_to(0)).p.reduce_type == 0
    assert deserialize_plugin("ScatterTo", d3d.data_s_scatter_to(1)).p.reduce_type == 1
    g = deserialize_plugin("GatherBack", d3d.data_s_gather_back(6.9)).p
    assert g.fill == 1 and abs(g.fill_val - 6.9) < 1e-6
    assert deserialize_plugin("GatherBack", d3d.data_s_gather_back(None)).p.fill == 0
    assert abs(deserialize_plugin("NMS3d", b"").p.iou_threshold - 0.1) < 1e-7


def test_ops_refuse_cpu_tensors(d3d):
    import torch
    with pytest.raises(RuntimeError):
        d3d.nms3d(torch.zeros(1, 4), torch.zeros(1, 4, 7))


def test_blobs_match_the_reference_exporter(d3d):
    """tests/golden/plugin_blobs.npz holds the `data_s` the reference's own exporter writes (the symbolic() of every
    op under deploy3d/symfun/ops, recorded by tests/golden/make_golden_blobs.py).  The blob builders of this package
    must produce the same bytes for the same parameters, and the plugin objects must accept the reference's bytes and
    report the exporter's number of outputs."""
    import importlib.util
    import os
    import numpy as np
    from deploy3d_b200 import ops
    from deploy3d_b200.plugins import deserialize_plugin
    here = os.path.join(os.path.dirname(__file__), "golden")
    spec = importlib.util.spec_from_file_location("make_golden_blobs", os.path.join(here, "make_golden_blobs.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    g = np.load(os.path.join(here, "plugin_blobs.npz"))
    build = {"SPConvIdx3d": ops.data_s_spconv_index, "SPConvMM": ops.data_s_spconv_mm,
             "BEVDensify": ops.data_s_bev_densify, "SimpleMeanEncoder": ops.data_s_voxel_encoder,
             "CylinderEncoder": ops.data_s_voxel_encoder, "ScatterTo": ops.data_s_scatter_to,
             "GatherBack": ops.data_s_gather_back, "NMS3d": lambda: b"", "YoloX3dDecode": ops.data_s_yolox3d_decode}
    for key, cls, params in gen.CASES:
        want = bytes(g[key + "_data"])
        assert bytes(g[key + "_name"]).decode() == cls and bytes(g[key + "_version"]) == b"2.0"
        got = bytes(build[cls](*params))
        assert got == want, "%s: blob differs from the reference exporter's" % key
        plug = deserialize_plugin(cls, want)
        import torch
        from deploy3d_b200.plugins import _D3D2TORCH, _desc_of
        inputs = gen.make_inputs(cls)  # CPU tensors: only their descriptors are taken
        descs = plug.output_descs([_desc_of(t) for t in inputs])
        n_out = len(descs)
        assert n_out == int(g[key + "_outputs"]), "%s: %d outputs, the exporter declares %d" % (
            key, n_out, int(g[key + "_outputs"]))
        # shapes and dtypes the reference's shape-only forward() allocates for the same inputs
        for oi, d in enumerate(descs):
            want_shape = [int(v) for v in g["%s_out%d_shape" % (key, oi)]]
            want_dtype = bytes(g["%s_out%d_dtype" % (key, oi)]).decode()
            assert list(d.dims[:d.nb_dims]) == want_shape, "%s output %d: %s vs %s" % (
                key, oi, list(d.dims[:d.nb_dims]), want_shape)
            assert str(_D3D2TORCH[d.dtype]) == want_dtype, "%s output %d: dtype" % (key, oi)
