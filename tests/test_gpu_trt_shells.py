"""The TensorRT plugin shells on the GPU: configurePlugin / getWorkspaceSize / enqueue of every shell (through the
test harness of tests/_trt.py, which stands in for TensorRT) against the same plugin reached directly through the
C ABI, on the same tensors: the shell adds no arithmetic, so the outputs are identical bit for bit."""
import numpy as np
import pytest
import torch

from tests import _trt
from tests._util import rng, unique_coors

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _t(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return t if dtype is None else t.to(dtype)


def _both(name, blob, inputs, zero_outputs=False):
    """Runs plugin `name` through its shell and directly; returns (shell outputs, direct outputs)."""
    from deploy3d_b200.plugins import _D3D2TORCH, _desc_of, deserialize_plugin
    plug = deserialize_plugin(name, blob)
    if name == "SPConvMM":
        plug.configure(inputs[0].dtype)
    descs = plug.output_descs([_desc_of(t) for t in inputs])
    make = torch.zeros if zero_outputs else torch.empty
    outs_a = [make(tuple(d.dims[:d.nb_dims]), dtype=_D3D2TORCH[d.dtype], device=DEV) for d in descs]
    outs_b = [make(tuple(d.dims[:d.nb_dims]), dtype=_D3D2TORCH[d.dtype], device=DEV) for d in descs]
    shell = _trt.Shell(name, blob)
    try:
        assert shell.enqueue(inputs, outs_a) == 0
        torch.cuda.synchronize()
    finally:
        shell.close()
    plug.enqueue(*inputs, outputs=outs_b)
    torch.cuda.synchronize()
    return outs_a, outs_b


def test_detection_chain_through_the_shells(d3d):
    """SimpleMeanEncoder -> SPConvIdx3d (SubM, then strided) -> SPConvMM (fp16) -> BEVDensify -> NMS3d."""
    from deploy3d_b200 import ops, synth
    r = rng(11)
    n_pts = 30000
    pts = np.concatenate([r.uniform(0, 20, (n_pts, 2)), r.uniform(0, 4, (n_pts, 1)), r.uniform(0, 1, (n_pts, 1))],
                         1).astype(np.float32)
    cfg = np.array([0, 0, 0, 0.1, 0.1, 0.2], np.float32)
    shape = [1, 0, 20, 200, 200]
    shp = torch.empty(shape, dtype=torch.int32, device=DEV)
    a, b = _both("SimpleMeanEncoder", ops.data_s_voxel_encoder(n_pts),
                 [_t(pts), _t(np.zeros(n_pts, np.int32)), _t(cfg), shp], zero_outputs=True)
    n = int(b[2].item())
    assert int(a[2].item()) == n and torch.equal(a[1][:n], b[1][:n])
    assert torch.allclose(a[0][:n], b[0][:n], rtol=1e-5, atol=1e-5)  # float atomics: the addition order varies
    coors, num = b[1], b[2]
    # SubM rulebook
    blob = ops.data_s_spconv_index((3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), n_pts, True, False)
    ia, ib = _both("SPConvIdx3d", blob, [coors, num, shp])
    assert torch.equal(ia[0], ib[0]) and torch.equal(ia[1], ib[1])
    # strided rulebook: five outputs, the last one shape-only
    blob = ops.data_s_spconv_index((3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1), (0, 0, 0), 2 * n_pts, False, False)
    sa, sb = _both("SPConvIdx3d", blob, [coors, num, shp], zero_outputs=True)
    m = int(sb[3].item())
    assert int(sa[3].item()) == m and torch.equal(sa[0], sb[0]) and torch.equal(sa[2][:m], sb[2][:m])
    assert list(sa[4].shape) == [1, 0, 10, 100, 100]
    # convolution over the strided rulebook, half precision
    w = synth.kaiming_weight(r, 27, 16, 32)
    bias = (r.standard_normal(32) * 0.1).astype(np.float32)
    feats = torch.randn((n_pts, 16), device=DEV).half()
    blob = ops.data_s_spconv_mm((3, 3, 3), 16, 32, 2 * n_pts, False, False, w, bias)
    ca, cb = _both("SPConvMM", blob, [feats, num, sb[3], sb[0], sb[1]])
    assert torch.equal(ca[0][:m], cb[0][:m]) and float(cb[0][:m].abs().sum()) > 0
    # densify
    oshape = torch.empty([1, 0, 10, 100, 100], dtype=torch.int32, device=DEV)
    da, db = _both("BEVDensify", ops.data_s_bev_densify(32 * 10), [cb[0], sb[2], sb[3], oshape])
    assert torch.equal(da[0], db[0]) and list(da[0].shape) == [1, 320, 100, 100]
    # NMS
    boxes = synth.config4_boxes(n_class=3, k=300)
    na, nb = _both("NMS3d", b"", [_t(boxes["scores"]), _t(boxes["boxes"])])
    assert torch.equal(na[0], nb[0]) and bool((nb[0] < 0).any()) and bool((nb[0] > 0).any())


def test_segmentation_chain_through_the_shells(d3d):
    """CylinderEncoder -> ScatterTo (max, mean) -> GatherBack, and YoloX3dDecode."""
    from deploy3d_b200 import ops, synth
    f = synth.config5_points()
    n_pts = 20000
    pts = f["points"][:n_pts]
    shp = torch.empty(f["spatial_shape"], dtype=torch.int32, device=DEV)
    ea, eb = _both("CylinderEncoder", ops.data_s_voxel_encoder(n_pts),
                   [_t(pts), _t(np.zeros(n_pts, np.int32)), _t(f["cylinder_config"]), shp], zero_outputs=True)
    n = int(eb[4].item())
    assert int(ea[4].item()) == n
    for i in (1, 2, 3):
        assert torch.equal(ea[i], eb[i])
    assert torch.allclose(ea[0], eb[0], rtol=1e-5, atol=1e-5)
    for reduce in (0, 1):
        sa, sb = _both("ScatterTo", ops.data_s_scatter_to(reduce), [eb[0], eb[1], eb[2]], zero_outputs=True)
        if reduce == 0:
            assert torch.equal(sa[0][:n], sb[0][:n])
        else:  # float atomics: the order of the additions differs between two runs
            assert torch.allclose(sa[0][:n], sb[0][:n], rtol=1e-5, atol=1e-5)
    ga, gb = _both("GatherBack", ops.data_s_gather_back(-1.0), [sb[0], eb[1]])
    assert torch.allclose(ga[0], gb[0], rtol=1e-5, atol=1e-5) and list(ga[0].shape) == [n_pts, pts.shape[1] + 5]
    r = rng(5)
    cls = _t(r.uniform(0, 1, (2, 3, 40, 48)).astype(np.float32))
    reg = _t(r.standard_normal((2, 9, 40, 48)).astype(np.float32))
    cfg = _t(np.array([-54, -54, -5, 0.075, 0.075, 0.2], np.float32))
    ya, yb = _both("YoloX3dDecode", ops.data_s_yolox3d_decode(8, [0, 1, 2], 100), [cls, reg, cfg])
    assert len(ya) == 9
    for a, b in zip(ya, yb):
        assert torch.equal(a, b)
