"""GPU parity of SimpleMeanEncoder, CylinderEncoder, ScatterTo, GatherBack and BEVDensify against the CPU oracle.
Cases follow the reference's tests (tests/voxel_encoder/*.py, tests/point_voxel_mapping/*.py,
tests/spconv/test_bev_densify.py): voxel order is arbitrary, so coordinates are compared after lexicographic
sorting; features within 1e-3 as there; integer outputs exactly."""
import numpy as np
import pytest
import torch

from tests._util import rng

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _shape(s):
    return torch.empty(s, dtype=torch.int32, device=DEV)


def _mean_inputs(seed, n=200000):
    r = rng(seed)
    pts = np.stack([r.standard_normal(n) * 50, r.standard_normal(n) * 50, r.standard_normal(n) * 2 + 1,
                    r.standard_normal(n)], 1).astype(np.float32)
    batch = r.integers(0, 2, n).astype(np.int32)
    cfg = np.array([-76.8, -76.8, -2, 0.1, 0.1, 0.15], np.float32)
    from deploy3d_b200.synth import drop_edge_points
    keep = drop_edge_points(pts[:, :3], cfg[:3], cfg[3:])
    return pts[keep], batch[keep], cfg, [2, 0, 41, 1536, 1536]


@pytest.mark.parametrize("max_out", [200000, 100])
def test_simple_mean(d3d, orc, max_out):
    """tests/voxel_encoder/test_simple_mean.py:7-65."""
    pts, batch, cfg, shape = _mean_inputs(41)
    pts[::997, 1] = np.nan  # non-finite points are ignored (simple_mean_trt.cu:39-41)
    batch[::991] = -1       # as are points without a batch (:44)
    feats, coors, num = d3d.simple_mean_encoder(_t(pts), _t(batch), _t(cfg), _shape(shape), max_out)
    torch.cuda.synchronize()
    num = int(num.item())
    wf, wc, wn = orc.simple_mean(pts, batch, cfg, shape, 10 ** 7)
    assert num == min(wn, max_out)
    got_c, got_f = coors.cpu().numpy()[:num], feats.cpu().numpy()[:num]
    ids = {tuple(c): i for i, c in enumerate(wc[:wn].tolist())}
    sel = np.array([ids[tuple(c)] for c in got_c.tolist()])  # KeyError = a voxel the oracle does not have
    assert len(np.unique(sel)) == num
    if max_out >= wn:
        assert np.allclose(got_f, wf[sel], atol=1e-3, rtol=1e-3)
    else:
        # a truncated voxel still averages all of its points
        assert np.allclose(got_f, wf[sel], atol=1e-3, rtol=1e-3)
    assert (feats.cpu().numpy()[num:] == 0).all()


def test_simple_mean_config_shapes(d3d, orc):
    """benchmark configs 3 and 4 (120 000 x 4 and 300 000 x 5 points)."""
    from deploy3d_b200 import synth
    for c in (synth.config3_points(), synth.config4_points()):
        pts, cfg = c["points"], c["voxel_config"]
        keep = synth.drop_edge_points(pts[:, :3], cfg[:3], cfg[3:])
        pts, batch = pts[keep], c["batch"][keep]
        m = pts.shape[0]
        feats, coors, num = d3d.simple_mean_encoder(_t(pts), _t(batch), _t(cfg), _shape(c["spatial_shape"]), m)
        num = int(num.item())
        wf, wc, wn = orc.simple_mean(pts, batch, cfg, c["spatial_shape"], m)
        assert num == wn
        go, wo = orc.lex_order(coors.cpu().numpy()[:num]), orc.lex_order(wc[:wn])
        assert (coors.cpu().numpy()[:num][go] == wc[:wn][wo]).all()
        assert np.allclose(feats.cpu().numpy()[:num][go], wf[:wn][wo], atol=1e-3, rtol=1e-3)
        # first-touch numbering: voxel ids ascend with the first point that falls into them
        f = ((pts[:, :3] - cfg[:3]) / cfg[3:]).astype(np.int32)
        key = (f[:, 2].astype(np.int64) * 4096 + f[:, 1]) * 4096 + f[:, 0]
        _, first = np.unique(key, return_index=True)
        gk = coors.cpu().numpy()[:num].astype(np.int64)
        gkey = (gk[:, 1] * 4096 + gk[:, 2]) * 4096 + gk[:, 3]
        assert (gkey == key[np.sort(first)]).all()


@pytest.mark.parametrize("max_out", [200000, 100])
def test_cylinder(d3d, orc, max_out):
    """tests/voxel_encoder/test_cylinder.py:7-94."""
    r = rng(43)
    n = 200000
    pts = np.stack([r.standard_normal(n) * 100, r.standard_normal(n) * 100, r.standard_normal(n) * 3 + 1,
                    r.standard_normal(n)], 1).astype(np.float32)
    batch = r.integers(0, 2, n).astype(np.int32)
    cfg = np.array([-2, -np.pi, 0, 4, np.pi, 50], np.float32)
    shape = [2, 0, 480, 360, 32]
    rho = np.sqrt(pts[:, 0] ** 2 + pts[:, 1] ** 2)
    phi = np.arctan2(pts[:, 1], pts[:, 0])
    step = (cfg[3:] - cfg[:3]) / np.array([32, 360, 480], np.float32)
    from deploy3d_b200.synth import drop_edge_points
    keep = drop_edge_points(np.stack([pts[:, 2], phi, rho], 1), cfg[:3], step)
    pts, batch = pts[keep], batch[keep]
    n = pts.shape[0]
    aug, st, sc, coors, num = d3d.cylinder_encoder(_t(pts), _t(batch), _t(cfg), _shape(shape), max_out)
    torch.cuda.synchronize()
    num = int(num.item())
    wa, wst, wsc, wc, wn = orc.cylinder(pts, batch, cfg, shape, 10 ** 7)
    assert num == min(wn, max_out)
    st, sc, coors, aug = st.cpu().numpy(), sc.cpu().numpy(), coors.cpu().numpy(), aug.cpu().numpy()
    valid = st >= 0
    if max_out >= wn:
        assert (valid == (wst >= 0)).all()
    assert np.allclose(aug[valid], wa[valid], atol=1e-3, rtol=1e-3)
    assert (aug[wst < 0] == 0).all()
    ids = {tuple(c): i for i, c in enumerate(wc[:wn].tolist())}
    sel = np.array([ids[tuple(c)] for c in coors[:num].tolist()])
    assert len(np.unique(sel)) == num
    assert (sel[st[valid]] == wst[valid]).all()       # same point -> voxel mapping up to renumbering
    assert (sc[:num] == wsc[sel]).all()                # same population per voxel
    assert (sc[num:] == 0).all()
    if max_out < wn:
        assert (st < max_out).all() and valid.sum() == sc[:num].sum()


SCATTER = [(rt, act, inv) for rt in (0, 1) for act in (65536, 32768) for inv in (True, False)]


@pytest.mark.parametrize("reduce_type,num_act,has_invalid", SCATTER)
@pytest.mark.parametrize("c", [9, 16])
def test_scatter_to(d3d, orc, reduce_type, num_act, has_invalid, c):
    """tests/point_voxel_mapping/test_scatter_to.py:8-100 (plus a 16-channel case for the vector path)."""
    r = rng(50 + reduce_type + num_act % 7 + has_invalid)
    n, m = 200000, 65536
    lo = -1 if has_invalid else 0
    base = np.arange(lo, num_act, dtype=np.int32)
    idx = np.concatenate([base, r.integers(lo, num_act, n - base.size).astype(np.int32)])
    idx = idx[r.permutation(n)]
    cnt = np.zeros(m, np.int32)
    u, k = np.unique(idx[idx >= 0], return_counts=True)
    cnt[u] = k
    x = r.standard_normal((n, c)).astype(np.float32)
    x[3, 0] = -0.0
    out = d3d.scatter_to(_t(x), _t(idx), _t(cnt), reduce_type).cpu().numpy()
    want = orc.scatter_to(x, idx, cnt, reduce_type)
    if reduce_type == 0:
        assert (out[:num_act] == want[:num_act]).all()            # max is exact
        assert (out[num_act:] == np.float32(-3.402823466e38)).all()  # untouched rows keep lowest()
    else:
        assert np.allclose(out, want, atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("feat_shape", [(9,), (), (16,), (4, 3)])
@pytest.mark.parametrize("fill_val", [None, 6.9])
def test_gather_back(d3d, orc, feat_shape, fill_val):
    """tests/point_voxel_mapping/test_gather_back.py:6-43."""
    r = rng(60)
    n, m = 200000, 65536
    idx = r.integers(-1, m, n).astype(np.int32)
    x = r.standard_normal((m,) + feat_shape).astype(np.float32)
    from deploy3d_b200.ops import gather_back
    init = torch.full((n,) + feat_shape, 3.25, dtype=torch.float32, device=DEV)
    out = gather_back(_t(x), _t(idx), fill_val, out=init).cpu().numpy()
    want = orc.gather_back(x, idx, fill_val, out_init=np.full((n,) + feat_shape, 3.25, np.float32))
    assert (out == want).all()


@pytest.mark.parametrize("in_dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("widen", [True, False])
@pytest.mark.parametrize("fill_val", [None, 6.5])
def test_gather_back_half_precision_features(d3d, orc, in_dtype, widen, fill_val):
    """Half-precision features (an extension: the reference's GatherBack is float only, gather_back.cu:146-150) are
    gathered exactly, into rows of the same type or widened into a float output; the float oracle on the rounded
    features is the expected result either way.  A float output for float input stays the only other combination."""
    r = rng(61)
    n, m, c = 70001, 20000, 20
    idx = r.integers(-1, m, n).astype(np.int32)
    x = torch.from_numpy(r.standard_normal((m, c)).astype(np.float32)).to(in_dtype)
    out_dtype = torch.float32 if widen else in_dtype
    init = torch.full((n, c), 3.25, dtype=out_dtype, device=DEV)
    from deploy3d_b200.ops import data_s_gather_back
    from deploy3d_b200.plugins import deserialize_plugin
    plug = deserialize_plugin("GatherBack", data_s_gather_back(fill_val))
    out, = plug.enqueue(x.to(DEV), _t(idx), outputs=[init])
    want = orc.gather_back(x.float().numpy(), idx, fill_val, out_init=np.full((n, c), 3.25, np.float32))
    assert out.dtype == out_dtype and (out.float().cpu().numpy() == want).all()
    with pytest.raises(RuntimeError):  # float features never narrow
        plug.enqueue(x.float().to(DEV), _t(idx), outputs=[torch.zeros((n, c), dtype=torch.float16, device=DEV)])


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("num_act", [10000, 100, 0])
def test_bev_densify(d3d, orc, dtype, num_act):
    """tests/spconv/test_bev_densify.py:6-53."""
    from tests._util import unique_coors
    r = rng(70 + num_act)
    n_max, c = 10000, 128
    shape = [2, 0, 2, 128, 128]
    coors = np.zeros((n_max, 4), np.int32)
    coors[:num_act] = unique_coors(r, num_act, [2, 2, 128, 128]) if num_act else coors[:0]
    feats = torch.from_numpy(r.standard_normal((n_max, c)).astype(np.float32)).to(dtype)
    out = d3d.bev_densify(feats.to(DEV), _t(coors), torch.tensor([num_act], dtype=torch.int32, device=DEV),
                          _shape(shape), c * 2)
    want = orc.bev_densify(feats.float().numpy(), coors, num_act, shape)
    assert out.dtype == dtype and tuple(out.shape) == (2, 256, 128, 128)
    assert (out.float().cpu().numpy() == want).all()


def test_bev_densify_config3_shape(d3d, orc):
    """[1, 256, 200, 176] map of benchmark config 3 (C = 128, Z = 2), ragged X (176 is not a multiple of 32... it is;
    use 200 x 171 as well to cover a ragged strip)."""
    from tests._util import unique_coors
    r = rng(77)
    for (y, x) in ((200, 176), (200, 171)):
        n = 12000
        coors = unique_coors(r, n, [1, 2, y, x])
        feats = r.standard_normal((n, 128)).astype(np.float16)
        out = d3d.bev_densify(_t(feats), _t(coors), torch.tensor([n], dtype=torch.int32, device=DEV),
                              _shape([1, 0, 2, y, x]), 256)
        want = orc.bev_densify(feats.astype(np.float32), coors, n, [1, 0, 2, y, x])
        assert (out.float().cpu().numpy() == want).all()


@pytest.mark.parametrize("c,y,x", [(128, 180, 180), (40, 50, 62), (8, 3, 2), (136, 7, 130), (12, 20, 64)])
def test_bev_densify_strips(d3d, orc, c, y, x):
    """Row lengths that end inside a 64-cell strip, channel counts that are and are not a multiple of eight (the
    16-byte row loads of the half-precision kernel need one), the 180 x 180 map of benchmark config 4."""
    from tests._util import unique_coors
    r = rng(78 + c + x)
    n = min(9000, y * x)
    coors = unique_coors(r, n, [1, 2, y, x])
    feats = r.standard_normal((n, c)).astype(np.float16)
    out = d3d.bev_densify(_t(feats), _t(coors), torch.tensor([n], dtype=torch.int32, device=DEV),
                          _shape([1, 0, 2, y, x]), 2 * c)
    want = orc.bev_densify(feats.astype(np.float32), coors, n, [1, 0, 2, y, x])
    assert (out.float().cpu().numpy() == want).all()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_mean_encoder_low_precision_output(d3d, dtype):
    """The optional extra output of SimpleMeanEncoder: the voxel means in half / bfloat16, zero-padded to 16
    channels, equal to rounding the fp32 output (what a separate cast-and-pad kernel would give)."""
    from deploy3d_b200 import synth
    from deploy3d_b200.ops import data_s_voxel_encoder
    from deploy3d_b200.plugins import deserialize_plugin
    f = synth.config4_points()
    n = 50000
    pts = torch.from_numpy(f["points"][:n]).cuda()
    batch = torch.zeros(n, dtype=torch.int32, device="cuda")
    cfg = torch.from_numpy(f["voxel_config"]).cuda()
    shp = torch.empty(f["spatial_shape"], dtype=torch.int32, device="cuda")
    plug = deserialize_plugin("SimpleMeanEncoder", data_s_voxel_encoder(n))
    feats = torch.zeros((n, 5), device="cuda")
    coors = torch.zeros((n, 4), dtype=torch.int32, device="cuda")
    num = torch.zeros(1, dtype=torch.int32, device="cuda")
    lp = torch.full((n, 16), 7.0, dtype=dtype, device="cuda")
    plug.enqueue_lp(pts, batch, cfg, shp, outputs=[feats, coors, num], lp_feats=lp)
    torch.cuda.synchronize()
    m = int(num.item())
    assert 0 < m < n
    assert torch.equal(lp[:m, :5], feats[:m].to(dtype)) and bool((lp[:m, 5:] == 0).all())
    assert bool((lp[m:] == 7.0).all())  # rows beyond numActOut are left alone


def test_mean_encoder_status_word(d3d):
    """More voxels than maxNumActOut: the surplus is dropped and D3D_STATUS_OUTPUT_OVERFLOW is reported."""
    from deploy3d_b200 import _lib, synth
    from deploy3d_b200.ops import data_s_voxel_encoder
    from deploy3d_b200.plugins import deserialize_plugin
    f = synth.config4_points()
    n = 20000
    pts = torch.from_numpy(f["points"][:n]).cuda()
    batch = torch.zeros(n, dtype=torch.int32, device="cuda")
    cfg = torch.from_numpy(f["voxel_config"]).cuda()
    shp = torch.empty(f["spatial_shape"], dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for cap, want in ((500, _lib.D3D_STATUS_OUTPUT_OVERFLOW), (n, 0)):
        plug = deserialize_plugin("SimpleMeanEncoder", data_s_voxel_encoder(cap))
        outs = [torch.zeros((cap, 5), device="cuda"), torch.zeros((cap, 4), dtype=torch.int32, device="cuda"),
                torch.zeros(1, dtype=torch.int32, device="cuda")]
        status.zero_()
        plug.enqueue_lp(pts, batch, cfg, shp, outputs=outs, status=status)
        assert int(status.item()) == want and int(outs[2].item()) <= cap
