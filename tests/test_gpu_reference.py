"""The reference's own GPU code as the yardstick: trt/spconv/index.cu and trt/spconv/mm.h compiled for sm_100a
(oracle/_ref/libref_spconv.so, built by `make -C oracle ref_spconv`) run on the same inputs as the product library and
the CPU oracle.

* SubM rulebooks are deterministic in the reference (gather = input id, scatter = hash value = neighbour id, segments
  in offset order): reference == oracle == product byte for byte, padding included.
* Strided / transposed rulebooks number the outputs by hash-slot rank, which depends on the insertion race:
  compared after the canonicalisation the reference's own test performs (tests/spconv/test_spconv.py:72-124).
* Features: the reference accumulates with half-precision atomic adds in arbitrary order, so it is compared with
  the tolerance of its own test (rtol 1e-2, atol 1e-1, test_spconv.py:152-161) and a relative L2 bound."""
import numpy as np
import pytest
import torch

from tests._util import pairs_equal, rng, unique_coors
from tests.test_gpu_spconv import _t, check_index, run_index

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ref():
    from oracle import ref_gpu
    if ref_gpu.lib() is None:
        pytest.skip("oracle/_ref/libref_spconv.so was not built (no reference checkout where the repository was built)")
    return ref_gpu


CASES = [
    # name, ks, st, pd, dl, op, tr, subm, shape_b, n, n_max, max_out
    ("subm", (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), False, True, [2, 120, 90, 8], 20000, 20000, 20000),
    ("subm_padded_buffer", (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), False, True, [2, 120, 90, 8], 20000,
     40000, 40000),
    ("subm_dilated", (3, 3, 3), (1, 1, 1), (2, 2, 2), (2, 2, 2), (0, 0, 0), False, True, [1, 30, 30, 12], 5000, 5077,
     5077),
    ("subm_3x1x3", (3, 1, 3), (1, 1, 1), (1, 0, 1), (1, 1, 1), (0, 0, 0), False, True, [2, 48, 36, 16], 9000, 9077,
     9077),
    ("subm_5x5x5", (5, 5, 5), (1, 1, 1), (2, 2, 2), (1, 1, 1), (0, 0, 0), False, True, [1, 14, 14, 14], 1200, 1277,
     1277),
    ("strided_221", (3, 3, 3), (2, 2, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), False, False, [2, 120, 90, 8], 20000, 20000,
     50000),
    ("strided_221_truncated", (3, 3, 3), (2, 2, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), False, False, [2, 120, 90, 8],
     20000, 40000, 5000),
    ("strided_222_pad011", (3, 3, 3), (2, 2, 2), (0, 1, 1), (1, 1, 1), (0, 0, 0), False, False, [2, 11, 60, 50], 7000,
     7077, 200000),
    ("strided_3x1x1", (3, 1, 1), (2, 1, 1), (0, 0, 0), (1, 1, 1), (0, 0, 0), False, False, [2, 5, 60, 50], 6000, 6077,
     200000),
    ("strided_222_dilated_2", (3, 3, 3), (2, 2, 2), (2, 2, 2), (2, 2, 2), (0, 0, 0), False, False, [1, 20, 20, 12], 3000,
     3077, 200000),
    ("strided_212", (3, 3, 3), (2, 1, 2), (1, 1, 1), (1, 1, 1), (0, 0, 0), False, False, [2, 20, 14, 12], 4000, 4077,
     200000),
    ("transposed_222", (3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1), (1, 1, 1), True, False, [2, 20, 24, 10], 3000, 3077,
     200000),
    ("transposed_k2", (2, 2, 2), (2, 2, 2), (0, 0, 0), (1, 1, 1), (0, 0, 0), True, False, [1, 16, 16, 16], 1000, 1077,
     200000),
]


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_rulebook_matches_reference_gpu(d3d, orc, ref, case):
    name, ks, st, pd, dl, op, tr, subm, shape_b, n, n_max, max_out = case
    r = rng(7000 + sum(map(ord, name)))
    coors = unique_coors(r, n, shape_b)
    kvol = int(np.prod(ks))
    out_shape_b = shape_b if subm else orc.out_shape(shape_b, ks, st, pd, dl, op, tr)
    r_index, r_num, r_coors, r_nout = ref.spconv_index(_t(coors), n_max, out_shape_b, ks, st, pd, dl, max_out, subm,
                                                       tr)
    ref_outs = [r_index, r_num] if subm else [r_index, r_num, r_coors, r_nout]
    # 1. the reference against the CPU oracle (pins the oracle)
    check_index(orc, ref_outs, coors, n_max, shape_b, ks, st, pd, dl, op, max_out, subm, tr)
    # 2. the product against the reference, directly
    spatial = [shape_b[0], 0] + shape_b[1:]
    outs, _ = run_index(d3d, coors, n_max, spatial, ks, st, pd, dl, op, max_out, subm, tr)
    got_num, ref_num = int(outs[1].item()), int(r_num.item())
    if subm:
        assert got_num == ref_num
        assert torch.equal(outs[0], r_index), "SubM rulebook differs from the reference's byte for byte"
        return
    ref_nout, got_nout = int(r_nout.item()), int(outs[3].item())
    assert got_nout == ref_nout
    assert list(outs[4].shape) == [out_shape_b[0], 0] + list(out_shape_b[1:])
    # when maxNumActOut truncates, WHICH outputs survive is the reference's hash-slot order (implementation defined):
    # both sides were checked against the oracle's rules for the kept subset above and in test_gpu_spconv.py
    if ref_nout < max_out:  # nothing truncated: same output set, same pairs
        assert got_num == ref_num
        gc, gp, _ = orc.canonical_conv(outs[0].cpu().numpy(), got_num, outs[2].cpu().numpy(), got_nout, kvol)
        rc, rp, _ = orc.canonical_conv(r_index.cpu().numpy(), ref_num, r_coors.cpu().numpy(), ref_nout, kvol)
        assert (gc == rc).all(), "output coordinate sets differ from the reference's"
        pairs_equal(gp, rp, kvol)


def _features(r, n_rows, cin, cout, kvol):
    feats = r.standard_normal((n_rows, cin)).astype(np.float32)
    w = (r.standard_normal((kvol, cin, cout)) * np.sqrt(2.0 / (kvol * cin))).astype(np.float32)
    b = r.standard_normal(cout).astype(np.float32)
    return feats, w, b


@pytest.mark.parametrize("cin,cout", [(16, 32), (32, 32), (64, 64), (128, 128), (16, 24)])
@pytest.mark.parametrize("kind", ["subm", "strided", "inverse"])
def test_features_match_reference_gpu(d3d, orc, ref, kind, cin, cout):
    if not ref.lib().has_mm:
        pytest.skip("the reference convolution was not built (no CUTLASS header tree where the repository was built)")
    r = rng(8000 + cin * 7 + cout + len(kind))
    shape_b, spatial, n = [2, 120, 90, 8], [2, 0, 120, 90, 8], 20000
    coors = unique_coors(r, n, shape_b)
    ks, pd, dl, op = (3, 3, 3), (1, 1, 1), (1, 1, 1), (0, 0, 0)
    subm = kind == "subm"
    st = (1, 1, 1) if subm else (2, 2, 1)
    max_out = n if subm else 50000
    outs, num_in = run_index(d3d, coors, n, spatial, ks, st, pd, dl, op, max_out, subm, False)
    num_out = num_in if subm else outs[3]
    inverse = kind == "inverse"
    n_in_rows, n_out_rows, a, b_ = (max_out, n, num_out, num_in) if inverse else (n, max_out, num_in, num_out)
    feats, w, b = _features(r, n_in_rows, cin, cout, 27)
    feats_t = _t(feats, torch.float16)
    got = d3d.spconv_mm(feats_t, a, b_, outs[0], outs[1], ks, cin, cout, n_out_rows, False, inverse, w, b)
    want = ref.spconv_mm(feats_t, _t(w, torch.float16), _t(b, torch.float16), outs[0], outs[1], inverse, n_out_rows)
    torch.cuda.synchronize()
    got, want = got.float().cpu().numpy(), want.float().cpu().numpy()
    assert got.shape == want.shape
    assert np.allclose(got, want, rtol=1e-2, atol=1e-1), "worst |diff| %.3e" % np.abs(got - want).max()
    rel_l2 = np.sqrt(((got - want) ** 2).sum() / (want ** 2).sum())
    assert rel_l2 < 5e-3, "relative L2 distance to the reference %.3e" % rel_l2
    # and the reference itself sits inside the oracle's tolerance band around the fp32-accumulated result
    exact = orc.spconv_mm(feats_t.float().cpu().numpy(), _t(w, torch.float16).float().cpu().numpy(),
                          _t(b, torch.float16).float().cpu().numpy(), outs[0].cpu().numpy(), int(outs[1].item()),
                          inverse, n_out_rows)
    assert np.allclose(want, exact, rtol=1e-2, atol=1e-1)
    # one rounding of an fp32 accumulator is no further from it than a chain of half-precision atomic adds
    assert np.sqrt(((got - exact) ** 2).sum()) <= 1.05 * np.sqrt(((want - exact) ** 2).sum()) + 1e-6


# ---- the reference's other plugins, run through their own plugin classes (oracle/ref_plugin.cu) ------------------
# Each test feeds the product library and the reference plugin the same tensors and the same serialised parameters
# (the blob the reference's exporter writes), compares the two directly, and holds the CPU oracle against the
# reference's output as well (which is what pins the oracle for these operators).

def _ref_plugin(ref, name):
    if ref.plugin_lib(name) is None:
        pytest.skip("oracle/_ref/libref_%s.so was not built" % name)
    return lambda data_s, inputs, outputs: ref.run_plugin(name, data_s, inputs, outputs)


def _shape_t(s):
    return torch.empty(s, dtype=torch.int32, device=DEV)


def _by_coors(orc, coors, num, *arrays):
    o = orc.lex_order(coors[:num])
    return (coors[:num][o],) + tuple(a[:num][o] for a in arrays)


def test_simple_mean_matches_reference_gpu(d3d, orc, ref):
    from deploy3d_b200.ops import data_s_voxel_encoder
    from tests.test_gpu_encoders import _mean_inputs
    run = _ref_plugin(ref, "simple_mean")
    pts, batch, cfg, shape = _mean_inputs(45, n=60000)
    pts[::997, 1] = np.nan
    batch[::991] = -1
    max_out = 60000
    ins = [_t(pts), _t(batch), _t(cfg), _shape_t(shape)]
    got = d3d.simple_mean_encoder(*ins, max_out)
    want = run(data_s_voxel_encoder(max_out), ins, [torch.zeros_like(t) for t in got])
    torch.cuda.synchronize()
    gn, wn = int(got[2].item()), int(want[2].item())
    assert gn == wn
    gc, gf = _by_coors(orc, got[1].cpu().numpy(), gn, got[0].cpu().numpy())
    wc, wf = _by_coors(orc, want[1].cpu().numpy(), wn, want[0].cpu().numpy())
    assert (gc == wc).all(), "voxel sets differ from the reference's"
    assert np.allclose(gf, wf, atol=1e-3, rtol=1e-3)  # float atomics in a different order
    of, oc, on = orc.simple_mean(pts, batch, cfg, shape, max_out)
    assert on == wn
    oc, of = _by_coors(orc, oc, on, of)
    assert (oc == wc).all() and np.allclose(of, wf, atol=1e-3, rtol=1e-3)


def test_cylinder_matches_reference_gpu(d3d, orc, ref):
    from deploy3d_b200.ops import data_s_voxel_encoder
    from deploy3d_b200.synth import drop_edge_points
    run = _ref_plugin(ref, "cylinder")
    r = rng(46)
    n = 60000
    pts = np.stack([r.standard_normal(n) * 100, r.standard_normal(n) * 100, r.standard_normal(n) * 3 + 1,
                    r.standard_normal(n)], 1).astype(np.float32)
    batch = r.integers(0, 2, n).astype(np.int32)
    batch[::983] = -1
    cfg = np.array([-2, -np.pi, 0, 4, np.pi, 50], np.float32)
    shape = [2, 0, 480, 360, 32]
    rho, phi = np.sqrt(pts[:, 0] ** 2 + pts[:, 1] ** 2), np.arctan2(pts[:, 1], pts[:, 0])
    step = (cfg[3:] - cfg[:3]) / np.array([32, 360, 480], np.float32)
    keep = drop_edge_points(np.stack([pts[:, 2], phi, rho], 1), cfg[:3], step)
    pts, batch = pts[keep], batch[keep]
    n = len(pts)
    ins = [_t(pts), _t(batch), _t(cfg), _shape_t(shape)]
    got = [t.cpu().numpy() for t in d3d.cylinder_encoder(*ins, n)]
    want = run(data_s_voxel_encoder(n), ins, [torch.zeros_like(_t(g)) for g in got])
    want = [t.cpu().numpy() for t in want]
    (g_aug, g_st, g_sc, g_co, g_n), (w_aug, w_st, w_sc, w_co, w_n) = got, want
    gn, wn = int(g_n[0]), int(w_n[0])
    assert gn == wn
    valid = w_st >= 0
    assert ((g_st >= 0) == valid).all()
    assert np.allclose(g_aug[valid], w_aug[valid], atol=1e-5, rtol=1e-5)
    # same point -> voxel mapping up to the (race-dependent) voxel numbering
    assert (g_co[:gn][g_st[valid]] == w_co[:wn][w_st[valid]]).all()
    gc, gs = _by_coors(orc, g_co, gn, g_sc)
    wc, ws = _by_coors(orc, w_co, wn, w_sc)
    assert (gc == wc).all() and (gs == ws).all()
    o_aug, o_st, o_sc, o_co, o_n = orc.cylinder(pts, batch, cfg, shape, n)
    assert o_n == wn and ((o_st >= 0) == valid).all()
    assert np.allclose(o_aug[valid], w_aug[valid], atol=1e-3, rtol=1e-3)  # host libm vs device atan2f / sqrtf
    assert (o_co[:o_n][o_st[valid]] == w_co[:wn][w_st[valid]]).all()


@pytest.mark.parametrize("reduce_type", [0, 1])
def test_scatter_to_matches_reference_gpu(d3d, orc, ref, reduce_type):
    from deploy3d_b200.ops import data_s_scatter_to
    run = _ref_plugin(ref, "scatter_to")
    r = rng(52 + reduce_type)
    n, m, num_act, c = 100000, 32768, 30000, 9
    base = np.arange(-1, num_act, dtype=np.int32)
    idx = np.concatenate([base, r.integers(-1, num_act, n - base.size).astype(np.int32)])[r.permutation(n)]
    cnt = np.zeros(m, np.int32)
    u, k = np.unique(idx[idx >= 0], return_counts=True)
    cnt[u] = k
    x = r.standard_normal((n, c)).astype(np.float32)
    ins = [_t(x), _t(idx), _t(cnt)]
    got = d3d.scatter_to(*ins, reduce_type)
    want = run(data_s_scatter_to(reduce_type), ins, [torch.zeros_like(got)])[0]
    got, want = got.cpu().numpy(), want.cpu().numpy()
    oracle_out = orc.scatter_to(x, idx, cnt, reduce_type)
    if reduce_type == 0:
        assert (got == want).all() and (oracle_out == want).all()  # max is exact, untouched rows included
    else:
        assert np.allclose(got, want, atol=1e-3, rtol=1e-3) and np.allclose(oracle_out, want, atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("fill_val", [None, 6.9])
def test_gather_back_matches_reference_gpu(d3d, orc, ref, fill_val):
    from deploy3d_b200.ops import data_s_gather_back, gather_back
    run = _ref_plugin(ref, "gather_back")
    r = rng(61)
    n, m = 100000, 32768
    idx = r.integers(-1, m, n).astype(np.int32)
    x = r.standard_normal((m, 9)).astype(np.float32)
    init = torch.full((n, 9), 3.25, dtype=torch.float32, device=DEV)
    got = gather_back(_t(x), _t(idx), fill_val, out=init.clone()).cpu().numpy()
    want = run(data_s_gather_back(fill_val), [_t(x), _t(idx)], [init.clone()])[0].cpu().numpy()
    assert (got == want).all()
    assert (orc.gather_back(x, idx, fill_val, out_init=np.full((n, 9), 3.25, np.float32)) == want).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_bev_densify_matches_reference_gpu(d3d, orc, ref, dtype):
    from deploy3d_b200.ops import data_s_bev_densify
    run = _ref_plugin(ref, "bev_densify")
    r = rng(71)
    n_max, num_act, c = 10000, 8000, 128
    shape = [2, 0, 2, 128, 128]
    coors = np.zeros((n_max, 4), np.int32)
    coors[:num_act] = unique_coors(r, num_act, [2, 2, 128, 128])
    feats = torch.from_numpy(r.standard_normal((n_max, c)).astype(np.float32)).to(dtype).to(DEV)
    ins = [feats, _t(coors), torch.tensor([num_act], dtype=torch.int32, device=DEV), _shape_t(shape)]
    got = d3d.bev_densify(*ins, c * 2)
    want = run(data_s_bev_densify(c * 2), ins, [torch.full_like(got, 7.0)])[0]  # the reference clears the map itself
    assert torch.equal(got, want)
    assert (orc.bev_densify(feats.float().cpu().numpy(), coors, num_act, shape) == want.float().cpu().numpy()).all()


def test_nms3d_matches_reference_gpu(d3d, orc, ref):
    from deploy3d_b200 import synth
    run = _ref_plugin(ref, "nms3d")
    b = synth.config4_boxes(4, 700)
    scores, boxes = _t(b["scores"]), _t(b["boxes"])
    got = d3d.nms3d(scores, boxes)  # the plugin's constant threshold 0.1 (trt/decoder/nms3d.cu:138)
    want = run(b"", [scores, boxes], [torch.zeros_like(got)])[0]
    assert torch.equal(got, want)
    assert (orc.nms3d(b["scores"], b["boxes"], 0.1) == want.cpu().numpy()).all()


def test_nms3d_reference_gpu_at_the_threshold(d3d, ref):
    """The reference's build lets the compiler contract multiply-adds, this library's does not: on pairs within a few
    roundings of the plugin's threshold (0.1) the two may decide differently, and only there."""
    from tests.test_gpu_nms import _threshold_pairs
    run = _ref_plugin(ref, "nms3d")
    scores, boxes, iou = _threshold_pairs(0.1)
    scores, boxes = _t(scores), _t(boxes)
    got = d3d.nms3d(scores, boxes)
    want = run(b"", [scores, boxes], [torch.zeros_like(got)])[0]
    differ = (got != want).any(dim=1).cpu().numpy()
    assert (np.abs(iou[differ] - 0.1) < 1e-5).all()
    assert differ.mean() < 0.5


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_yolox3d_decode_matches_reference_gpu(d3d, orc, ref, dtype):
    from deploy3d_b200.ops import data_s_yolox3d_decode
    from tests.test_gpu_decoder import _head
    run = _ref_plugin(ref, "yolox3d_decode")
    r = rng(13)
    scores, preds = _head(r, 2, 3, 96, 104, 2)
    cfg = np.array([-54.0, -54.0, -5.0, 0.075, 0.075, 0.2], dtype=np.float32)
    stride, class_ids, topk = 8, (0, 3, 7), 300
    ins = [_t(scores).to(dtype), _t(preds).to(dtype), _t(cfg)]
    got = d3d.yolox3d_decode(*ins, stride, class_ids, topk)
    want = run(data_s_yolox3d_decode(stride, class_ids, topk), ins, [torch.zeros_like(t) for t in got])
    orc_out = orc.yolox3d_decode(ins[0].float().cpu().numpy(), ins[1].float().cpu().numpy(), cfg, stride, class_ids,
                                 topk)
    for ci in range(len(class_ids)):
        g_ids, g_sc, g_bx = (t.cpu().numpy() for t in got[3 * ci:3 * ci + 3])
        w_ids, w_sc, w_bx = (t.cpu().numpy() for t in want[3 * ci:3 * ci + 3])
        assert (g_ids == w_ids).all() and (g_sc == w_sc).all(), "class %d: selection differs from the reference" % ci
        np.testing.assert_allclose(g_bx, w_bx, rtol=1e-5, atol=1e-5)
        o_ids, o_sc, o_bx = orc_out[ci]
        assert (o_ids == w_ids).all() and (o_sc == w_sc).all()
        np.testing.assert_allclose(o_bx, w_bx, rtol=1e-5, atol=1e-5)


def test_config4_rulebooks_match_reference_gpu(d3d, orc, ref):
    """Benchmark size: the first SubM rulebook (about 281 000 voxels) and the first strided rulebook (-> about
    463 000 outputs) of a config-4 frame, product against the reference's builders: SubM byte for byte, strided
    after canonicalisation (output coordinate sets and every per-offset pair list)."""
    from deploy3d_b200 import synth
    frame = synth.config4_points()
    cfg, shape = frame["voxel_config"], frame["spatial_shape"]
    pts = frame["points"]
    pts = pts[synth.drop_edge_points(pts[:, :3], cfg[:3], cfg[3:])]
    n_pts = len(pts)
    _, coors, num = d3d.simple_mean_encoder(_t(pts), _t(np.zeros(n_pts, np.int32)), _t(cfg),
                                            torch.empty(shape, dtype=torch.int32, device=DEV), n_pts)
    n = int(num.item())
    coors = coors[:n].contiguous()
    shape_b = [shape[0]] + list(shape[2:])
    one, ks = (1, 1, 1), (3, 3, 3)
    num_t = torch.tensor([n], dtype=torch.int32, device=DEV)
    shp = torch.empty(shape, dtype=torch.int32, device=DEV)
    # SubM
    got = d3d.spconv_index(coors, num_t, shp, ks, one, one, one, (0, 0, 0), n, True, False)
    want = ref.spconv_index(coors, n, shape_b, ks, one, one, one, n, True, False)
    assert int(got[1].item()) == int(want[1].item())
    assert torch.equal(got[0], want[0])
    del got, want
    # strided 2x2x2
    st = (2, 2, 2)
    oshape = orc.out_shape(shape_b, ks, st, one, one, (0, 0, 0), False)
    cap = 2 * n
    got = d3d.spconv_index(coors, num_t, shp, ks, st, one, one, (0, 0, 0), cap, False, False)
    want = ref.spconv_index(coors, n, oshape, ks, st, one, one, cap, False, False)
    g_num, w_num, g_out, w_out = (int(t.item()) for t in (got[1], want[1], got[3], want[3]))
    assert (g_num, g_out) == (w_num, w_out) and w_out < cap
    gc, gp, _ = orc.canonical_conv(got[0].cpu().numpy(), g_num, got[2].cpu().numpy(), g_out, 27)
    wc, wp, _ = orc.canonical_conv(want[0].cpu().numpy(), w_num, want[2].cpu().numpy(), w_out, 27)
    assert (gc == wc).all()
    pairs_equal(gp, wp, 27)
