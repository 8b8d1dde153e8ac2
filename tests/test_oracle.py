"""CPU tests of the oracle itself: it must agree with the reference's own code (golden vectors from the host
build of trt/decoder/iou_rotated.cuh), with the properties the reference's tests assert, and with a brute-force
dictionary model of the rulebook."""
import ctypes
import os

import numpy as np
import pytest

from tests._util import pairs_equal, rng, unique_coors

GOLD = os.path.join(os.path.dirname(__file__), "golden")
f32p = ctypes.POINTER(ctypes.c_float)


def test_iou_matches_reference_golden(orc):
    g = np.load(os.path.join(GOLD, "iou_ref.npz"))
    a, b = g["a"], g["b"]
    inter = np.array([orc.lib().orc_rotated_intersection(*[float(v) for v in a[i, [0, 1, 3, 4, 6]]],
                                                         *[float(v) for v in b[i, [0, 1, 3, 4, 6]]])
                      for i in range(len(a))], np.float32)
    iou = np.array([orc.bev_iou(a[i], b[i]) for i in range(len(a))], np.float32)
    assert (inter.view(np.uint32) == g["inter"].view(np.uint32)).all(), "intersection area not bit-identical"
    assert (iou.view(np.uint32) == g["iou"].view(np.uint32)).all(), "IoU not bit-identical"
    assert (g["inter"] > 0).sum() > 300  # the vectors exercise the clipping path


def test_iou_matches_reference_library_when_present(orc):
    ref = orc.ref_iou_lib()
    if ref is None:
        pytest.skip("oracle/_ref/libref_iou.so not built on this machine (the golden vectors cover it)")
    r = rng(7)
    for _ in range(3000):
        a = np.r_[r.standard_normal(3), r.uniform(0.2, 3, 3), r.uniform(-4, 4)].astype(np.float32)
        b = np.r_[r.standard_normal(3), r.uniform(0.2, 3, 3), r.uniform(-4, 4)].astype(np.float32)
        want = ref.ref_bev_iou(a.ctypes.data_as(f32p), b.ctypes.data_as(f32p))
        got = orc.bev_iou(a, b)
        assert np.float32(got).view(np.uint32) == np.float32(want).view(np.uint32)


def test_nms_matches_reference_golden(orc):
    g = np.load(os.path.join(GOLD, "nms_ref.npz"))
    for name in ("b1k128", "b2k256", "b3k200"):
        for thr, tag in ((0.1, "01"), (0.2, "02")):
            out = orc.nms3d(g[name + "_scores"], g[name + "_boxes"], thr)
            assert ((out >= 0) == g["%s_keep_%s" % (name, tag)]).all()
            assert (out[out >= 0] == g[name + "_scores"][out >= 0]).all()


def test_rulebook_golden(orc):
    g = np.load(os.path.join(GOLD, "rulebook_small.npz"))
    coors, shape = g["coors"], [int(v) for v in g["shape"]]
    index, num = orc.rulebook_subm(coors, shape, (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1))
    assert (index[:, :num] == g["subm_index"]).all()
    index, num, oc, nout, _ = orc.rulebook_conv(coors, shape, (3, 3, 3), (2, 2, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0),
                                                False, 100000)
    assert (index[:, :num] == g["down_index"]).all()
    assert (oc[orc.lex_order(oc[:nout])] == g["down_out_coors"]).all()


def _ref_gpu_golden():
    path = os.path.join(GOLD, "spconv_ref_gpu.npz")
    return np.load(path) if os.path.exists(path) else None


REF_GPU_CASES = ["subm", "subm_pad", "subm_dil", "subm_313", "down221", "down222", "down_k2", "up222"]


@pytest.mark.parametrize("name", REF_GPU_CASES)
def test_rulebook_matches_reference_gpu_golden(orc, name):
    """The oracle against rulebooks the reference's own GPU code produced on a B200 (trt/spconv/index.cu compiled
    for sm_100a; generator tests/golden/make_golden_gpu.py): SubM byte for byte with the padding, strided and
    transposed after the canonicalisation that removes the reference's race-dependent output numbering."""
    g = _ref_gpu_golden()
    assert g is not None, "tests/golden/spconv_ref_gpu.npz is part of the repository"
    p = [int(v) for v in g[name + "_params"]]
    ks, st, pd, dl, op = (tuple(p[i * 3:i * 3 + 3]) for i in range(5))
    tr, subm, n_max, max_out = bool(p[15]), bool(p[16]), p[17], p[18]
    coors, shape = g[name + "_coors"], [int(v) for v in g[name + "_shape"]]
    kvol = int(np.prod(ks))
    if subm:
        index, num = orc.rulebook_subm(coors, shape, ks, st, pd, dl, max_num_act_in=n_max)
        assert num == int(g[name + "_num"])
        assert index.shape == g[name + "_index"].shape and (index == g[name + "_index"]).all()
        return
    index, num, oc, nout, _ = orc.rulebook_conv(coors, shape, ks, st, pd, dl, op, tr, max_out, max_num_act_in=n_max)
    assert num == int(g[name + "_num"])
    cc, pairs, _ = orc.canonical_conv(index, num, oc, nout, kvol)
    assert cc.shape == g[name + "_out_coors"].shape and (cc == g[name + "_out_coors"]).all()
    flat = np.concatenate([np.concatenate([np.full((len(pairs[k]), 1), k, np.int64), pairs[k]], 1)
                           for k in range(kvol)])
    assert flat.shape == g[name + "_pairs"].shape and (flat == g[name + "_pairs"]).all()


@pytest.mark.parametrize("tag,index_key,inverse", [("mm_subm", "subm_index", False),
                                                   ("mm_down221", "mm_down221_index", False),
                                                   ("mm_down221_inv", "mm_down221_inv_index", True)])
def test_conv_matches_reference_gpu_golden(orc, tag, index_key, inverse):
    """The oracle's fp32 gather-GEMM-scatter against the reference's indexedSpConv output (fp16 operands, half
    atomic adds, trt/spconv/mm.h:35-71) recorded on a B200, at the tolerance of the reference's own test
    (tests/spconv/test_spconv.py:152-161: rtol 1e-2, atol 1e-1)."""
    g = _ref_gpu_golden()
    assert g is not None
    index, want = g[index_key], g[tag + "_out"].astype(np.float32)
    num = int(g["subm_num"] if tag == "mm_subm" else g["down221_num"])
    got = orc.spconv_mm(g[tag + "_feats"].astype(np.float32), g[tag + "_w"].astype(np.float32),
                        g[tag + "_b"].astype(np.float32), index, num, inverse, want.shape[0])
    assert got.shape == want.shape
    assert np.allclose(got, want, rtol=1e-2, atol=1e-1), "worst |diff| %.3e" % np.abs(got - want).max()
    assert np.sqrt(((got - want) ** 2).sum() / (want ** 2).sum()) < 5e-3


CASES = [
    # ksize, stride, pad, dil, out_pad, transpose, subm
    ((3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), False, True),
    ((3, 1, 3), (1, 1, 1), (1, 0, 1), (1, 1, 1), (0, 0, 0), False, True),
    ((1, 3, 3), (1, 1, 1), (0, 1, 1), (1, 1, 1), (0, 0, 0), False, True),
    ((3, 3, 3), (1, 1, 1), (2, 2, 2), (2, 2, 2), (0, 0, 0), False, True),
    ((3, 3, 3), (2, 2, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), False, False),
    ((3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1), (0, 0, 0), False, False),
    ((3, 3, 3), (2, 2, 2), (0, 1, 1), (1, 1, 1), (0, 0, 0), False, False),
    ((3, 1, 1), (2, 1, 1), (0, 0, 0), (1, 1, 1), (0, 0, 0), False, False),
    ((2, 2, 2), (2, 2, 2), (0, 0, 0), (1, 1, 1), (0, 0, 0), False, False),
    ((3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1), (1, 1, 1), True, False),
    ((2, 2, 2), (2, 2, 2), (0, 0, 0), (1, 1, 1), (0, 0, 0), True, False),
]


@pytest.mark.parametrize("case", CASES)
def test_rulebook_vs_brute_force(orc, case):
    ks, st, pd, dl, op, tr, subm = case
    r = rng(hash(case) % 100000)
    shape = [2, 7, 9, 8]
    coors = unique_coors(r, 300, shape)
    kvol = int(np.prod(ks))
    bc, bp = orc.brute_rulebook(coors, shape, ks, st, pd, dl, op, tr, subm)
    if subm:
        index, num = orc.rulebook_subm(coors, shape, ks, st, pd, dl, max_num_act_in=350)
        orc.check_layout(index, num, kvol)
        pairs_equal(orc.canonical_pairs(index, num, kvol), bp, kvol)
    else:
        index, num, oc, nout, oshape = orc.rulebook_conv(coors, shape, ks, st, pd, dl, op, tr, 100000,
                                                         max_num_act_in=350)
        orc.check_layout(index, num, kvol)
        cc, pairs, _ = orc.canonical_conv(index, num, oc, nout, kvol)
        assert nout == len(bc) and (cc == np.asarray(bc)).all()
        pairs_equal(pairs, bp, kvol)


def test_subm_mirror_property(orc):
    """tests/spconv/test_spconv.py:101-108: offset k and kVol-1-k are mirror images with swapped roles and the
    centre offset is the identity."""
    r = rng(11)
    shape = [2, 20, 18, 8]
    coors = unique_coors(r, 1500, shape)
    index, num = orc.rulebook_subm(coors, shape, (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1))
    p = orc.canonical_pairs(index, num, 27)
    assert (p[13] == np.stack([np.arange(1500)] * 2, 1)).all()
    for k in range(13):
        m = p[26 - k][:, ::-1]
        m = m[np.lexsort((m[:, 1], m[:, 0]))]
        assert (p[k] == m).all()


def test_truncation(orc):
    """maxNumActOut smaller than the number of outputs: exactly max are kept, all genuine, pairs restricted to them
    (tests/spconv/test_spconv.py:72-80, :110-114)."""
    r = rng(12)
    shape = [2, 30, 24, 8]
    coors = unique_coors(r, 2000, shape)
    args = ((3, 3, 3), (2, 2, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), False)
    full = orc.rulebook_conv(coors, shape, *args, 100000)
    cut = orc.rulebook_conv(coors, shape, *args, 500)
    assert cut[3] == 500 and full[3] > 500
    full_set = {tuple(c) for c in full[2][:full[3]].tolist()}
    kept = [tuple(c) for c in cut[2][:500].tolist()]
    assert len(set(kept)) == 500 and set(kept) <= full_set
    orc.check_layout(cut[0], cut[1], 27)
    _, bp = orc.brute_rulebook(coors, shape, *args, False)
    bc, _ = orc.brute_rulebook(coors, shape, *args, False)
    ids = {tuple(c): i for i, c in enumerate(np.asarray(bc).tolist())}
    cut_ids = np.array([ids[c] for c in kept])
    pairs = orc.canonical_pairs(cut[0], cut[1], 27, cut_ids)
    present = np.zeros(len(bc), bool)
    present[cut_ids] = True
    for k in range(27):
        want = bp[k][present[bp[k][:, 1]]]
        assert (pairs[k] == want).all()


def test_empty_inputs(orc):
    index, num = orc.rulebook_subm(np.zeros((0, 4), np.int32), [1, 4, 4, 4], (3, 3, 3), (1, 1, 1), (1, 1, 1),
                                   (1, 1, 1), max_num_act_in=16)
    assert num == 0
    out = orc.spconv_mm(np.zeros((4, 3), np.float32), np.ones((27, 3, 2), np.float32), np.array([1, 2], np.float32),
                        index, num, False, 5)
    assert (out == np.array([1, 2], np.float32)).all()
    f, c, n = orc.simple_mean(np.zeros((0, 4), np.float32), np.zeros(0, np.int32), [0, 0, 0, 1, 1, 1],
                              [1, 0, 4, 4, 4], 8)
    assert n == 0


def test_mm_against_dense_convolution(orc):
    """The gather-GEMM-scatter restatement equals a dense 3-D cross-correlation on a small grid."""
    import torch
    r = rng(13)
    shape = [1, 6, 7, 5]
    coors = unique_coors(r, 120, shape)
    cin, cout = 3, 4
    feats = r.standard_normal((120, cin)).astype(np.float32)
    w = r.standard_normal((27, cin, cout)).astype(np.float32)
    bias = r.standard_normal(cout).astype(np.float32)
    dense = np.zeros((1, cin, 6, 7, 5), np.float32)
    dense[0, :, coors[:, 1], coors[:, 2], coors[:, 3]] = feats
    wt = torch.from_numpy(w.reshape(3, 3, 3, cin, cout)).permute(4, 3, 0, 1, 2).contiguous()
    for stride in ((1, 1, 1), (2, 2, 1)):
        index, num, oc, nout, oshape = orc.rulebook_conv(coors, shape, (3, 3, 3), stride, (1, 1, 1), (1, 1, 1),
                                                         (0, 0, 0), False, 10000)
        out = orc.spconv_mm(feats, w, bias, index, num, False, nout)
        ref = torch.nn.functional.conv3d(torch.from_numpy(dense), wt, torch.from_numpy(bias), stride=stride,
                                         padding=1).numpy()
        got = out[:nout]
        want = ref[0][:, oc[:nout, 1], oc[:nout, 2], oc[:nout, 3]].T
        assert np.allclose(got, want, rtol=1e-4, atol=1e-4)


def test_encoders_against_numpy(orc):
    """simple-mean / cylinder / scatter / gather restatements against direct numpy group-bys
    (the semantics the reference's tests use: tests/voxel_encoder/*.py, tests/point_voxel_mapping/*.py)."""
    r = rng(14)
    n = 5000
    pts = np.stack([r.uniform(-12, 12, n), r.uniform(-12, 12, n), r.uniform(-3, 3, n), r.standard_normal(n)],
                   1).astype(np.float32)
    pts[5] = np.nan
    batch = r.integers(-1, 2, n).astype(np.int32)
    cfg = np.array([-10, -10, -2, 0.5, 0.5, 0.25], np.float32)
    shape = [2, 0, 16, 40, 40]
    feats, coors, num = orc.simple_mean(pts, batch, cfg, shape, 100000)
    f = (pts[:, :3] - cfg[:3]) / cfg[3:]
    with np.errstate(invalid="ignore"):
        c = f.astype(np.int32)  # truncation toward zero
    ok = np.isfinite(pts).all(1) & (batch >= 0) & (c[:, 0] >= 0) & (c[:, 0] < 40) & (c[:, 1] >= 0) & (c[:, 1] < 40) & \
        (c[:, 2] >= 0) & (c[:, 2] < 16)
    key = np.stack([batch, c[:, 2], c[:, 1], c[:, 0]], 1)[ok]
    uniq, inv = np.unique(key, axis=0, return_inverse=True)
    inv = inv.reshape(-1)
    assert num == len(uniq)
    order = orc.lex_order(coors[:num])
    assert (coors[:num][order] == uniq).all()
    sums = np.zeros((len(uniq), 4))
    np.add.at(sums, inv, pts[ok].astype(np.float64))
    cnt = np.bincount(inv, minlength=len(uniq))[:, None]
    assert np.allclose(feats[:num][order], sums / cnt, rtol=1e-4, atol=1e-4)
    # scatter / gather
    m = 300
    idx = r.integers(-1, m, n).astype(np.int32)
    cnts = np.bincount(idx[idx >= 0], minlength=m).astype(np.int32)
    x = r.standard_normal((n, 6)).astype(np.float32)
    mx = orc.scatter_to(x, idx, cnts, 0)
    mean = orc.scatter_to(x, idx, cnts, 1)
    for v in range(0, m, 37):
        sel = x[idx == v]
        if len(sel):
            assert (mx[v] == sel.max(0)).all()
            assert np.allclose(mean[v], sel.mean(0), rtol=1e-4, atol=1e-5)
    back = orc.gather_back(mx, idx, fill_val=6.9)
    assert (back[idx >= 0] == mx[idx[idx >= 0]]).all() and (back[idx < 0] == np.float32(6.9)).all()
    keep = orc.gather_back(mx, idx, out_init=np.full((n, 6), 3.0, np.float32))
    assert (keep[idx < 0] == 3.0).all()
    dense = orc.bev_densify(feats[:num], coors[:num], num, shape)
    assert dense.shape == (2, 4 * 16, 40, 40)
    i = 17
    b, z, y, xx = coors[i]
    assert (dense[b].reshape(4, 16, 40, 40)[:, z, y, xx] == feats[i]).all()
    assert np.count_nonzero(dense) <= num * 4


def test_cylinder_against_numpy(orc):
    r = rng(15)
    n = 4000
    pts = np.stack([r.standard_normal(n) * 20, r.standard_normal(n) * 20, r.standard_normal(n) * 3 + 1,
                    r.standard_normal(n)], 1).astype(np.float32)
    batch = r.integers(0, 2, n).astype(np.int32)
    cfg = np.array([-2, -np.pi, 0, 4, np.pi, 50], np.float32)
    shape = [2, 0, 48, 36, 8]
    aug, st, sc, coors, num = orc.cylinder(pts, batch, cfg, shape, 100000)
    rho = np.sqrt(pts[:, 0] ** 2 + pts[:, 1] ** 2)
    phi = np.arctan2(pts[:, 1], pts[:, 0])
    step = (cfg[3:] - cfg[:3]) / np.array([8, 36, 48], np.float32)
    f = (np.stack([pts[:, 2], phi, rho], 1) - cfg[:3]) / step
    c = f.astype(np.int32)
    valid = (c[:, 1] >= 0) & (c[:, 1] < 36) & (c[:, 2] >= 0) & (c[:, 2] < 48)
    c[:, 0] = np.clip(c[:, 0], 0, 7)
    assert ((st >= 0) == valid).all()
    key = np.stack([batch, c[:, 2], c[:, 1], c[:, 0]], 1)
    uniq, inv, cnt = np.unique(key[valid], axis=0, return_inverse=True, return_counts=True)
    assert num == len(uniq)
    assert (coors[st[valid]] == key[valid]).all()
    assert (sc[st[valid]] == cnt[inv.reshape(-1)]).all()
    ctr = (c + 0.5) * step + cfg[:3]
    want = np.concatenate([np.stack([pts[:, 2], phi, rho], 1), np.stack([pts[:, 2], phi, rho], 1) - ctr,
                           pts[:, :2], pts[:, 3:]], 1)
    assert np.allclose(aug[valid], want[valid], atol=1e-3, rtol=1e-3)
    assert (aug[~valid] == 0).all()


def test_yolox3d_decode_oracle_properties(orc):
    """The numpy restatement of YoloX3dDecode: K = min(topk, Y*X), scores non-increasing per row apart from the
    -1 of invalid boxes, equal scores in ascending cell order, nearly square boxes get dx == dy and the heading of
    the direction head, headings of elongated boxes end up in (-pi, pi] on the side of the direction head."""
    r = rng(5)
    b, c, ny, nx = 2, 2, 9, 11
    scores = (np.round(r.uniform(0, 1, (b, c, ny, nx)) * 10) / 10).astype(np.float32)
    preds = r.uniform(-1, 1, (b, 9, ny, nx)).astype(np.float32)
    preds[:, 0:2] = r.uniform(0, 1, (b, 2, ny, nx))
    cfg = np.array([-10, -20, -3, 0.25, 0.25, 4], dtype=np.float32)
    out = orc.yolox3d_decode(scores, preds, cfg, 4, (2, 5), 1000)
    assert len(out) == 2
    for ci, (ids, sc, bx) in enumerate(out):
        assert ids.shape == (b, ny * nx) and (ids == (2, 5)[ci]).all() and bx.shape == (b, ny * nx, 7)
        for bi in range(b):
            flat = scores[bi, ci].reshape(-1)
            order = np.lexsort((np.arange(flat.size), -flat))
            assert (np.where(sc[bi] >= 0, sc[bi], flat[order]) == flat[order]).all()
            x0 = -10 + 4 * 0.25 * (preds[bi, 0].reshape(-1)[order] + order % nx)
            ok = sc[bi] >= 0
            np.testing.assert_allclose(bx[bi, ok, 0], x0[ok], rtol=1e-5, atol=1e-5)
            assert (np.abs(bx[bi, ok, 6]) <= np.pi + 1e-5).all()
            square = ok & (bx[bi, :, 3] == bx[bi, :, 4])
            want_dir = np.arctan2(preds[bi, 7].reshape(-1)[order], preds[bi, 8].reshape(-1)[order])
            np.testing.assert_allclose(bx[bi, square, 6], want_dir[square], rtol=1e-5, atol=1e-6)
            assert (bx[bi, ok & ~square, 3] >= bx[bi, ok & ~square, 4]).all()
