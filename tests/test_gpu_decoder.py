"""GPU parity of YoloX3dDecode (top-K select + box decode) against the numpy restatement of the reference
(oracle.yolox3d_decode): class ids and the selected cells exact, scores exact (they are copied), boxes to 1e-5
(expf / atan2f of the device and of the host libm differ in the last ulp)."""
import numpy as np
import pytest
import torch

from _util import rng

pytestmark = pytest.mark.gpu


def _head(r, b, c, ny, nx, extra, ties=False):
    scores = r.uniform(0, 1, (b, c, ny, nx)).astype(np.float32)
    if ties:  # many equal scores: the order among them must be ascending cell index
        scores = np.round(scores * 20) / 20
    preds = np.zeros((b, 9 + extra, ny, nx), dtype=np.float32)
    preds[:, 0:2] = r.uniform(-0.5, 1.5, (b, 2, ny, nx))  # a few centres leave the map: invalid boxes
    preds[:, 2] = r.uniform(-3, 1, (b, ny, nx))
    preds[:, 3:6] = r.uniform(-1.0, 1.5, (b, 3, ny, nx))
    preds[:, 6] = r.uniform(-4, 4, (b, ny, nx))
    ang = r.uniform(-np.pi, np.pi, (b, ny, nx))
    preds[:, 7], preds[:, 8] = np.sin(ang), np.cos(ang)
    preds[:, 9:] = r.standard_normal((b, extra, ny, nx))
    # keep the square / elongated decision away from its thresholds so that one ulp cannot flip it
    ratio = np.exp(preds[:, 4] - preds[:, 3])
    near = (np.abs(ratio - 0.9) < 1e-3) | (np.abs(ratio - 1.11) < 1e-3) | (np.abs(ratio - 1.0) < 1e-4)
    preds[:, 4][near] += 0.05
    return scores, preds.astype(np.float32)


def _check(d3d, orc, scores, preds, cfg, stride, class_ids, topk, dtype):
    tdt = torch.float32 if dtype == "fp32" else torch.float16
    s_t = torch.from_numpy(scores).cuda().to(tdt)
    p_t = torch.from_numpy(preds).cuda().to(tdt)
    got = d3d.yolox3d_decode(s_t, p_t, torch.from_numpy(cfg).cuda(), stride, class_ids, topk)
    want = orc.yolox3d_decode(s_t.float().cpu().numpy(), p_t.float().cpu().numpy(), cfg, stride, class_ids, topk)
    assert len(got) == 3 * len(class_ids)
    for ci, (ids, sc, bx) in enumerate(want):
        g_ids, g_sc, g_bx = (t.cpu().numpy() for t in got[3 * ci:3 * ci + 3])
        assert g_ids.dtype == np.int32 and g_ids.shape == ids.shape and (g_ids == ids).all()
        assert g_sc.shape == sc.shape and (g_sc == sc).all(), "class %d: selected cells or their order differ" % ci
        assert g_bx.shape == bx.shape
        np.testing.assert_allclose(g_bx, bx, rtol=1e-5, atol=1e-5)
    return got


@pytest.mark.parametrize("dtype", ["fp32", "fp16"])
def test_centerpoint_head_shape(d3d, orc, dtype):
    """Config-4-like head: 180 x 180 map, 3 classes in this head, top 500, one extra regression channel pair."""
    r = rng(11)
    scores, preds = _head(r, 2, 3, 180, 180, 2)
    cfg = np.array([-54.0, -54.0, -5.0, 0.075, 0.075, 0.2], dtype=np.float32)
    _check(d3d, orc, scores, preds, cfg, 8, (0, 3, 7), 500, dtype)


def test_ties_keep_ascending_cell_order(d3d, orc):
    r = rng(12)
    scores, preds = _head(r, 1, 2, 40, 56, 0, ties=True)
    cfg = np.array([0.0, -40.0, -3.0, 0.1, 0.1, 4.0], dtype=np.float32)
    _check(d3d, orc, scores, preds, cfg, 4, (1, 2), 300, "fp32")


def test_topk_larger_than_map_and_eight_classes(d3d, orc):
    r = rng(13)
    scores, preds = _head(r, 3, 8, 6, 7, 1)
    cfg = np.array([0.0, 0.0, 0.0, 0.5, 0.5, 1.0], dtype=np.float32)
    got = _check(d3d, orc, scores, preds, cfg, 2, tuple(range(8)), 100, "fp32")
    assert got[1].shape == (3, 42)  # K = min(topk, Y * X)


def test_invalid_boxes_are_marked(d3d, orc):
    r = rng(14)
    scores, preds = _head(r, 1, 1, 16, 16, 0)
    preds[0, 7:9, :4, :] = 0.0       # no direction: invalid
    preds[0, 0, 4:8, :] = np.inf     # non-finite centre
    preds[0, 3, 8:10, :] = 200.0     # exp overflows
    cfg = np.array([0.0, 0.0, 0.0, 0.2, 0.2, 1.0], dtype=np.float32)
    got = _check(d3d, orc, scores, preds, cfg, 1, (5,), 256, "fp32")
    sc = got[1].cpu().numpy()
    assert (sc == -1).sum() >= 10 * 16


def test_rejects_oversize_topk(d3d):
    from deploy3d_b200 import _lib
    s = torch.zeros((1, 1, 100, 100), device="cuda")
    p = torch.zeros((1, 9, 100, 100), device="cuda")
    with pytest.raises(_lib.D3DError):
        d3d.yolox3d_decode(s, p, torch.ones(6, device="cuda"), 1, (0,), 5000)
