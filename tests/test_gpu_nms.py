"""GPU parity of NMS3d: keep-sets must equal the oracle's (which is pinned bit-for-bit to the reference's
iou_rotated.cuh) and the committed golden keep-masks computed with the reference's own IoU code."""
import os

import numpy as np
import pytest
import torch

from tests._util import rng

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def test_golden_keep_masks(d3d):
    g = np.load(os.path.join(GOLD, "nms_ref.npz"))
    for name in ("b1k128", "b2k256", "b3k200"):
        for thr, tag in ((None, "01"), (0.2, "02")):
            out = d3d.nms3d(_t(g[name + "_scores"]), _t(g[name + "_boxes"]), thr).cpu().numpy()
            keep = g["%s_keep_%s" % (name, tag)]
            assert ((out >= 0) == keep).all()
            assert (out[keep] == g[name + "_scores"][keep]).all() and (out[~keep] == -1).all()


@pytest.mark.parametrize("batch,topk", [(1, 256), (2, 256), (1, 128), (2, 128), (3, 1000), (1, 65), (2, 1), (1, 1300)])
def test_reference_cases(d3d, orc, batch, topk):
    """tests/decoder/test_nms3d.py:8-40 (monotone scores, unit-normal centres, sizes in [0.5, 1.5])."""
    r = rng(80 + batch * 1000 + topk)
    scores = np.tile(1 - np.arange(topk, dtype=np.float32) / topk, (batch, 1))
    spread = 1.0 if topk <= 256 else 4.0
    boxes = np.concatenate([r.standard_normal((batch, topk, 3)) * spread, r.uniform(0, 1, (batch, topk, 3)) + 0.5,
                            (r.uniform(0, 1, (batch, topk, 1)) - 0.5) * 2 * np.pi], -1).astype(np.float32)
    out = d3d.nms3d(_t(scores), _t(boxes)).cpu().numpy()
    want = orc.nms3d(scores, boxes, 0.1)
    assert (out == want).all()
    assert (out >= 0).sum() >= batch


def _threshold_pairs(thr, n=4096, seed=81):
    """n rows of two equal axis-aligned boxes whose IoU = (w - dx) / (w + dx) steps through `thr` in float32 ulps of
    the shift dx (three in ten pairs are a thousandth of dx away from it instead).  Returns scores, boxes and the IoU of every pair in double precision."""
    r = rng(seed)
    w = r.uniform(0.5, 4.0, n).astype(np.float32)
    h = r.uniform(0.5, 4.0, n).astype(np.float32)
    dx = (w.astype(np.float64) * (1 - thr) / (1 + thr)).astype(np.float32)
    steps = r.integers(-6, 7, n)
    for _ in range(6):  # move dx by up to six representable numbers either way
        dx = np.where(steps > 0, np.nextafter(dx, np.float32(np.inf)), dx)
        dx = np.where(steps < 0, np.nextafter(dx, np.float32(-np.inf)), dx)
        steps = steps - np.sign(steps)
    clear = r.random(n) < 0.3  # and some pairs clearly on either side
    dx = np.where(clear, dx * np.where(r.random(n) < 0.5, 1.001, 0.999).astype(np.float32), dx).astype(np.float32)
    boxes = np.zeros((n, 2, 7), np.float32)
    boxes[:, :, 0] = r.uniform(-50, 50, n).astype(np.float32)[:, None]
    boxes[:, 1, 0] += dx
    boxes[:, :, 1] = r.uniform(-50, 50, n).astype(np.float32)[:, None]
    boxes[:, :, 3], boxes[:, :, 4], boxes[:, :, 5] = w[:, None], h[:, None], 1.0
    true_dx = boxes[:, 1, 0].astype(np.float64) - boxes[:, 0, 0].astype(np.float64)
    iou = (w - true_dx) / (w + true_dx)
    scores = np.tile(np.array([0.9, 0.8], np.float32), (n, 1))
    return scores, boxes, iou


@pytest.mark.parametrize("thr", [0.1, 0.2])
def test_pairs_at_the_threshold(d3d, orc, thr):
    """Pairs whose IoU lies within a few float32 roundings of the threshold: this library evaluates the reference's
    arithmetic without fused multiply-adds, as the oracle does, so the two agree on every pair, whichever side of
    the threshold the rounding puts it.  Axis-aligned boxes: no sine / cosine implementation enters."""
    scores, boxes, iou = _threshold_pairs(thr)
    out = d3d.nms3d(_t(scores), _t(boxes), thr).cpu().numpy()
    want = orc.nms3d(scores, boxes, thr)
    assert (out == want).all()
    dropped = out[:, 1] < 0
    assert 0.2 < dropped.mean() < 0.8  # the cases straddle the threshold
    far = np.abs(iou - thr) > 1e-5     # away from it the outcome is the exact one
    assert (dropped[far] == (iou[far] > thr)).all()


def test_config4_boxes(d3d, orc):
    """benchmark config 4: 10 classes x 1000 boxes, IoU 0.2, 9-wide boxes (extra columns are ignored)."""
    from deploy3d_b200 import synth
    c = synth.config4_boxes()
    boxes = np.concatenate([c["boxes"], np.ones((10, 1000, 2), np.float32)], -1)
    out = d3d.nms3d(_t(c["scores"]), _t(boxes), c["iou_threshold"]).cpu().numpy()
    want = orc.nms3d(c["scores"], boxes, c["iou_threshold"])
    assert (out == want).all()
    # dense scene: many overlaps
    r = rng(90)
    boxes[..., :2] = r.uniform(-8, 8, (10, 1000, 2))
    out = d3d.nms3d(_t(c["scores"]), _t(boxes), 0.2).cpu().numpy()
    want = orc.nms3d(c["scores"], boxes, 0.2)
    assert (out == want).all() and (out < 0).mean() > 0.5
