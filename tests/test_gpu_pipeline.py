"""GPU parity of the whole frame pipeline (voxel encoder -> VoxelResBackBone8x / VoxelBackBone8x -> BEV densify,
plus NMS) against the CPU restatement in oracle/pipeline_cpu.py, on an azimuth sector of a synthetic frame.
The dense BEV map is independent of the voxel numbering, so it is compared directly."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _sector(frame, denom, which=0):
    pts = frame["points"]
    az = np.arctan2(pts[:, 1], pts[:, 0])
    edges = np.quantile(az, np.linspace(0, 1, denom + 1))
    m = (az >= edges[which]) & (az < edges[which + 1])
    return pts[m]


@pytest.mark.parametrize("kind,denom", [("centerpoint", 24), ("second", 10)])
@pytest.mark.parametrize("graph", [False, True])
def test_frame_matches_cpu_pipeline(d3d, kind, denom, graph):
    from deploy3d_b200 import synth
    from deploy3d_b200.pipeline import DetectionPipeline
    from oracle import pipeline_cpu
    frame = synth.config4_points() if kind == "centerpoint" else synth.config3_points()
    pts = _sector(frame, denom)
    cfg = frame["voxel_config"]
    pts = pts[synth.drop_edge_points(pts[:, :3], cfg[:3], cfg[3:])]
    n = len(pts)
    boxes = synth.config4_boxes(3, 300)
    sub = dict(points=pts, batch=np.zeros(n, np.int32))
    pipe = DetectionPipeline(kind, "cuda:0", n_class=3, topk=300, n_pts=n,
                             caps={"in": n, "down2": 8 * n, "down3": 8 * n, "down4": 8 * n, "out": 8 * n})
    pipe.load_frame(sub, boxes)
    if graph:
        pipe.capture()
        pipe.replay()
        pipe.replay()  # replays are idempotent: every buffer is rewritten from the inputs
    else:
        pipe.enqueue()
    torch.cuda.synchronize()
    want = pipeline_cpu.run_frame(kind, pts, sub["batch"], cfg, frame["spatial_shape"], boxes, 0.2)
    counts = pipe.net.counts()
    assert int(pipe.vox_num.item()) == want["num_voxels"]
    assert counts[pipe.net.out_set] == len(want["coors"])
    got = pipe.bev.float().cpu().numpy()
    ref = want["bev"]
    assert got.shape == ref.shape
    assert ((got != 0) == (ref != 0)).mean() > 0.999  # same occupied cells (ReLU zeros may differ by rounding)
    # 21 (or 12) fp16 layers deep: every layer rounds its output to fp16 on both sides, in different summation
    # orders.  Tolerance 1e-2 of the feature scale (RMS over occupied cells) in the L2 sense, 2e-2 per element.
    scale = np.sqrt((ref[ref != 0] ** 2).mean()) + 1e-12
    err = np.abs(got - ref)
    rel_l2 = np.sqrt((err ** 2).sum() / ((ref ** 2).sum() + 1e-30))
    assert rel_l2 < 1e-2, "relative L2 error %.3e" % rel_l2
    bad = err > 2e-2 * (np.abs(ref) + scale)
    assert not bad.any(), "%d cells off, worst %.3e at scale %.3e" % (bad.sum(), err[bad].max(), scale)
    assert (pipe.nms_scores.cpu().numpy() == want["nms_scores"]).all()
