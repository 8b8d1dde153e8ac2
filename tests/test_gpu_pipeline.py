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


@pytest.mark.parametrize("net", ["cylinder3d", "unet"])
def test_segmentation_frame_matches_cpu_pipeline(d3d, net):
    """Cylinder3D-shaped chain on an azimuth sector of a config-5 frame: CylinderEncoder -> ScatterTo(max) ->
    encoder-decoder -> GatherBack.  'cylinder3d' is the network of benchmark config 5: asymmetric 3x1x3 / 1x3x3 SubM
    blocks over shared rulebooks, channels 32 / 64 / 128 / 256, strided pooling and its inverse, skip connections,
    the sigmoid ReconBlock and 20 classes (the composition of tests/cylinder/test_cylinder3d.py:100-272).  Per-point
    logits do not depend on the (implementation-defined) voxel numbering, so they are compared directly; the frame is
    then captured in a CUDA graph and replayed with the same result."""
    from deploy3d_b200 import synth
    from deploy3d_b200.pipeline import SegmentationPipeline
    from oracle import pipeline_cpu
    frame = synth.config5_points()
    pts = _sector(frame, 16)
    rho = np.sqrt(pts[:, 0] ** 2 + pts[:, 1] ** 2)
    phi = np.arctan2(pts[:, 1], pts[:, 0])
    cyl = np.stack([rho, phi, pts[:, 2]], 1)
    cfg = frame["cylinder_config"]
    shape = frame["spatial_shape"]
    mins = np.array([cfg[2], cfg[1], cfg[0]], np.float32)  # (rho, phi, z) lower bounds
    steps = (np.array([cfg[5], cfg[4], cfg[3]], np.float32) - mins) / np.array(shape[2:], np.float32)
    pts = pts[synth.drop_edge_points(cyl, mins, steps)]
    n = len(pts)
    batch = np.zeros(n, np.int32)
    probe = SegmentationPipeline("cuda:0", n_pts=n, net=net)
    caps = {k: (n if k == "in" else 4 * n) for k in probe.set_names}
    del probe
    pipe = SegmentationPipeline("cuda:0", n_pts=n, caps=caps, net=net)
    pipe.load_frame(dict(points=pts, batch=batch))
    got = pipe.enqueue().float().cpu().numpy()
    torch.cuda.synchronize()
    want = pipeline_cpu.run_segmentation_frame(pts, batch, cfg, shape, net=net)
    assert int(pipe.vox_num.item()) == want["num_voxels"]
    ref = want["logits"]
    assert got.shape == ref.shape and got.shape[1] == (20 if net == "cylinder3d" else 16)
    scale = np.sqrt((ref ** 2).mean()) + 1e-12
    err = np.abs(got - ref)
    rel_l2 = np.sqrt((err ** 2).sum() / ((ref ** 2).sum() + 1e-30))
    assert rel_l2 < 1e-2, "relative L2 error %.3e" % rel_l2
    bad = err > 2e-2 * (np.abs(ref) + scale)
    assert not bad.any(), "%d logits off, worst %.3e at scale %.3e" % (bad.sum(), err[bad].max(), scale)
    pipe.capture()
    pipe.logits.zero_()
    pipe.replay()
    torch.cuda.synchronize()
    assert np.array_equal(pipe.logits.cpu().numpy(), got), "graph replay differs from the eager frame"
    assert np.array_equal(pipe.labels.cpu().numpy(), got.argmax(1))


def test_regrouped_tables_leave_the_frames_unchanged(d3d):
    """Both pipelines with every neighbour table regrouped by offset mask (d3d_spconv_mm_regroup between the table
    build and the layers, the packed stage walk in the kernel): the detection frame's sparse features, BEV map and
    NMS scores and the segmentation frame's logits are the bytes the plain tables give, eagerly and from the graph,
    and the regrouped tables have fewer (tile, offset) blocks."""
    from deploy3d_b200 import synth
    from deploy3d_b200.pipeline import DetectionPipeline, SegmentationPipeline
    from tests._util import table_parts
    frame = synth.config4_points()
    pts = _sector(frame, 12)
    cfg = frame["voxel_config"]
    pts = pts[synth.drop_edge_points(pts[:, :3], cfg[:3], cfg[3:])]
    n = len(pts)
    boxes = synth.config4_boxes(3, 300)
    sub = dict(points=pts, batch=np.zeros(n, np.int32))
    caps = {"in": n, "down2": 8 * n, "down3": 8 * n, "down4": 8 * n, "out": 8 * n}
    outs = {}
    for regroup in (False, True):
        pipe = DetectionPipeline("centerpoint", "cuda:0", n_class=3, topk=300, n_pts=n, caps=caps, regroup=regroup)
        pipe.load_frame(sub, boxes)
        feats, coors, num = pipe.enqueue()
        torch.cuda.synchronize()
        eager = [t.clone() for t in (feats, coors, num, pipe.bev, pipe.nms_scores)]
        pipe.capture()
        pipe.bev.zero_()
        pipe.replay()
        torch.cuda.synchronize()
        for a, b in zip(eager, (feats, coors, num, pipe.bev, pipe.nms_scores)):
            assert torch.equal(a, b), "graph replay differs from the eager frame (regroup=%s)" % regroup
        blocks = 0
        for rb in pipe.net.rulebooks.values():
            cap = pipe.net.sets[rb.out_set]["cap"]
            mask = table_parts(rb.table_fwd, rb.kvol, cap)[1]
            blocks += int(sum(bin(int(v) & 0xFFFFFFFF).count("1") for v in mask.cpu().numpy()))
        outs[regroup] = (eager, blocks)
        del pipe
    for a, b in zip(outs[False][0], outs[True][0]):
        assert torch.equal(a, b), "regrouped tables change the detection frame"
    assert outs[True][1] < outs[False][1], (outs[True][1], outs[False][1])

    frame5 = synth.config5_points()
    pts5 = _sector(frame5, 16)[:20000]
    batch5 = np.zeros(len(pts5), np.int32)
    logits = {}
    for regroup in (False, True):
        probe = SegmentationPipeline("cuda:0", n_pts=len(pts5))
        caps5 = {k: (len(pts5) if k == "in" else 4 * len(pts5)) for k in probe.set_names}
        del probe
        pipe = SegmentationPipeline("cuda:0", n_pts=len(pts5), caps=caps5, regroup=regroup)
        pipe.load_frame(dict(points=pts5, batch=batch5))
        logits[regroup] = pipe.enqueue().clone()
        torch.cuda.synchronize()
        del pipe
    assert torch.equal(logits[False], logits[True]), "regrouped tables change the segmentation logits"
