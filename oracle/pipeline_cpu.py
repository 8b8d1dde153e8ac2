"""TEST INFRASTRUCTURE ONLY -- the frame pipeline of deploy3d_b200/pipeline.py restated on the CPU oracle.

Runs the same layer list with the same seeded weights through oracle.c (scalar C, one thread per call): voxel
encoder, rulebooks, gather-GEMM-scatter with fp16-rounded operands and fp32 accumulation, ReLU / residual, BEV
densify, NMS.  Used as the parity reference of the pipeline tests and as the timed CPU baseline of bench.py.
"""
import numpy as np

from deploy3d_b200 import backbone

from . import oracle


def _round_lp(a, dtype):
    if dtype == "fp16":
        return a.astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        import torch
        return torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).to(torch.float32).numpy()
    return a


def run_net(layers, weights, feats, coors, spatial_b, dtype="fp16"):
    """feats [N, Cin] float32 (already rounded to `dtype`), coors [N, 4]; returns (feats, coors, shape, stats)."""
    rulebooks, sets = {}, {"in": (coors, list(spatial_b))}
    saved, set_of_tag = {"input": feats}, {"input": "in"}
    cur = "in"
    x = feats
    stats = []
    for L, wb in zip(layers, weights):
        if L.kind == "ew":  # element-wise graph op between plugins (fp32, result rounded like any activation)
            y = backbone.ew_apply(L.ew[0], [saved[t] for t in L.ew[1]], np)
            x, cur = _round_lp(y.astype(np.float32), dtype), set_of_tag[L.ew[1][0]]
            if L.save:
                saved[L.save], set_of_tag[L.save] = x, cur
            continue
        w, b = wb
        if L.source is not None:
            x, cur = saved[L.source], set_of_tag[L.source]
        c_in, shape_in = sets[cur]
        kvol = int(np.prod(L.ksize))
        if L.key not in rulebooks:
            if L.kind == "subm":
                index, num = oracle.rulebook_subm(c_in, shape_in, L.ksize, L.stride, L.padding, (1, 1, 1))
                rulebooks[L.key] = (index, num, cur, cur)
            else:
                index, num, oc, nout, oshape = oracle.rulebook_conv(c_in, shape_in, L.ksize, L.stride, L.padding,
                                                                    (1, 1, 1), (0, 0, 0), False,
                                                                    max(8 * len(c_in), 1))
                sets[L.key] = (oc[:nout].copy(), oshape)
                rulebooks[L.key] = (index, num, cur, L.key)
        index, num, in_set, out_set = rulebooks[L.key]
        if L.kind == "inverse":
            in_set, out_set = out_set, in_set
        m = len(sets[out_set][0])
        y = oracle.spconv_mm(x, _round_lp(w, dtype), _round_lp(b, dtype), index, num, L.kind == "inverse", m)
        if L.relu and L.act_first:
            y = np.maximum(y, 0)
        if L.residual:
            y = y + saved[L.residual]
        if L.relu and not L.act_first:
            y = np.maximum(y, 0)
        x = _round_lp(y, dtype)
        cur = out_set
        if L.save:
            saved[L.save], set_of_tag[L.save] = x, cur
        stats.append((L.cin, L.cout, kvol, m, int((index[2, :num] >= 0).sum())))
    return x, sets[cur][0], sets[cur][1], stats


def run_frame(kind, points, batch, voxel_config, spatial, boxes=None, iou_threshold=0.2, dtype="fp16", seed=0):
    """One frame on the CPU; returns dict(bev, feats, coors, nms_scores, stats, num_voxels)."""
    layers = backbone.voxel_res_backbone_8x(points.shape[1]) if kind == "centerpoint" else \
        backbone.voxel_backbone_8x(points.shape[1])
    weights = backbone.make_weights(layers, seed)
    vf, vc, vn = oracle.simple_mean(points, batch, voxel_config, spatial, len(points))
    spatial_b = [spatial[0]] + list(spatial[2:])
    x, coors, shape, stats = run_net(layers, weights, _round_lp(vf[:vn], dtype), vc[:vn], spatial_b, dtype)
    bev = oracle.bev_densify(x, coors, len(coors), [shape[0], 0] + shape[1:])
    out = dict(bev=bev, feats=x, coors=coors, stats=stats, num_voxels=vn, vox_feats=vf[:vn], vox_coors=vc[:vn])
    if boxes is not None:
        out["nms_scores"] = oracle.nms3d(boxes["scores"], boxes["boxes"], iou_threshold)
    return out


def run_segmentation_frame(points, batch, cylinder_config, spatial, n_class=None, dtype="fp16", seed=0,
                           net="cylinder3d"):
    """The Cylinder3D-shaped frame on the CPU: cylinder encoder -> scatter (max) -> network -> gather back.
    Returns dict(logits [N_pts, n_class], num_voxels)."""
    if net == "cylinder3d":
        layers = backbone.cylinder3d(points.shape[1] + 5, n_class or 20)
    else:
        layers = backbone.seg_unet(points.shape[1] + 5, n_class or 16)
    weights = backbone.make_weights(layers, seed)
    n = len(points)
    aug, scatter_index, scatter_count, coors, nv = oracle.cylinder(points, batch, cylinder_config, spatial, n)
    vox = oracle.scatter_to(aug, scatter_index, scatter_count[:nv].copy(), 0)
    spatial_b = [spatial[0]] + list(spatial[2:])
    x, _, _, _ = run_net(layers, weights, _round_lp(vox[:nv], dtype), coors[:nv], spatial_b, dtype)
    logits = oracle.gather_back(x, scatter_index, fill_val=0.0)
    return dict(logits=logits, num_voxels=nv, scatter_index=scatter_index)
