"""Seeded synthetic inputs with the shapes, sizes and value distributions of the five benchmark
configurations (numpy only; ``numpy.random.Generator(PCG64(seed))``, seed = 1000 + config, + frame id).

They stand in for KITTI-/nuScenes-/SemanticKITTI-shaped data: no dataset record is reproduced, only
the geometry (grid extents, point ranges, ground-plane bias, object-like clusters, density falling
off with range).
"""
import numpy as np


def _rng(cfg, frame=0):
    return np.random.Generator(np.random.PCG64(1000 + cfg + 7919 * frame))


def kaiming_weight(rng, kvol, cin, cout):
    """[kVol, Cin, Cout] float32, std = sqrt(2 / (kVol * Cin))."""
    return (rng.standard_normal((kvol, cin, cout)) * np.sqrt(2.0 / (kvol * cin))).astype(np.float32)


def unique_voxels(rng, n, shape, batch=1):
    """n distinct (b, z, y, x) rows drawn uniformly without replacement from a [batch, Z, Y, X] grid."""
    z, y, x = shape
    total = batch * z * y * x
    ids = rng.choice(total, size=n, replace=False) if total < (1 << 26) else _sample_distinct(rng, n, total)
    out = np.empty((n, 4), dtype=np.int32)
    out[:, 3] = ids % x
    ids = ids // x
    out[:, 2] = ids % y
    ids = ids // y
    out[:, 1] = ids % z
    out[:, 0] = ids // z
    return out


def _sample_distinct(rng, n, total):
    got = np.empty(0, dtype=np.int64)
    while got.size < n:
        got = np.unique(np.concatenate([got, rng.integers(0, total, size=int((n - got.size) * 1.2) + 16)]))
    return rng.permutation(got)[:n]


def config1():
    """Single SubMConv3d 3x3x3, 16->16, fp32, 20 000 uniform voxels in 41x1600x1408, batch 1."""
    rng = _rng(1)
    shape = (41, 1600, 1408)
    coors = unique_voxels(rng, 20000, shape)
    feats = rng.standard_normal((20000, 16)).astype(np.float32)
    weight = kaiming_weight(rng, 27, 16, 16)
    bias = np.zeros(16, dtype=np.float32)
    return dict(coors=coors, feats=feats, weight=weight, bias=bias, spatial_shape=[1, 0, *shape],
                ksize=(3, 3, 3), stride=(1, 1, 1), padding=(1, 1, 1), dilation=(1, 1, 1))


def lidar_like_voxels(rng, n, shape, n_clusters=40, sigma=8.0):
    """n distinct (z, y, x) voxels: 70 % ground (z in 0..3, radius uniform so density ~ 1/r about the grid
    centre), 30 % in Gaussian clusters of `sigma` voxels."""
    z, y, x = shape
    cy, cx = y / 2.0, x / 2.0
    rmax = min(cy, cx) - 1
    centres = np.stack([rng.uniform(0, z, n_clusters), rng.uniform(0, y, n_clusters), rng.uniform(0, x, n_clusters)], 1)
    got = np.empty((0, 3), dtype=np.int64)
    while got.shape[0] < n:
        need = int((n - got.shape[0]) * 1.3) + 64
        ng = int(need * 0.7)
        r = rng.uniform(1.0, rmax, ng)
        th = rng.uniform(0, 2 * np.pi, ng)
        ground = np.stack([rng.integers(0, 4, ng), np.floor(cy + r * np.sin(th)), np.floor(cx + r * np.cos(th))], 1)
        nc = need - ng
        which = rng.integers(0, n_clusters, nc)
        clus = np.floor(centres[which] + rng.standard_normal((nc, 3)) * np.array([sigma / 4, sigma, sigma]))
        pts = np.concatenate([ground, clus]).astype(np.int64)
        pts[:, 0] = np.clip(pts[:, 0], 0, z - 1)
        pts[:, 1] = np.clip(pts[:, 1], 0, y - 1)
        pts[:, 2] = np.clip(pts[:, 2], 0, x - 1)
        got = np.unique(np.concatenate([got, pts]), axis=0)
    got = got[rng.permutation(got.shape[0])[:n]]
    return got.astype(np.int32)


def config2():
    """Strided conv k3 s2 p1 32->64 then its inverse 64->32, fp16, batch 2 x 60 000 LiDAR-like voxels."""
    rng = _rng(2)
    shape = (41, 1600, 1408)
    coors = []
    for b in range(2):
        v = lidar_like_voxels(rng, 60000, shape)
        coors.append(np.concatenate([np.full((v.shape[0], 1), b, np.int32), v], 1))
    coors = np.concatenate(coors)
    feats = rng.standard_normal((coors.shape[0], 32)).astype(np.float16)
    return dict(coors=coors, feats=feats, spatial_shape=[2, 0, *shape], ksize=(3, 3, 3), stride=(2, 2, 2),
                padding=(1, 1, 1), dilation=(1, 1, 1),
                w_down=kaiming_weight(rng, 27, 32, 64), b_down=(rng.standard_normal(64) * 0.1).astype(np.float32),
                w_up=kaiming_weight(rng, 27, 64, 32), b_up=(rng.standard_normal(32) * 0.1).astype(np.float32))


def lidar_like_points(rng, n, xr, yr, zr, extra, ground_z=-1.7, n_clusters=40, max_per_voxel=None, voxel=None):
    """n points [x, y, z, extra...]: 70 % near a ground plane with 1/r density about the sensor, 30 % in object-like
    Gaussian clusters.  `extra` is a list of callables rng,count -> column.  With `max_per_voxel`, points are thinned
    so that no cell of size `voxel` holds more (and the set is topped up)."""
    x0, x1 = xr
    y0, y1 = yr
    z0, z1 = zr
    rmax = max(abs(x0), abs(x1), abs(y0), abs(y1))
    centres = np.stack([rng.uniform(x0, x1, n_clusters), rng.uniform(y0, y1, n_clusters),
                        rng.uniform(ground_z, ground_z + 1.5, n_clusters)], 1)
    pts = np.empty((0, 3), dtype=np.float32)
    while pts.shape[0] < n:
        need = int((n - pts.shape[0]) * 1.5) + 256
        ng = int(need * 0.7)
        r = rng.uniform(2.0, rmax * 1.2, ng)
        th = rng.uniform(0, 2 * np.pi, ng)
        g = np.stack([r * np.cos(th), r * np.sin(th), ground_z + rng.standard_normal(ng) * 0.08], 1)
        nc = need - ng
        which = rng.integers(0, n_clusters, nc)
        c = centres[which] + rng.standard_normal((nc, 3)) * np.array([0.9, 0.9, 0.5])
        new = np.concatenate([g, c]).astype(np.float32)
        keep = (new[:, 0] > x0) & (new[:, 0] < x1) & (new[:, 1] > y0) & (new[:, 1] < y1) & (new[:, 2] > z0) & \
               (new[:, 2] < z1)
        new = new[keep]
        pts = np.concatenate([pts, new[rng.permutation(new.shape[0])]])
        if max_per_voxel is not None:
            cell = np.floor((pts - np.array([x0, y0, z0], np.float32)) / np.asarray(voxel, np.float32)).astype(np.int64)
            key = (cell[:, 2] * 100000 + cell[:, 1]) * 100000 + cell[:, 0]
            order = np.argsort(key, kind="stable")
            ks = key[order]
            start = np.r_[0, np.flatnonzero(np.diff(ks)) + 1]
            rank = np.arange(ks.size) - np.repeat(start, np.diff(np.r_[start, ks.size]))
            pts = pts[np.sort(order[rank < max_per_voxel])]
    pts = pts[:n]
    cols = [pts] + [f(rng, n).astype(np.float32).reshape(n, 1) for f in extra]
    return np.concatenate(cols, 1).astype(np.float32)


def config3_points():
    """SECOND-style frame: 120 000 points x (x, y, z, intensity); x [0,70.4], y [-40,40], z [-3,1];
    at most 5 points per 0.05 x 0.05 x 0.1 voxel."""
    rng = _rng(3)
    pts = lidar_like_points(rng, 120000, (0, 70.4), (-40, 40), (-3, 1), [lambda r, n: r.uniform(0, 1, n)],
                            max_per_voxel=5, voxel=(0.05, 0.05, 0.1))
    return dict(points=pts, batch=np.zeros(120000, np.int32),
                voxel_config=np.array([0, -40, -3, 0.05, 0.05, 0.1], np.float32), spatial_shape=[1, 0, 41, 1600, 1408])


def config4_points(frame=0):
    """CenterPoint-style frame: 300 000 points x (x, y, z, intensity, time); x, y [-54,54], z [-5,3];
    time in 10 sweeps of 0.05 s."""
    rng = _rng(4, frame)
    pts = lidar_like_points(rng, 300000, (-54, 54), (-54, 54), (-5, 3),
                            [lambda r, n: r.uniform(0, 1, n), lambda r, n: r.integers(0, 10, n) * 0.05])
    return dict(points=pts, batch=np.zeros(300000, np.int32),
                voxel_config=np.array([-54, -54, -5, 0.075, 0.075, 0.2], np.float32),
                spatial_shape=[1, 0, 41, 1440, 1440])


def config4_boxes(n_class=10, k=1000):
    """NMS input: `n_class` rows x `k` boxes (cx,cy,cz,dx,dy,dz,yaw), scores U(0,1) sorted descending."""
    rng = _rng(4, 99)
    xyz = np.stack([rng.uniform(-54, 54, (n_class, k)), rng.uniform(-54, 54, (n_class, k)),
                    rng.uniform(-5, 3, (n_class, k))], -1)
    dims = rng.uniform(0.5, 5.0, (n_class, k, 3))
    yaw = rng.uniform(-np.pi, np.pi, (n_class, k, 1))
    boxes = np.concatenate([xyz, dims, yaw], -1).astype(np.float32)
    scores = -np.sort(-rng.uniform(0, 1, (n_class, k)), axis=1)
    return dict(scores=scores.astype(np.float32), boxes=boxes, iou_threshold=0.2)


def config5_points(frame=0):
    """Cylinder3D-style frame: 120 000 points x (x, y, z, intensity) inside rho < 50, z in [-4, 2]."""
    rng = _rng(5, frame)
    pts = lidar_like_points(rng, 120000, (-50, 50), (-50, 50), (-4, 2), [lambda r, n: r.uniform(0, 1, n)],
                            ground_z=-1.8)
    return dict(points=pts, batch=np.zeros(120000, np.int32),
                cylinder_config=np.array([-4, -np.pi, 0, 2, np.pi, 50], np.float32),
                spatial_shape=[1, 0, 480, 360, 32])


def drop_edge_points(points, mins, steps, tol=1e-3):
    """Remove points closer than `tol` (in cell units) to a cell boundary, as the reference's encoder tests do
    (tests/voxel_encoder/test_simple_mean.py:21-24) so that float rounding cannot move a point across cells."""
    f = (points - np.asarray(mins, np.float32)) / np.asarray(steps, np.float32)
    return np.abs(f - np.round(f)).min(axis=1) > tol
