"""TEST INFRASTRUCTURE ONLY -- Python face of the CPU oracle.

Loads ``oracle/liboracle.so`` (built from ``oracle/oracle.c`` by ``make -C oracle``) and
exposes numpy-in / numpy-out wrappers, the canonicalisation used to compare rulebooks whose
output-voxel order is implementation defined, and a brute-force dictionary model of the
rulebook used to cross-check the C restatement on small grids.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may import
this module; the product package never does.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

_i32p = ctypes.POINTER(ctypes.c_int32)
_i64p = ctypes.POINTER(ctypes.c_int64)
_f32p = ctypes.POINTER(ctypes.c_float)


def build():
    """Compile the oracle and, when the reference checkout is present, the reference-derived libraries under
    oracle/_ref (host build of its IoU header; its GPU sources for sm_100a).  Only the oracle itself is required:
    a reference target that cannot be built here leaves the prebuilt library, if any, in place."""
    subprocess.run(["make", "-C", _HERE, "--no-print-directory", "liboracle.so"], check=True, capture_output=True)
    subprocess.run(["make", "-C", _HERE, "--no-print-directory", "-k", "ref", "ref_spconv", "ref_plugins"],
                   check=False, capture_output=True)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        _LIB = ctypes.CDLL(path)
        _LIB.orc_rotated_intersection.restype = ctypes.c_float
        _LIB.orc_rotated_intersection.argtypes = [ctypes.c_float] * 10
        _LIB.orc_bev_iou.restype = ctypes.c_float
        _LIB.orc_bev_iou.argtypes = [_f32p, _f32p]
    return _LIB


def ref_iou_lib():
    """The reference's own iou_rotated.cuh compiled for the host, or None when it was never built."""
    global _REF
    if _REF is None:
        path = os.path.join(_HERE, "_ref", "libref_iou.so")
        if not os.path.exists(path):
            return None
        _REF = ctypes.CDLL(path)
        _REF.ref_rotated_intersection.restype = ctypes.c_float
        _REF.ref_rotated_intersection.argtypes = [ctypes.c_float] * 10
        _REF.ref_bev_iou.restype = ctypes.c_float
        _REF.ref_bev_iou.argtypes = [_f32p, _f32p]
    return _REF


def _p(a, t):
    return a.ctypes.data_as(t)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _vec(v, ndim):
    a = np.asarray(v, dtype=np.int32).reshape(-1)
    assert a.size == ndim
    return np.ascontiguousarray(a)


def kernel_volume(ksize):
    return int(np.prod(np.asarray(ksize, dtype=np.int64)))


def out_shape(in_shape, ksize, stride, pad, dil, out_pad, transpose):
    """[B, D..] -> [B, D'..] (trt/spconv/geometry.h:118-169)."""
    ndim = len(ksize)
    ins = np.ascontiguousarray(in_shape, dtype=np.int64)
    outs = np.zeros(ndim + 1, dtype=np.int64)
    lib().orc_out_shape(ndim, _p(ins, _i64p), _p(_vec(ksize, ndim), _i32p), _p(_vec(stride, ndim), _i32p),
                        _p(_vec(pad, ndim), _i32p), _p(_vec(dil, ndim), _i32p), _p(_vec(out_pad, ndim), _i32p),
                        int(bool(transpose)), _p(outs, _i64p))
    return [int(v) for v in outs]


def index_row_len(max_num_act_in, ksize):
    """Row length of the ``index`` tensor: kVol * (maxNumActIn + 128) (trt/spconv/index_trt.cu:91-92)."""
    return kernel_volume(ksize) * (int(max_num_act_in) + 128)


def rulebook_subm(coors, shape, ksize, stride, pad, dil, max_num_act_in=None):
    """Returns (index [3, L] int32, num_index)."""
    coors = _i32(coors)
    n, ndim = coors.shape[0], coors.shape[1] - 1
    row_len = index_row_len(n if max_num_act_in is None else max_num_act_in, ksize)
    index = np.full((3, row_len), -1, dtype=np.int32)
    num_index = ctypes.c_int32(0)
    shp = np.ascontiguousarray(shape, dtype=np.int64)
    rc = lib().orc_rulebook_subm(ndim, _p(coors, _i32p), ctypes.c_int64(n), _p(shp, _i64p),
                                 _p(_vec(ksize, ndim), _i32p), _p(_vec(stride, ndim), _i32p),
                                 _p(_vec(pad, ndim), _i32p), _p(_vec(dil, ndim), _i32p), _p(index, _i32p),
                                 ctypes.c_int64(row_len), ctypes.byref(num_index))
    assert rc == 0
    return index, int(num_index.value)


def rulebook_conv(coors, in_shape, ksize, stride, pad, dil, out_pad, transpose, max_num_act_out,
                  max_num_act_in=None):
    """Returns (index [3, L], num_index, out_coors [max_out, ndim+1], num_act_out, out_shape)."""
    coors = _i32(coors)
    n, ndim = coors.shape[0], coors.shape[1] - 1
    oshape = out_shape(in_shape, ksize, stride, pad, dil, out_pad, transpose)
    row_len = index_row_len(n if max_num_act_in is None else max_num_act_in, ksize)
    index = np.full((3, row_len), -1, dtype=np.int32)
    out_coors = np.zeros((max_num_act_out, ndim + 1), dtype=np.int32)
    num_index, num_out = ctypes.c_int32(0), ctypes.c_int32(0)
    shp = np.ascontiguousarray(oshape, dtype=np.int64)
    rc = lib().orc_rulebook_conv(ndim, _p(coors, _i32p), ctypes.c_int64(n), _p(shp, _i64p),
                                 _p(_vec(ksize, ndim), _i32p), _p(_vec(stride, ndim), _i32p),
                                 _p(_vec(pad, ndim), _i32p), _p(_vec(dil, ndim), _i32p), int(bool(transpose)),
                                 ctypes.c_int32(max_num_act_out), _p(index, _i32p), ctypes.c_int64(row_len),
                                 ctypes.byref(num_index), _p(out_coors, _i32p), ctypes.byref(num_out))
    assert rc == 0
    return index, int(num_index.value), out_coors, int(num_out.value), oshape


def spconv_mm(in_feats, weight, bias, index, num_index, inverse, max_num_act_out):
    """fp32 gather-GEMM-scatter; weight [kVol, Cin, Cout]; returns [max_out, Cout] float32."""
    in_feats, weight = _f32(in_feats), _f32(weight)
    index = _i32(index)
    kvol, cin, cout = weight.shape
    out = np.empty((max_num_act_out, cout), dtype=np.float32)
    b = None if bias is None else _f32(bias)
    lib().orc_spconv_mm(_p(in_feats, _f32p), _p(weight, _f32p), None if b is None else _p(b, _f32p),
                        _p(index, _i32p), ctypes.c_int64(index.shape[1]), ctypes.c_int32(num_index),
                        int(bool(inverse)), cin, cout, _p(out, _f32p), ctypes.c_int64(max_num_act_out))
    return out


def bev_densify(feats, coors, num_act_in, spatial_shape):
    """spatial_shape = [B, 0, Z, Y, X]; returns [B, C*Z, Y, X] float32."""
    feats, coors = _f32(feats), _i32(coors)
    b, _, z, y, x = [int(v) for v in spatial_shape]
    c = feats.shape[1]
    out = np.empty((b, c * z, y, x), dtype=np.float32)
    lib().orc_bev_densify(_p(feats, _f32p), _p(coors, _i32p), ctypes.c_int32(num_act_in), c, ctypes.c_int64(b),
                          ctypes.c_int64(z), ctypes.c_int64(y), ctypes.c_int64(x), _p(out, _f32p))
    return out


def simple_mean(pts, batch, voxel_config, spatial_shape, max_num_act_out):
    """spatial_shape = [B, 0, Z, Y, X]; returns (feats, coors, num_act_out)."""
    pts, batch, cfg = _f32(pts), _i32(batch), _f32(voxel_config)
    n, c = pts.shape
    shp = np.array([spatial_shape[0], spatial_shape[2], spatial_shape[3], spatial_shape[4]], dtype=np.int64)
    feats = np.zeros((max_num_act_out, c), dtype=np.float32)
    coors = np.zeros((max_num_act_out, 4), dtype=np.int32)
    num = ctypes.c_int32(0)
    lib().orc_simple_mean(_p(pts, _f32p), _p(batch, _i32p), ctypes.c_int64(n), c, _p(cfg, _f32p), _p(shp, _i64p),
                          ctypes.c_int64(max_num_act_out), _p(feats, _f32p), _p(coors, _i32p), ctypes.byref(num))
    return feats, coors, int(num.value)


def cylinder(pts, batch, cylinder_config, spatial_shape, max_num_act_out):
    """spatial_shape = [B, 0, RHO, PHI, Z]; returns (aug, scatter_to, scatter_count, coors, num_act_out)."""
    pts, batch, cfg = _f32(pts), _i32(batch), _f32(cylinder_config)
    n, c = pts.shape
    shp = np.array([spatial_shape[0], spatial_shape[2], spatial_shape[3], spatial_shape[4]], dtype=np.int64)
    aug = np.zeros((n, c + 5), dtype=np.float32)
    scatter_to = np.zeros(n, dtype=np.int32)
    scatter_count = np.zeros(max_num_act_out, dtype=np.int32)
    coors = np.zeros((max_num_act_out, 4), dtype=np.int32)
    num = ctypes.c_int32(0)
    lib().orc_cylinder(_p(pts, _f32p), _p(batch, _i32p), ctypes.c_int64(n), c, _p(cfg, _f32p), _p(shp, _i64p),
                       ctypes.c_int64(max_num_act_out), _p(aug, _f32p), _p(scatter_to, _i32p),
                       _p(scatter_count, _i32p), _p(coors, _i32p), ctypes.byref(num))
    return aug, scatter_to, scatter_count, coors, int(num.value)


def scatter_to(in_feats, scatter_index, scatter_count, reduce_type):
    in_feats, scatter_index, scatter_count = _f32(in_feats), _i32(scatter_index), _i32(scatter_count)
    n, c = in_feats.shape
    m = scatter_count.shape[0]
    out = np.empty((m, c), dtype=np.float32)
    lib().orc_scatter_to(_p(in_feats, _f32p), _p(scatter_index, _i32p), _p(scatter_count, _i32p), ctypes.c_int64(n),
                         c, ctypes.c_int64(m), int(reduce_type), _p(out, _f32p))
    return out


def gather_back(in_feats, scatter_index, fill_val=None, out_init=None):
    """Rows with a negative index keep ``out_init`` unless ``fill_val`` is given."""
    in_feats, scatter_index = _f32(in_feats), _i32(scatter_index)
    n = scatter_index.shape[0]
    c = int(np.prod(in_feats.shape[1:])) if in_feats.ndim > 1 else 1
    shape = (n,) + tuple(in_feats.shape[1:])
    out = np.zeros(shape, dtype=np.float32) if out_init is None else _f32(out_init).copy()
    lib().orc_gather_back(_p(in_feats, _f32p), _p(scatter_index, _i32p), ctypes.c_int64(n), ctypes.c_int64(c),
                          int(fill_val is not None), ctypes.c_float(0.0 if fill_val is None else fill_val),
                          _p(out, _f32p))
    return out


def nms3d(scores, boxes, thr=0.1):
    scores, boxes = _f32(scores), _f32(boxes)
    b, k = scores.shape
    out = np.empty_like(scores)
    lib().orc_nms3d(_p(scores, _f32p), _p(boxes, _f32p), b, k, boxes.shape[2], ctypes.c_float(thr), _p(out, _f32p))
    return out


def yolox3d_decode(cls_scores, bbox_preds, voxel_config, stride, class_ids, topk):
    """Restatement of the reference's YoloX3dDecode in numpy (trt/decoder/yolox3d_decode.cu): per (batch, class) a
    stable descending sort of the Y*X scores (:341-355; equal scores keep ascending cell order), the first
    K = min(topk, Y*X) entries (:192-206) decoded by `kernel::decode` (:25-126) with its float / double mix:
    float arithmetic, M_PI terms in double, floorf on the value rounded to float.  Pinned on a B200 against the
    reference's own plugin compiled for sm_100a (tests/test_gpu_reference.py).
    Returns [(class_ids int32 [B,K], scores float32 [B,K], boxes float32 [B,K,7+a])] per class."""
    f32, f64 = np.float32, np.float64
    s = np.asarray(cls_scores).astype(f32)
    p = np.asarray(bbox_preds).astype(f32)
    cfg = _f32(voxel_config)
    b, c, ny, nx = s.shape
    n = ny * nx
    k = min(int(topk), n)
    extra = p.shape[1] - 9
    feat_stride = f32(f32(stride) * cfg[3])
    out = []
    with np.errstate(all="ignore"):
        for ci in range(c):
            ids = np.full((b, k), class_ids[ci], dtype=np.int32)
            sc = np.empty((b, k), dtype=f32)
            bx = np.empty((b, k, 7 + extra), dtype=f32)
            for bi in range(b):
                flat = s[bi, ci].reshape(-1)
                key = np.where(flat == 0, f32(0), flat)  # the sort treats -0 and +0 alike
                order = np.argsort(-key.astype(f64), kind="stable")[:k]
                pr = p[bi].reshape(9 + extra, n)[:, order]
                score = flat[order].copy()
                cx = (pr[0] + (order % nx).astype(f32)).astype(f32)
                cx_valid = (cx <= f32(nx)) & (cx >= 0)
                cx = (cfg[0] + feat_stride * cx).astype(f32)
                cy = (pr[1] + (order // nx).astype(f32)).astype(f32)
                cy_valid = (cy <= f32(ny)) & (cy >= 0)
                cy = (cfg[1] + feat_stride * cy).astype(f32)
                cz = pr[2].copy()
                dx = (feat_stride * np.exp(pr[3])).astype(f32)
                dy = (feat_stride * np.exp(pr[4])).astype(f32)
                dz = np.exp(pr[5]).astype(f32)
                yaw = pr[6].copy()
                ds, dc = pr[7], pr[8]
                direction = np.arctan2(ds, dc).astype(f32)
                ok = (np.isfinite(cx) & np.isfinite(cy) & np.isfinite(cz) & np.isfinite(dx) & np.isfinite(dy) &
                      np.isfinite(dz) & np.isfinite(yaw) & (dx > 0) & (dy > 0) & (dz > 0) & ((ds != 0) | (dc != 0)) &
                      cx_valid & cy_valid)
                square = ok & (f32(0.9) * dx < dy) & (dy < f32(1.11) * dx)
                longish = ok & ~square
                # elongated boxes: make dx the long side, then move yaw into the half-plane of the direction head
                swap = longish & (dy > dx)
                yaw_l = np.where(swap, (yaw.astype(f64) + np.pi / 2).astype(f32), yaw)
                dx_l, dy_l = np.where(swap, dy, dx), np.where(swap, dx, dy)
                q = ((direction - yaw_l).astype(f32).astype(f64) / np.pi + 0.5).astype(f32)
                yaw_l = (yaw_l.astype(f64) + np.floor(q).astype(f64) * np.pi).astype(f32)
                q = (yaw_l.astype(f64) / (2 * np.pi) + 0.5).astype(f32)
                yaw_l = (yaw_l.astype(f64) - np.floor(q).astype(f64) * (2 * np.pi)).astype(f32)
                big = np.maximum(dx, dy)
                sc[bi] = np.where(ok, score, f32(-1))
                bx[bi, :, 0] = np.where(ok, cx, f32(10000))
                bx[bi, :, 1] = np.where(ok, cy, f32(10000))
                bx[bi, :, 2] = np.where(ok, cz, f32(10000))
                bx[bi, :, 3] = np.where(square, big, np.where(longish, dx_l, f32(1)))
                bx[bi, :, 4] = np.where(square, big, np.where(longish, dy_l, f32(1)))
                bx[bi, :, 5] = np.where(ok, dz, f32(1))
                bx[bi, :, 6] = np.where(square, direction, np.where(longish, yaw_l, f32(0)))
                for e in range(extra):
                    bx[bi, :, 7 + e] = pr[9 + e]
            out.append((ids, sc, bx))
    return out


def bev_iou(a, b):
    a, b = _f32(a), _f32(b)
    return float(lib().orc_bev_iou(_p(a, _f32p), _p(b, _f32p)))


# ------------------------------------------------------------------------------------------
# Canonicalisation (what "bit-exact" means where the reference's voxel order is arbitrary;
# mirrors the comparison in the reference's tests/spconv/test_spconv.py:72-124).
# ------------------------------------------------------------------------------------------

def lex_order(coors):
    """Permutation that sorts coordinate rows lexicographically."""
    coors = np.asarray(coors)
    keys = tuple(coors[:, c] for c in range(coors.shape[1] - 1, -1, -1))
    return np.lexsort(keys)


def check_layout(index, num_index, kvol):
    """Structural invariants of the index tensor (test_spconv.py:82-91, trt/spconv/index.cu:123-156).

    Returns the list of (k, start, count) segments."""
    index = np.asarray(index)
    gather, scatter, koff = index
    assert num_index % 128 == 0
    assert num_index <= index.shape[1]
    assert (index[:, num_index:] == -1).all(), "tail beyond numIndex must be -1"
    pad = koff[:num_index] < 0
    assert (gather[:num_index][pad] == -1).all() and (scatter[:num_index][pad] == -1).all()
    assert (gather[:num_index][~pad] >= 0).all() and (scatter[:num_index][~pad] >= 0).all()
    segs, pos = [], 0
    for k in range(kvol):
        cnt = int((koff[:num_index] == k).sum())
        if cnt:
            assert pos % 128 == 0
            assert (koff[pos:pos + cnt] == k).all(), "segment of offset %d is not contiguous at %d" % (k, pos)
            g = gather[pos:pos + cnt]
            assert (np.diff(g) > 0).all(), "entries must ascend by input index inside a segment"
            end = (pos + cnt + 127) // 128 * 128
            assert (koff[pos + cnt:end] == -1).all()
            segs.append((k, pos, cnt))
            pos = end
    assert pos == num_index
    return segs


def canonical_pairs(index, num_index, kvol, out_perm=None):
    """Dict k -> int64 array [cnt, 2] of (gather, scatter) sorted by (gather, scatter).

    ``out_perm[old_id] = canonical_id`` renames output voxels first (forward rulebooks)."""
    gather, scatter, koff = np.asarray(index)
    res = {}
    for k in range(kvol):
        m = koff[:num_index] == k
        g = gather[:num_index][m].astype(np.int64)
        s = scatter[:num_index][m].astype(np.int64)
        if out_perm is not None:
            s = np.asarray(out_perm)[s]
        o = np.lexsort((s, g))
        res[k] = np.stack([g[o], s[o]], axis=1)
    return res


def canonical_conv(index, num_index, out_coors, num_out, kvol):
    """Canonical form of a strided/transposed rulebook: (sorted coords, pairs dict)."""
    oc = np.asarray(out_coors)[:num_out]
    order = lex_order(oc)
    perm = np.empty(num_out, dtype=np.int64)
    perm[order] = np.arange(num_out)
    return oc[order], canonical_pairs(index, num_index, kvol, perm), order


# ------------------------------------------------------------------------------------------
# Brute-force model of the rulebook (dictionary of coordinates, no hashing, no layout).
# ------------------------------------------------------------------------------------------

def brute_rulebook(coors, in_shape, ksize, stride, pad, dil, out_pad, transpose, subm):
    """Returns (sorted unique out coords [M, ndim+1], {k: [(i, out_id)]}) with out ids in lexicographic order."""
    coors = np.asarray(coors, dtype=np.int64)
    ndim = coors.shape[1] - 1
    oshape = list(in_shape) if subm else out_shape(in_shape, ksize, stride, pad, dil, out_pad, transpose)
    kvol = kernel_volume(ksize)
    pairs = []
    for i, c in enumerate(coors):
        for k in range(kvol):
            rem, o, ok = k, [int(c[0])], True
            ks = []
            for d in range(ndim - 1, -1, -1):
                ks.append(rem % ksize[d])
                rem //= ksize[d]
            ks = ks[::-1]
            for d in range(ndim):
                if transpose:
                    v = int(c[d + 1]) * stride[d] - pad[d] + ks[d] * dil[d]
                else:
                    v = int(c[d + 1]) + pad[d] - ks[d] * dil[d]
                    if v % stride[d] != 0:
                        ok = False
                        break
                    v //= stride[d]
                if v < 0 or v >= oshape[d + 1]:
                    ok = False
                    break
                o.append(v)
            if ok:
                pairs.append((k, i, tuple(o)))
    if subm:
        ids = {tuple(int(v) for v in c): i for i, c in enumerate(coors)}
        outc = coors
        pairs = [(k, i, o) for (k, i, o) in pairs if o in ids]
    else:
        uniq = sorted({o for (_, _, o) in pairs})
        ids = {o: j for j, o in enumerate(uniq)}
        outc = np.array(uniq, dtype=np.int64).reshape(-1, ndim + 1)
    res = {k: [] for k in range(kvol)}
    for k, i, o in pairs:
        res[k].append((i, ids[o]))
    res = {k: np.array(sorted(v), dtype=np.int64).reshape(-1, 2) for k, v in res.items()}
    return outc, res
