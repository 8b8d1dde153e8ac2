"""Generates the committed golden vectors under tests/golden/ (run here, where the reference checkout exists):

  iou_ref.npz      seeded box pairs and the intersection area / BEV IoU computed by the REFERENCE's own
                   trt/decoder/iou_rotated.cuh compiled for the host (oracle/_ref/libref_iou.so, built by
                   `make -C oracle ref`).  Pins oracle.c's restatement of the rotated-IoU arithmetic.
  nms_ref.npz      seeded NMS cases; keep-masks computed with the greedy rule of trt/decoder/nms3d.cu:106-127
                   over the reference IoU above, thresholds 0.1 (the plugin's constant) and 0.2.
  rulebook_small.npz  a small strided / transposed / SubM rulebook from the oracle, checked against the brute-force
                   dictionary model at generation time (regression anchor for the index layout).

Usage: python tests/golden/make_golden.py
"""
import ctypes
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle  # noqa: E402


def boxes(rng, n, spread):
    xyz = rng.standard_normal((n, 3)) * spread
    dims = rng.uniform(0.5, 1.5, (n, 3))
    yaw = rng.uniform(-np.pi, np.pi, (n, 1))
    return np.concatenate([xyz, dims, yaw], 1).astype(np.float32)


def main():
    oracle.build()
    ref = oracle.ref_iou_lib()
    assert ref is not None, "oracle/_ref/libref_iou.so missing: run `make -C oracle ref` with the reference present"
    f32p = ctypes.POINTER(ctypes.c_float)
    rng = np.random.Generator(np.random.PCG64(20240))
    a = np.concatenate([boxes(rng, 1500, 1.0), boxes(rng, 500, 0.2)])
    b = np.concatenate([boxes(rng, 1500, 1.0), boxes(rng, 500, 0.2)])
    # degenerate / axis-aligned / identical / touching cases
    extra_a = np.array([[0, 0, 0, 1, 1, 1, 0], [0, 0, 0, 2, 1, 1, 0], [0, 0, 0, 1, 1, 1, 0], [0, 0, 0, 1, 1, 1, 0.3],
                        [0, 0, 0, 1, 2, 1, np.pi / 2], [5, 5, 0, 1, 1, 1, 1.0]], np.float32)
    extra_b = np.array([[0, 0, 0, 1, 1, 1, 0], [1, 0, 0, 2, 1, 1, 0], [1, 0, 0, 1, 1, 1, 0], [0, 0, 0, 1, 1, 1, 0.3],
                        [0, 0, 0, 2, 1, 1, 0], [-5, -5, 0, 1, 1, 1, 2.0]], np.float32)
    a, b = np.concatenate([a, extra_a]), np.concatenate([b, extra_b])
    inter = np.empty(len(a), np.float32)
    iou = np.empty(len(a), np.float32)
    for i in range(len(a)):
        inter[i] = ref.ref_rotated_intersection(*[float(v) for v in a[i, [0, 1, 3, 4, 6]]],
                                                *[float(v) for v in b[i, [0, 1, 3, 4, 6]]])
        iou[i] = ref.ref_bev_iou(a[i].ctypes.data_as(f32p), b[i].ctypes.data_as(f32p))
    np.savez_compressed(os.path.join(HERE, "iou_ref.npz"), a=a, b=b, inter=inter, iou=iou)

    cases = {}
    for name, (nb, k, spread) in {"b1k128": (1, 128, 1.0), "b2k256": (2, 256, 1.0), "b3k200": (3, 200, 3.0)}.items():
        bx = np.stack([boxes(rng, k, spread) for _ in range(nb)])
        sc = np.tile(1 - np.arange(k, dtype=np.float32) / k, (nb, 1))
        cases[name + "_boxes"], cases[name + "_scores"] = bx, sc
        for thr in (0.1, 0.2):
            keep = np.ones((nb, k), bool)
            for bi in range(nb):
                for i in range(k):
                    if not keep[bi, i]:
                        continue
                    for j in range(i + 1, k):
                        if keep[bi, j] and ref.ref_bev_iou(bx[bi, i].ctypes.data_as(f32p),
                                                           bx[bi, j].ctypes.data_as(f32p)) >= np.float32(thr):
                            keep[bi, j] = False
            cases["%s_keep_%02d" % (name, int(thr * 10))] = keep
    np.savez_compressed(os.path.join(HERE, "nms_ref.npz"), **cases)

    rb = {}
    coors = np.unique(np.stack([rng.integers(0, 2, 400), rng.integers(0, 9, 400), rng.integers(0, 12, 400),
                                rng.integers(0, 10, 400)], 1).astype(np.int32), axis=0)
    coors = coors[rng.permutation(len(coors))]
    shape = [2, 9, 12, 10]
    rb["coors"], rb["shape"] = coors, np.array(shape)
    for name, (ks, st, pd, dl, op, tr, subm) in {
            "subm": ((3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), False, True),
            "down": ((3, 3, 3), (2, 2, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), False, False),
            "up": ((3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1), (1, 1, 1), True, False)}.items():
        kvol = 27
        if subm:
            index, num = oracle.rulebook_subm(coors, shape, ks, st, pd, dl)
            oc, pairs = coors, oracle.canonical_pairs(index, num, kvol)
        else:
            index, num, oc, nout, oshape = oracle.rulebook_conv(coors, shape, ks, st, pd, dl, op, tr, 100000)
            oc, pairs, _ = oracle.canonical_conv(index, num, oc, nout, kvol)
        bc, bp = oracle.brute_rulebook(coors, shape, ks, st, pd, dl, op, tr, subm)
        assert (np.asarray(bc) == oc).all()
        for k in range(kvol):
            assert (bp[k] == pairs[k]).all()
        oracle.check_layout(index, num, kvol)
        rb[name + "_index"] = index[:, :num]
        rb[name + "_out_coors"] = oc
    np.savez_compressed(os.path.join(HERE, "rulebook_small.npz"), **rb)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
