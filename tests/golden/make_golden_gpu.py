"""Generates tests/golden/spconv_ref_gpu.npz: rulebooks and convolution outputs computed by the REFERENCE's own GPU
code (trt/spconv/index.cu, trt/spconv/mm.h compiled for sm_100a into oracle/_ref/libref_spconv.so by
`make -C oracle ref_spconv`).  Needs a CUDA device; the library is built where the reference checkout exists and
travels as a build product, so this script reads no reference source.

Usage (on a machine with a GPU):  python tests/golden/make_golden_gpu.py [output.npz]

Contents, for every case `c`: `c_coors` (input voxels), `c_params` (ks, st, pd, dl, op as 5 x 3, then transpose,
subm, n_max, max_out), `c_shape`; SubM: `c_index` (the [3, L] tensor as written by the reference, padding
included), `c_num`; strided / transposed: `c_out_coors` (sorted lexicographically), `c_num`, and the canonical
pair list `c_pairs` [P, 3] = (offset, gather, renamed scatter) sorted, which is what survives the reference's
race-dependent output numbering.  Convolution: `mm_*` = fp16 inputs and the reference's fp16 output for one SubM
and one strided rulebook (16 -> 32 channels, the shape of the reference's own test)."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

CASES = {
    # name: ks, st, pd, dl, op, transpose, subm, shape_b, n, n_max, max_out
    "subm": ((3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), False, True, [2, 24, 20, 8], 1500, 1500, 1500),
    "subm_pad": ((3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), False, True, [2, 24, 20, 8], 1500, 1700, 1700),
    "subm_dil": ((3, 3, 3), (1, 1, 1), (2, 2, 2), (2, 2, 2), (0, 0, 0), False, True, [1, 16, 16, 12], 900, 900, 900),
    "subm_313": ((3, 1, 3), (1, 1, 1), (1, 0, 1), (1, 1, 1), (0, 0, 0), False, True, [2, 24, 20, 8], 1500, 1500, 1500),
    "down221": ((3, 3, 3), (2, 2, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), False, False, [2, 24, 20, 8], 1500, 1500, 2500),
    "down222": ((3, 3, 3), (2, 2, 2), (0, 1, 1), (1, 1, 1), (0, 0, 0), False, False, [2, 11, 20, 18], 1200, 1300,
                1500),
    "down_k2": ((2, 2, 2), (2, 2, 2), (0, 0, 0), (1, 1, 1), (0, 0, 0), False, False, [1, 16, 16, 16], 1000, 1000,
                1000),
    "up222": ((3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1), (1, 1, 1), True, False, [2, 10, 12, 6], 600, 600, 12000),
}


def main():
    import torch
    from oracle import oracle, ref_gpu
    from tests._util import rng, unique_coors
    assert ref_gpu.lib() is not None and ref_gpu.lib().has_mm, "oracle/_ref/libref_spconv.so missing"
    out = {}
    for ci, (name, (ks, st, pd, dl, op, tr, subm, shape_b, n, n_max, max_out)) in enumerate(CASES.items()):
        r = rng(9100 + ci)
        coors = unique_coors(r, n, shape_b)
        kvol = int(np.prod(ks))
        oshape = shape_b if subm else oracle.out_shape(shape_b, ks, st, pd, dl, op, tr)
        index, num, out_coors, nout = ref_gpu.spconv_index(torch.from_numpy(coors).cuda(), n_max, oshape, ks, st, pd,
                                                           dl, max_out, subm, tr)
        out[name + "_coors"] = coors
        out[name + "_params"] = np.array(list(ks) + list(st) + list(pd) + list(dl) + list(op) +
                                         [int(tr), int(subm), n_max, max_out], np.int64)
        out[name + "_shape"] = np.array(shape_b, np.int64)
        out[name + "_num"] = np.int64(num.item())
        index = index.cpu().numpy()
        if subm:
            out[name + "_index"] = index
        else:
            k = int(nout.item())
            assert k <= max_out and k < int(np.prod(oshape)) + 1
            oc, pairs, _ = oracle.canonical_conv(index, int(num.item()), out_coors.cpu().numpy(), k, kvol)
            out[name + "_out_coors"] = oc
            rows = [np.concatenate([np.full((len(pairs[kk]), 1), kk, np.int64), pairs[kk]], 1) for kk in range(kvol)]
            out[name + "_pairs"] = np.concatenate(rows).astype(np.int32)
        if name in ("subm", "down221"):  # convolution on this rulebook, forward and (strided) inverse
            idx_t, num_t = torch.from_numpy(index).cuda(), num
            n_out_rows = n_max if subm else max_out
            for inverse in ([False] if subm else [False, True]):
                rows_in, rows_out = (n_out_rows, n_max) if inverse else (n_max, n_out_rows)
                feats = torch.from_numpy(r.standard_normal((rows_in, 16)).astype(np.float32)).cuda().half()
                w = torch.from_numpy((r.standard_normal((kvol, 16, 32)) * np.sqrt(2.0 / (kvol * 16))).astype(
                    np.float32)).cuda().half()
                b = torch.from_numpy(r.standard_normal(32).astype(np.float32)).cuda().half()
                y = ref_gpu.spconv_mm(feats, w, b, idx_t, num_t, inverse, rows_out)
                tag = "mm_%s%s" % (name, "_inv" if inverse else "")
                out[tag + "_feats"], out[tag + "_w"], out[tag + "_b"] = (t.cpu().numpy() for t in (feats, w, b))
                out[tag + "_out"] = y.cpu().numpy()
                if not subm:
                    out[tag + "_index"] = index  # the reference's own numbering, needed to replay its output rows
    path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "spconv_ref_gpu.npz")
    np.savez_compressed(path, **out)
    print("wrote %s (%d arrays, %.0f KB)" % (path, len(out), os.path.getsize(path) / 1024))


if __name__ == "__main__":
    main()
