"""The reference's own GPU code as the yardstick: trt/spconv/index.cu and trt/spconv/mm.h compiled for sm_100a
(oracle/_ref/libref_spconv.so, built by `make -C oracle ref_spconv`) run on the same inputs as the product library and
the CPU oracle.

* SubM rulebooks are deterministic in the reference (gather = input id, scatter = hash value = neighbour id, segments
  in offset order): reference == oracle == product byte for byte, padding included.
* Strided / transposed rulebooks number the outputs by hash-slot rank, which depends on the insertion race:
  compared after the canonicalisation the reference's own test performs (tests/spconv/test_spconv.py:72-124).
* Features: the reference accumulates with half-precision atomic adds in arbitrary order, so it is compared with
  the tolerance of its own test (rtol 1e-2, atol 1e-1, test_spconv.py:152-161) and a relative L2 bound."""
import numpy as np
import pytest
import torch

from tests._util import pairs_equal, rng, unique_coors
from tests.test_gpu_spconv import _t, check_index, run_index

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ref():
    from oracle import ref_gpu
    if ref_gpu.lib() is None:
        pytest.skip("oracle/_ref/libref_spconv.so was not built (no reference checkout on the build machine)")
    return ref_gpu


CASES = [
    # name, ks, st, pd, dl, op, tr, subm, shape_b, n, n_max, max_out
    ("subm", (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), False, True, [2, 120, 90, 8], 20000, 20000, 20000),
    ("subm_padded_buffer", (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), False, True, [2, 120, 90, 8], 20000,
     40000, 40000),
    ("subm_dilated", (3, 3, 3), (1, 1, 1), (2, 2, 2), (2, 2, 2), (0, 0, 0), False, True, [1, 30, 30, 12], 5000, 5077,
     5077),
    ("subm_3x1x3", (3, 1, 3), (1, 1, 1), (1, 0, 1), (1, 1, 1), (0, 0, 0), False, True, [2, 48, 36, 16], 9000, 9077,
     9077),
    ("subm_5x5x5", (5, 5, 5), (1, 1, 1), (2, 2, 2), (1, 1, 1), (0, 0, 0), False, True, [1, 14, 14, 14], 1200, 1277,
     1277),
    ("strided_221", (3, 3, 3), (2, 2, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), False, False, [2, 120, 90, 8], 20000, 20000,
     50000),
    ("strided_221_truncated", (3, 3, 3), (2, 2, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), False, False, [2, 120, 90, 8],
     20000, 40000, 5000),
    ("strided_222_pad011", (3, 3, 3), (2, 2, 2), (0, 1, 1), (1, 1, 1), (0, 0, 0), False, False, [2, 11, 60, 50], 7000,
     7077, 200000),
    ("strided_3x1x1", (3, 1, 1), (2, 1, 1), (0, 0, 0), (1, 1, 1), (0, 0, 0), False, False, [2, 5, 60, 50], 6000, 6077,
     200000),
    ("transposed_222", (3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1), (1, 1, 1), True, False, [2, 20, 24, 10], 3000, 3077,
     200000),
    ("transposed_k2", (2, 2, 2), (2, 2, 2), (0, 0, 0), (1, 1, 1), (0, 0, 0), True, False, [1, 16, 16, 16], 1000, 1077,
     200000),
]


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_rulebook_matches_reference_gpu(d3d, orc, ref, case):
    name, ks, st, pd, dl, op, tr, subm, shape_b, n, n_max, max_out = case
    r = rng(7000 + sum(map(ord, name)))
    coors = unique_coors(r, n, shape_b)
    kvol = int(np.prod(ks))
    out_shape_b = shape_b if subm else orc.out_shape(shape_b, ks, st, pd, dl, op, tr)
    r_index, r_num, r_coors, r_nout = ref.spconv_index(_t(coors), n_max, out_shape_b, ks, st, pd, dl, max_out, subm,
                                                       tr)
    ref_outs = [r_index, r_num] if subm else [r_index, r_num, r_coors, r_nout]
    # 1. the reference against the CPU oracle (pins the oracle)
    check_index(orc, ref_outs, coors, n_max, shape_b, ks, st, pd, dl, op, max_out, subm, tr)
    # 2. the product against the reference, directly
    spatial = [shape_b[0], 0] + shape_b[1:]
    outs, _ = run_index(d3d, coors, n_max, spatial, ks, st, pd, dl, op, max_out, subm, tr)
    got_num, ref_num = int(outs[1].item()), int(r_num.item())
    if subm:
        assert got_num == ref_num
        assert torch.equal(outs[0], r_index), "SubM rulebook differs from the reference's byte for byte"
        return
    ref_nout, got_nout = int(r_nout.item()), int(outs[3].item())
    assert got_nout == ref_nout
    assert list(outs[4].shape) == [out_shape_b[0], 0] + list(out_shape_b[1:])
    # when maxNumActOut truncates, WHICH outputs survive is the reference's hash-slot order (implementation defined):
    # both sides were checked against the oracle's rules for the kept subset above and in test_gpu_spconv.py
    if ref_nout < max_out:  # nothing truncated: same output set, same pairs
        assert got_num == ref_num
        gc, gp, _ = orc.canonical_conv(outs[0].cpu().numpy(), got_num, outs[2].cpu().numpy(), got_nout, kvol)
        rc, rp, _ = orc.canonical_conv(r_index.cpu().numpy(), ref_num, r_coors.cpu().numpy(), ref_nout, kvol)
        assert (gc == rc).all(), "output coordinate sets differ from the reference's"
        pairs_equal(gp, rp, kvol)


def _features(r, n_rows, cin, cout, kvol):
    feats = r.standard_normal((n_rows, cin)).astype(np.float32)
    w = (r.standard_normal((kvol, cin, cout)) * np.sqrt(2.0 / (kvol * cin))).astype(np.float32)
    b = r.standard_normal(cout).astype(np.float32)
    return feats, w, b


@pytest.mark.parametrize("cin,cout", [(16, 32), (32, 32), (64, 64), (128, 128), (16, 24)])
@pytest.mark.parametrize("kind", ["subm", "strided", "inverse"])
def test_features_match_reference_gpu(d3d, orc, ref, kind, cin, cout):
    if not ref.lib().has_mm:
        pytest.skip("the reference convolution was not built (no CUTLASS header tree on the build machine)")
    r = rng(8000 + cin * 7 + cout + len(kind))
    shape_b, spatial, n = [2, 120, 90, 8], [2, 0, 120, 90, 8], 20000
    coors = unique_coors(r, n, shape_b)
    ks, pd, dl, op = (3, 3, 3), (1, 1, 1), (1, 1, 1), (0, 0, 0)
    subm = kind == "subm"
    st = (1, 1, 1) if subm else (2, 2, 1)
    max_out = n if subm else 50000
    outs, num_in = run_index(d3d, coors, n, spatial, ks, st, pd, dl, op, max_out, subm, False)
    num_out = num_in if subm else outs[3]
    inverse = kind == "inverse"
    n_in_rows, n_out_rows, a, b_ = (max_out, n, num_out, num_in) if inverse else (n, max_out, num_in, num_out)
    feats, w, b = _features(r, n_in_rows, cin, cout, 27)
    feats_t = _t(feats, torch.float16)
    got = d3d.spconv_mm(feats_t, a, b_, outs[0], outs[1], ks, cin, cout, n_out_rows, False, inverse, w, b)
    want = ref.spconv_mm(feats_t, _t(w, torch.float16), _t(b, torch.float16), outs[0], outs[1], inverse, n_out_rows)
    torch.cuda.synchronize()
    got, want = got.float().cpu().numpy(), want.float().cpu().numpy()
    assert got.shape == want.shape
    assert np.allclose(got, want, rtol=1e-2, atol=1e-1), "worst |diff| %.3e" % np.abs(got - want).max()
    rel_l2 = np.sqrt(((got - want) ** 2).sum() / (want ** 2).sum())
    assert rel_l2 < 5e-3, "relative L2 distance to the reference %.3e" % rel_l2
    # and the reference itself sits inside the oracle's tolerance band around the fp32-accumulated result
    exact = orc.spconv_mm(feats_t.float().cpu().numpy(), _t(w, torch.float16).float().cpu().numpy(),
                          _t(b, torch.float16).float().cpu().numpy(), outs[0].cpu().numpy(), int(outs[1].item()),
                          inverse, n_out_rows)
    assert np.allclose(want, exact, rtol=1e-2, atol=1e-1)
    # one rounding of an fp32 accumulator is no further from it than a chain of half-precision atomic adds
    assert np.sqrt(((got - exact) ** 2).sum()) <= 1.05 * np.sqrt(((want - exact) ** 2).sum()) + 1e-6
