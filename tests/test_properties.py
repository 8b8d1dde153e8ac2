"""Property-based parity on small random grids (hypothesis, derandomised so that every run sees the same examples):
the CPU oracle against the brute-force dictionary model of the rulebook, and -- on the GPU -- the product library
against the oracle, over kernel sizes 1-3, strides 1-3, dilations 1-2, paddings 0-2, transposed and SubM, grids of
ragged extents and voxel counts from 0 upwards."""
import numpy as np
import pytest
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from tests._util import pairs_equal, rng, unique_coors


@st.composite
def geometries(draw):
    subm = draw(st.booleans())
    transpose = (not subm) and draw(st.booleans())
    ks = tuple(draw(st.integers(1, 3)) for _ in range(3))
    stride = (1, 1, 1) if subm else tuple(draw(st.integers(1, 3)) for _ in range(3))
    dil = tuple(draw(st.integers(1, 2)) for _ in range(3))
    pad = tuple(draw(st.integers(0, 2)) for _ in range(3))
    out_pad = tuple(draw(st.integers(0, s - 1)) for s in stride) if transpose else (0, 0, 0)
    shape = [draw(st.integers(1, 2))] + [draw(st.integers(3, 11)) for _ in range(3)]
    if not transpose:  # the forward output extent must be at least 1
        for d in range(3):
            while shape[d + 1] + 2 * pad[d] - dil[d] * (ks[d] - 1) - 1 < 0:
                shape[d + 1] += 1
    total = int(np.prod(shape))
    n = draw(st.integers(0, min(total, 260)))
    seed = draw(st.integers(0, 10 ** 6))
    return dict(subm=subm, transpose=transpose, ks=ks, stride=stride, dil=dil, pad=pad, out_pad=out_pad, shape=shape,
                n=n, seed=seed)


COMMON = dict(derandomize=True, deadline=None, suppress_health_check=[HealthCheck.function_scoped_fixture,
                                                                       HealthCheck.too_slow])


@settings(max_examples=60, **COMMON)
@given(geo=geometries())
def test_oracle_rulebook_equals_brute_force(orc, geo):
    coors = unique_coors(rng(geo["seed"]), geo["n"], geo["shape"])
    kvol = int(np.prod(geo["ks"]))
    args = (geo["ks"], geo["stride"], geo["pad"], geo["dil"])
    bc, bp = orc.brute_rulebook(coors, geo["shape"], *args, geo["out_pad"], geo["transpose"], geo["subm"])
    if geo["subm"]:
        index, num = orc.rulebook_subm(coors, geo["shape"], *args, max_num_act_in=geo["n"] + 5)
        orc.check_layout(index, num, kvol)
        pairs_equal(orc.canonical_pairs(index, num, kvol), bp, kvol)
    else:
        index, num, oc, nout, _ = orc.rulebook_conv(coors, geo["shape"], *args, geo["out_pad"], geo["transpose"],
                                                     100000, max_num_act_in=geo["n"] + 5)
        orc.check_layout(index, num, kvol)
        cc, pairs, _ = orc.canonical_conv(index, num, oc, nout, kvol)
        assert nout == len(bc) and (cc.reshape(-1, 4) == np.asarray(bc).reshape(-1, 4)).all()
        pairs_equal(pairs, bp, kvol)


@pytest.mark.gpu
@settings(max_examples=40, **COMMON)
@given(geo=geometries())
def test_product_rulebook_and_features_equal_oracle(d3d, orc, geo):
    from tests.test_gpu_spconv import check_index, run_index, run_mm
    coors = unique_coors(rng(geo["seed"]), geo["n"], geo["shape"])
    n_max = geo["n"] + 5
    spatial = [geo["shape"][0], 0] + geo["shape"][1:]
    max_out = n_max if geo["subm"] else 40000
    args = (geo["ks"], geo["stride"], geo["pad"], geo["dil"], geo["out_pad"])
    outs, num_in = run_index(d3d, coors, n_max, spatial, *args, max_out, geo["subm"], geo["transpose"])
    nout = check_index(orc, outs, coors, n_max, geo["shape"], *args, max_out, geo["subm"], geo["transpose"])
    num_out = num_in if geo["subm"] else outs[3]
    run_mm(d3d, orc, outs[0], outs[1], num_in, num_out, n_max, max_out, 8, 16, geo["ks"], False, "fp32",
           geo["seed"] % 97, 1e-4, geo["n"] if geo["subm"] else nout)


@pytest.mark.gpu
@settings(max_examples=30, **COMMON)
@given(geo=geometries())
def test_product_rulebook_equals_reference_gpu(d3d, orc, geo):
    """The same random geometries against the reference's own rulebook builders (trt/spconv/index.cu compiled for
    sm_100a): SubM byte for byte, strided / transposed after canonicalisation."""
    import torch
    from oracle import ref_gpu
    from tests.test_gpu_spconv import _t, run_index
    if ref_gpu.lib() is None:
        pytest.skip("oracle/_ref/libref_spconv.so was not built")
    if geo["n"] == 0:
        return
    coors = unique_coors(rng(geo["seed"]), geo["n"], geo["shape"])
    n_max = geo["n"] + 5
    kvol = int(np.prod(geo["ks"]))
    args = (geo["ks"], geo["stride"], geo["pad"], geo["dil"])
    oshape = geo["shape"] if geo["subm"] else orc.out_shape(geo["shape"], *args, geo["out_pad"], geo["transpose"])
    max_out = n_max if geo["subm"] else 40000
    want = ref_gpu.spconv_index(_t(coors), n_max, oshape, *args, max_out, geo["subm"], geo["transpose"])
    spatial = [geo["shape"][0], 0] + geo["shape"][1:]
    got, _ = run_index(d3d, coors, n_max, spatial, *args, geo["out_pad"], max_out, geo["subm"], geo["transpose"])
    assert int(got[1].item()) == int(want[1].item())
    if geo["subm"]:
        assert torch.equal(got[0], want[0])
        return
    g_out, w_out = int(got[3].item()), int(want[3].item())
    assert g_out == w_out
    gc, gp, _ = orc.canonical_conv(got[0].cpu().numpy(), int(got[1].item()), got[2].cpu().numpy(), g_out, kvol)
    wc, wp, _ = orc.canonical_conv(want[0].cpu().numpy(), int(want[1].item()), want[2].cpu().numpy(), w_out, kvol)
    assert (gc == wc).all()
    pairs_equal(gp, wp, kvol)
