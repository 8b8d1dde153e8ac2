"""GPU parity of SPConvIdx3d / SPConvMM through the C ABI against the CPU oracle.

Mirrors the reference's tests/spconv/test_spconv.py (same 16-case grid: strided (2,2,1) / SubM x padded input
buffer x truncating maxNumActOut x inverse) and adds transposed, asymmetric, dilated, 2-D and empty cases plus
benchmark configs 1 and 2.  Rulebooks are compared bit-exactly (SubM raw, strided after canonicalisation);
features within 1e-4 (fp32) / 1e-2 (fp16, bf16) of the fp32-accumulating oracle."""
import numpy as np
import pytest
import torch

from tests._util import (assert_feats_close, assert_table_consistent, assert_tables_equal, pairs_equal, rng,
                         round_to, table_parts, unique_coors)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _t(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return t if dtype is None else t.to(dtype)


def run_index(d3d, coors, n_max, spatial_shape, ks, st, pd, dl, op, max_out, subm, tr):
    n = coors.shape[0]
    buf = torch.full((n_max, coors.shape[1]), 12345, dtype=torch.int32, device=DEV)  # garbage beyond numActIn
    buf[:n] = _t(coors)
    num_in = torch.tensor([n], dtype=torch.int32, device=DEV)
    shp = torch.empty(spatial_shape, dtype=torch.int32, device=DEV)
    outs = d3d.spconv_index(buf, num_in, shp, ks, st, pd, dl, op, max_out, subm, tr)
    torch.cuda.synchronize()
    return outs, num_in


def check_index(orc, outs, coors, n_max, shape_b, ks, st, pd, dl, op, max_out, subm, tr):
    kvol = int(np.prod(ks))
    index = outs[0].cpu().numpy()
    num = int(outs[1].item())
    assert index.shape == (3, kvol * (n_max + 128))
    orc.check_layout(index, num, kvol)
    if subm:
        want, wnum = orc.rulebook_subm(coors, shape_b, ks, st, pd, dl, max_num_act_in=n_max)
        assert num == wnum
        assert (index == want).all(), "SubM rulebook differs from the oracle byte for byte"
        return None
    want = orc.rulebook_conv(coors, shape_b, ks, st, pd, dl, op, tr, 10 ** 7, max_num_act_in=n_max)
    wc, wpairs, _ = orc.canonical_conv(want[0], want[1], want[2], want[3], kvol)
    out_coors = outs[2].cpu().numpy()
    nout = int(outs[3].item())
    if len(outs) > 4:  # the plugin's fifth output; absent when `outs` come from the reference's builders
        assert list(outs[4].shape) == [want[4][0], 0] + want[4][1:]
    assert nout == min(want[3], max_out)
    got = out_coors[:nout]
    if nout == want[3]:
        gc, gpairs, order = orc.canonical_conv(index, num, out_coors, nout, kvol)
        assert (gc == wc).all(), "output coordinate sets differ"
        pairs_equal(gpairs, wpairs, kvol)
    else:  # truncated: kept voxels are genuine and unique, pairs are the oracle's restricted to them
        ids = {tuple(c): i for i, c in enumerate(wc.tolist())}
        sel = np.array([ids[tuple(c)] for c in got.tolist()])
        assert len(np.unique(sel)) == nout
        present = np.zeros(len(wc), bool)
        present[sel] = True
        gpairs = orc.canonical_pairs(index, num, kvol, sel)
        for k in range(kvol):
            w = wpairs[k][present[wpairs[k][:, 1]]]
            assert gpairs[k].shape == w.shape and (gpairs[k] == w).all()
    return nout


def run_mm(d3d, orc, index_t, num_index_t, num_in_t, num_out_t, n_in_max, n_out_max, cin, cout, ks, inverse, dtype,
           seed, rtol, n_out_valid):
    r = rng(seed)
    kvol = int(np.prod(ks))
    feats = r.standard_normal((n_in_max, cin)).astype(np.float32)
    w = (r.standard_normal((kvol, cin, cout)) * np.sqrt(2.0 / (kvol * cin))).astype(np.float32)
    b = r.standard_normal(cout).astype(np.float32)
    tdt = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}[dtype]
    out = d3d.spconv_mm(_t(feats, tdt), num_in_t, num_out_t, index_t, num_index_t, ks, cin, cout, n_out_max, False,
                        inverse, w, b)
    torch.cuda.synchronize()
    assert out.dtype == tdt and tuple(out.shape) == (n_out_max, cout)
    want = orc.spconv_mm(round_to(feats, dtype), round_to(w, dtype), round_to(b, dtype), index_t.cpu().numpy(),
                         int(num_index_t.item()), inverse, n_out_max)
    got = out.float().cpu().numpy()
    assert_feats_close(got[:n_out_valid], want[:n_out_valid], rtol, "features")
    # rows beyond numActOut hold the bias, as after the reference's bias initialisation (trt/spconv/mm.h:51-56)
    if n_out_valid < n_out_max:
        assert_feats_close(got[n_out_valid:], want[n_out_valid:], rtol, "bias rows")
    return got


REF_GRID = []
for subm in (False, True):
    for inverse in (False, True):
        for n_max in (20000, 40000):
            for max_out in (50000, 5000):
                REF_GRID.append((subm, inverse, n_max, max_out))


@pytest.mark.parametrize("subm,inverse,n_max,max_out", REF_GRID)
def test_reference_grid(d3d, orc, subm, inverse, n_max, max_out):
    """tests/spconv/test_spconv.py:165-197."""
    r = rng(100 + int(subm) * 8 + int(inverse) * 4 + (n_max > 20000) * 2 + (max_out < 10000))
    shape_b, spatial = [2, 120, 90, 8], [2, 0, 120, 90, 8]
    coors = unique_coors(r, 20000, shape_b)
    ks, pd, dl, op = (3, 3, 3), (1, 1, 1), (1, 1, 1), (0, 0, 0)
    st = (1, 1, 1) if subm else (2, 2, 1)
    if subm:
        max_out = n_max  # test_spconv.py:34-35
    outs, num_in = run_index(d3d, coors, n_max, spatial, ks, st, pd, dl, op, max_out, subm, False)
    nout = check_index(orc, outs, coors, n_max, shape_b, ks, st, pd, dl, op, max_out, subm, False)
    num_out = num_in if subm else outs[3]
    nout = 20000 if subm else nout
    n_in_max, n_out_max, a, b, valid = n_max, max_out, num_in, num_out, nout
    if inverse:  # test_spconv.py:126-128
        n_in_max, n_out_max, a, b, valid = max_out, n_max, num_out, num_in, 20000
    for dtype, rtol in (("fp32", 1e-4), ("fp16", 1e-2)):
        run_mm(d3d, orc, outs[0], outs[1], a, b, n_in_max, n_out_max, 16, 32, ks, inverse, dtype, 5, rtol, valid)


EXTRA = [
    # ks, st, pd, dl, op, tr, subm, shape_b, n
    ((3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1), (1, 1, 1), True, False, [2, 20, 24, 10], 3000),
    ((2, 2, 2), (2, 2, 2), (0, 0, 0), (1, 1, 1), (0, 0, 0), True, False, [1, 16, 16, 16], 1000),
    ((3, 1, 3), (1, 1, 1), (1, 0, 1), (1, 1, 1), (0, 0, 0), False, True, [2, 48, 36, 16], 9000),
    ((1, 3, 3), (1, 1, 1), (0, 1, 1), (1, 1, 1), (0, 0, 0), False, True, [2, 48, 36, 16], 9000),
    ((3, 3, 3), (1, 1, 1), (2, 2, 2), (2, 2, 2), (0, 0, 0), False, True, [1, 30, 30, 12], 5000),
    ((3, 1, 1), (2, 1, 1), (0, 0, 0), (1, 1, 1), (0, 0, 0), False, False, [2, 5, 60, 50], 6000),
    ((3, 3, 3), (2, 2, 2), (0, 1, 1), (1, 1, 1), (0, 0, 0), False, False, [2, 11, 60, 50], 7000),
    ((5, 5, 5), (1, 1, 1), (2, 2, 2), (1, 1, 1), (0, 0, 0), False, True, [1, 14, 14, 14], 1200),
    ((3, 3), (2, 2), (1, 1), (1, 1), (0, 0), False, False, [3, 100, 90], 8000),
    ((3, 3), (1, 1), (1, 1), (1, 1), (0, 0), False, True, [3, 100, 90], 8000),
    ((3,), (2,), (1,), (1,), (0,), False, False, [4, 3000], 4000),
    ((3, 3, 3, 3), (1, 1, 1, 1), (1, 1, 1, 1), (1, 1, 1, 1), (0, 0, 0, 0), False, True, [1, 8, 8, 8, 8], 1500),
    # dilation and stride share a factor: an even coordinate reaches an output through all three taps of an axis
    ((3, 3, 3), (2, 2, 2), (2, 2, 2), (2, 2, 2), (0, 0, 0), False, False, [1, 20, 20, 12], 3000),
    ((3, 3, 3), (2, 1, 2), (1, 1, 1), (1, 1, 1), (0, 0, 0), False, False, [2, 20, 14, 12], 4000),
]


@pytest.mark.parametrize("case", EXTRA)
def test_extra_geometries(d3d, orc, case):
    ks, st, pd, dl, op, tr, subm, shape_b, n = case
    r = rng(abs(hash(str(case))) % 100000)
    coors = unique_coors(r, n, shape_b)
    n_max = n + 77
    spatial = [shape_b[0], 0] + shape_b[1:]
    max_out = n_max if subm else 200000
    outs, num_in = run_index(d3d, coors, n_max, spatial, ks, st, pd, dl, op, max_out, subm, tr)
    nout = check_index(orc, outs, coors, n_max, shape_b, ks, st, pd, dl, op, max_out, subm, tr)
    num_out = num_in if subm else outs[3]
    run_mm(d3d, orc, outs[0], outs[1], num_in, num_out, n_max, max_out, 8, 24, ks, False, "fp32", 6, 1e-4,
           n if subm else nout)


def test_empty_and_tiny(d3d, orc):
    ks, one, zero = (3, 3, 3), (1, 1, 1), (0, 0, 0)
    for n in (0, 1, 2):
        coors = unique_coors(rng(3), n, [1, 4, 4, 4]) if n else np.zeros((0, 4), np.int32)
        outs, num_in = run_index(d3d, coors, 64, [1, 0, 4, 4, 4], ks, one, one, one, zero, 64, True, False)
        check_index(orc, outs, coors, 64, [1, 4, 4, 4], ks, one, one, one, zero, 64, True, False)
        outs, num_in = run_index(d3d, coors, 64, [1, 0, 4, 4, 4], ks, (2, 2, 2), one, one, zero, 64, False, False)
        nout = check_index(orc, outs, coors, 64, [1, 4, 4, 4], ks, (2, 2, 2), one, one, zero, 64, False, False)
        run_mm(d3d, orc, outs[0], outs[1], num_in, outs[3], 64, 64, 4, 4, ks, False, "fp32", 1, 1e-4, nout)


def test_index_is_deterministic(d3d):
    coors = unique_coors(rng(21), 30000, [2, 60, 90, 40])
    a, _ = run_index(d3d, coors, 30000, [2, 0, 60, 90, 40], (3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1), (0, 0, 0),
                     100000, False, False)
    a = [t.clone() for t in a]
    b, _ = run_index(d3d, coors, 30000, [2, 0, 60, 90, 40], (3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1), (0, 0, 0),
                     100000, False, False)
    n = int(a[3].item())
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and torch.equal(a[2][:n], b[2][:n])
    # first-touch numbering: output ids ascend with the smallest (input, offset) pair that produces them
    idx = a[0].cpu().numpy()
    num = int(a[1].item())
    g, s, k = idx[0, :num], idx[1, :num], idx[2, :num]
    m = k >= 0
    first = np.full(n, np.iinfo(np.int64).max)
    np.minimum.at(first, s[m], g[m].astype(np.int64) * 27 + k[m])
    assert (np.diff(first) > 0).all()


def test_config1_subm_fp32(d3d, orc):
    """benchmark config 1: SubM 3x3x3, 16->16, fp32, 20 000 uniform voxels in 41x1600x1408."""
    from deploy3d_b200 import synth
    c = synth.config1()
    outs, num_in = run_index(d3d, c["coors"], 20000, c["spatial_shape"], c["ksize"], c["stride"], c["padding"],
                             c["dilation"], (0, 0, 0), 20000, True, False)
    check_index(orc, outs, c["coors"], 20000, [1, 41, 1600, 1408], c["ksize"], c["stride"], c["padding"],
                c["dilation"], (0, 0, 0), 20000, True, False)
    out = d3d.spconv_mm(_t(c["feats"]), num_in, num_in, outs[0], outs[1], c["ksize"], 16, 16, 20000, True, False,
                        c["weight"], c["bias"])
    want = orc.spconv_mm(c["feats"], c["weight"], c["bias"], outs[0].cpu().numpy(), int(outs[1].item()), False, 20000)
    assert_feats_close(out.cpu().numpy(), want, 1e-4, "config 1")


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_config2_strided_and_inverse(d3d, orc, dtype):
    """benchmark config 2: conv k3 s2 p1 32->64 then its inverse 64->32 over the same rulebook, batch 2 x 60 000."""
    from deploy3d_b200 import synth
    c = synth.config2()
    n = c["coors"].shape[0]
    shape_b = [2, 41, 1600, 1408]
    outs, num_in = run_index(d3d, c["coors"], n, c["spatial_shape"], c["ksize"], c["stride"], c["padding"],
                             c["dilation"], (0, 0, 0), n, False, False)
    nout = check_index(orc, outs, c["coors"], n, shape_b, c["ksize"], c["stride"], c["padding"], c["dilation"],
                       (0, 0, 0), n, False, False)
    tdt = torch.float16 if dtype == "fp16" else torch.bfloat16
    feats = c["feats"].astype(np.float32)
    idx_np, num = outs[0].cpu().numpy(), int(outs[1].item())
    down = d3d.spconv_mm(_t(feats, tdt), num_in, outs[3], outs[0], outs[1], c["ksize"], 32, 64, n, False, False,
                         c["w_down"], c["b_down"])
    want_down = orc.spconv_mm(round_to(feats, dtype), round_to(c["w_down"], dtype), round_to(c["b_down"], dtype),
                              idx_np, num, False, n)
    assert_feats_close(down.float().cpu().numpy()[:nout], want_down[:nout], 1e-2, "down")
    up = d3d.spconv_mm(down, outs[3], num_in, outs[0], outs[1], c["ksize"], 64, 32, n, False, True, c["w_up"],
                       c["b_up"])
    want_up = orc.spconv_mm(down.float().cpu().numpy(), round_to(c["w_up"], dtype), round_to(c["b_up"], dtype),
                            idx_np, num, True, n)
    assert_feats_close(up.float().cpu().numpy(), want_up, 1e-2, "up")


def test_shared_table_and_fused_epilogue(d3d, orc):
    """prepare once / run twice over one rulebook, with the fused ReLU and residual epilogue."""
    from deploy3d_b200.plugins import SPConvMMPlugin, deserialize_plugin
    coors = unique_coors(rng(31), 15000, [1, 40, 80, 60])
    outs, num_in = run_index(d3d, coors, 15000, [1, 0, 40, 80, 60], (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1),
                             (0, 0, 0), 15000, True, False)
    r = rng(32)
    x = r.standard_normal((15000, 16)).astype(np.float32)
    w1 = (r.standard_normal((27, 16, 16)) * 0.1).astype(np.float32)
    w2 = (r.standard_normal((27, 16, 16)) * 0.1).astype(np.float32)
    b1, b2 = r.standard_normal(16).astype(np.float32), r.standard_normal(16).astype(np.float32)
    p1 = deserialize_plugin("SPConvMM", d3d.data_s_spconv_mm((3, 3, 3), 16, 16, 15000, True, False, w1, b1))
    p2 = deserialize_plugin("SPConvMM", d3d.data_s_spconv_mm((3, 3, 3), 16, 16, 15000, True, False, w2, b2))
    p1.configure(torch.float32), p2.configure(torch.float32)
    table = SPConvMMPlugin.prepare(27, False, 15000, outs[0], outs[1])
    xt = _t(x)
    y1 = p1.run(xt, num_in, table, relu=True)
    y2 = p2.run(y1, num_in, table, relu=True, residual=xt)
    idx_np, num = outs[0].cpu().numpy(), int(outs[1].item())
    w_y1 = np.maximum(orc.spconv_mm(x, w1, b1, idx_np, num, False, 15000), 0)
    w_y2 = np.maximum(orc.spconv_mm(w_y1, w2, b2, idx_np, num, False, 15000) + x, 0)
    assert_feats_close(y1.cpu().numpy(), w_y1, 1e-4, "relu")
    assert_feats_close(y2.cpu().numpy(), w_y2, 1e-4, "residual+relu")


def test_error_codes(d3d):
    from deploy3d_b200 import _lib
    from deploy3d_b200.plugins import deserialize_plugin
    plug = deserialize_plugin("SPConvIdx3d", d3d.data_s_spconv_index((3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1),
                                                                     (0, 0, 0), 0, True, False))
    coors = torch.zeros((10, 4), dtype=torch.int32, device=DEV)
    n = torch.tensor([10], dtype=torch.int32, device=DEV)
    with pytest.raises(_lib.D3DError) as e:  # wrong coordinate width
        plug.enqueue(torch.zeros((10, 3), dtype=torch.int32, device=DEV), n,
                     torch.empty((1, 0, 4, 4, 4), dtype=torch.int32, device=DEV))
    assert e.value.status == -1
    with pytest.raises(_lib.D3DError) as e:  # float coordinates
        plug.enqueue(coors.float(), n, torch.empty((1, 0, 4, 4, 4), dtype=torch.int32, device=DEV))
    assert e.value.status == -2
    mm = deserialize_plugin("SPConvMM", d3d.data_s_spconv_mm((3, 3, 3), 4, 4, 10, True, False,
                                                             np.zeros((27, 4, 4), np.float32)))
    idx = torch.full((3, 27 * 138), -1, dtype=torch.int32, device=DEV)
    with pytest.raises(_lib.D3DError) as e:  # int8 features are not supported
        mm.enqueue(torch.zeros((10, 4), dtype=torch.int8, device=DEV), n, n, idx, n)
    assert e.value.status == -2
    torch.cuda.synchronize()


@pytest.mark.parametrize("ks,dil", [((3, 3, 3), (1, 1, 1)), ((3, 1, 3), (1, 1, 1)), ((1, 3, 3), (1, 2, 1)),
                                    ((3, 1, 1), (1, 1, 1)), ((5, 3, 3), (1, 1, 1))])
def test_extended_enqueue_same_index_and_table(d3d, ks, dil):
    """d3d_spconv_index_enqueue_ex on buffers the caller keeps across calls: the index tensor is byte-identical to
    the plain entry point's on every call although only the stale padding is refilled (three voxel sets of
    different sizes in turn, shrinking and growing), and the neighbour table the probe kernel writes equals the one
    d3d_spconv_mm_prepare builds from the rulebook (ids, per-tile offset masks, row masks)."""
    from deploy3d_b200.ops import data_s_spconv_index
    from deploy3d_b200.plugins import SPConvMMPlugin, deserialize_plugin
    shape_b, cap = [2, 20, 26, 22], 5000
    pad = tuple(d * (k // 2) for k, d in zip(ks, dil))
    kvol = int(np.prod(ks))
    blob = data_s_spconv_index(ks, (1, 1, 1), pad, dil, (0, 0, 0), cap, True, False)
    plain, ex = deserialize_plugin("SPConvIdx3d", blob), deserialize_plugin("SPConvIdx3d", blob)
    assert ex.subm_table_ok()
    shp = torch.empty([shape_b[0], 0] + shape_b[1:], dtype=torch.int32, device=DEV)
    index = torch.full((3, kvol * (cap + 128)), 12345, dtype=torch.int32, device=DEV)  # garbage: first_call fills all
    num_index = torch.zeros(1, dtype=torch.int32, device=DEV)
    nbytes = SPConvMMPlugin.table_bytes(kvol, cap)
    table = torch.full((nbytes,), 77, dtype=torch.uint8, device=DEV)
    for call, n in enumerate((4000, 900, 2500, 4999, 1)):
        coors = torch.zeros((cap, 4), dtype=torch.int32, device=DEV)
        coors[:n] = _t(unique_coors(rng(500 + n), n, shape_b))
        num = torch.tensor([n], dtype=torch.int32, device=DEV)
        want = plain.enqueue(coors, num, shp)
        ex.enqueue_ex(coors, num, shp, outputs=[index, num_index], persistent=True, first_call=call == 0,
                      subm_table=table)
        assert int(num_index.item()) == int(want[1].item())
        assert torch.equal(index, want[0]), "call %d: index differs from the plain entry point's" % call
        ref_table = SPConvMMPlugin.prepare(kvol, False, cap, want[0], want[1])
        got_parts, want_parts = table_parts(table, kvol, cap), table_parts(ref_table, kvol, cap)
        assert_tables_equal(got_parts, want_parts, "call %d, probe kernel's table vs the prepared one" % call)
        assert_table_consistent(*got_parts)


def test_extended_enqueue_strided_persistent(d3d):
    """Stale-padding-only refill for a strided rulebook: same index bytes as the plain entry point over several
    voxel sets."""
    from deploy3d_b200.ops import data_s_spconv_index
    from deploy3d_b200.plugins import deserialize_plugin
    shape_b, cap, mout = [1, 24, 40, 36], 6000, 30000
    blob = data_s_spconv_index((3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1), (0, 0, 0), mout, False, False)
    plain, ex = deserialize_plugin("SPConvIdx3d", blob), deserialize_plugin("SPConvIdx3d", blob)
    assert not ex.subm_table_ok()
    shp = torch.empty([1, 0, 24, 40, 36], dtype=torch.int32, device=DEV)
    outs = None
    for call, n in enumerate((5000, 700, 3000)):
        coors = torch.zeros((cap, 4), dtype=torch.int32, device=DEV)
        coors[:n] = _t(unique_coors(rng(700 + n), n, shape_b))
        num = torch.tensor([n], dtype=torch.int32, device=DEV)
        want = plain.enqueue(coors, num, shp)
        if outs is None:
            outs = [torch.full_like(t, 99) if t.numel() else t for t in want]
        ex.enqueue_ex(coors, num, shp, outputs=outs, persistent=True, first_call=call == 0)
        m = int(want[3].item())
        assert int(outs[3].item()) == m and torch.equal(outs[0], want[0]) and torch.equal(outs[2][:m], want[2][:m])


def test_status_word_reports_output_overflow(d3d):
    """The optional status word: a strided rulebook whose maxNumActOut is smaller than the number of output voxels
    drops the surplus (as the reference does, silently, trt/spconv/index.cu:163-168) and says so in the word; a
    rulebook that fits leaves the word alone.  Nothing faults, nothing synchronises."""
    from deploy3d_b200 import _lib
    from deploy3d_b200.ops import data_s_spconv_index
    from deploy3d_b200.plugins import deserialize_plugin
    shape_b, n = [1, 24, 40, 36], 4000
    coors = _t(unique_coors(rng(900), n, shape_b))
    num = torch.tensor([n], dtype=torch.int32, device=DEV)
    shp = torch.empty([1, 0, 24, 40, 36], dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for max_out, want in ((300, _lib.D3D_STATUS_OUTPUT_OVERFLOW), (40000, 0)):
        plug = deserialize_plugin("SPConvIdx3d", data_s_spconv_index((3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1),
                                                                      (0, 0, 0), max_out, False, False))
        outs = plug.enqueue(coors, num, shp)
        status.zero_()
        plug.enqueue_ex(coors, num, shp, outputs=list(outs), status=status)
        assert int(status.item()) == want
        assert int(outs[3].item()) == min(max_out, int(outs[3].item()))
