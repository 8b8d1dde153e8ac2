"""GPU parity of the tcgen05/TMEM SPConvMM kernel: forced through set_kernel(2), compared with the fp32-accumulating
oracle at 1e-2 (fp16 / bf16) and with the SIMT kernel of the same library; the kernel's bounded waits must not
have expired (error word 0)."""
import ctypes

import numpy as np
import pytest
import torch

from tests._util import (assert_feats_close, assert_table_consistent, assert_tables_equal, rng, round_to, table_pairs,
                         table_parts, table_row_bits, unique_coors)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _t(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return t if dtype is None else t.to(dtype)


def _kernel_error():
    from deploy3d_b200 import _lib
    code = ctypes.c_int(-1)
    _lib.check("d3d_debug_take_kernel_error", _lib.lib().d3d_debug_take_kernel_error(ctypes.byref(code)))
    return code.value


def _rulebook(d3d, coors, shape_b, ks, st, pd, subm, max_out, dilation=(1, 1, 1)):
    n = coors.shape[0]
    num_in = torch.tensor([n], dtype=torch.int32, device=DEV)
    outs = d3d.spconv_index(_t(coors), num_in, torch.empty([shape_b[0], 0] + shape_b[1:], dtype=torch.int32,
                                                           device=DEV),
                            ks, st, pd, tuple(dilation), (0, 0, 0), max_out, subm, False)
    return outs, num_in


def _run(d3d, orc, outs, num_in, num_out, n_in, n_out_max, cin, cout, ks, inverse, dtype, seed, relu=False,
         residual=False):
    from deploy3d_b200.plugins import SPConvMMPlugin, deserialize_plugin
    r = rng(seed)
    kvol = int(np.prod(ks))
    feats = r.standard_normal((n_in, cin)).astype(np.float32)
    w = (r.standard_normal((kvol, cin, cout)) * np.sqrt(2.0 / (kvol * cin))).astype(np.float32)
    b = r.standard_normal(cout).astype(np.float32)
    res = r.standard_normal((n_out_max, cout)).astype(np.float32) if residual else None
    tdt = torch.float16 if dtype == "fp16" else torch.bfloat16
    table = SPConvMMPlugin.prepare(kvol, inverse, n_out_max, outs[0], outs[1])
    got = {}
    for which in (2, 3, 1):  # tcgen05 (two CTAs per SM where it applies), tcgen05 with one CTA per SM, SIMT
        plug = deserialize_plugin("SPConvMM", d3d.data_s_spconv_mm(ks, cin, cout, n_out_max, False, inverse, w, b))
        plug.configure(tdt)
        plug.set_kernel(which)
        y = plug.run(_t(feats, tdt), num_out, table, relu=relu, residual=None if res is None else _t(res, tdt))
        assert _kernel_error() == 0, "a bounded wait of the tensor-core kernel expired"
        got[which] = y.float().cpu().numpy()
    want = orc.spconv_mm(round_to(feats, dtype), round_to(w, dtype), round_to(b, dtype), outs[0].cpu().numpy(),
                         int(outs[1].item()), inverse, n_out_max)
    if res is not None:
        want = want + round_to(res, dtype)
    if relu:
        want = np.maximum(want, 0)
    assert_feats_close(got[2], want, 1e-2, "tcgen05 vs oracle")
    assert (got[2] == got[3]).all(), "one or two CTAs per SM accumulate in the same order: identical results"
    assert_feats_close(got[2], got[1], 1e-2, "tcgen05 vs SIMT")
    return got[2]


def test_smallest_case(d3d, orc):
    """One tile, 16 -> 16 channels: the first thing to run on a new box."""
    coors = unique_coors(rng(1), 100, [1, 6, 6, 6])
    outs, num_in = _rulebook(d3d, coors, [1, 6, 6, 6], (3, 3, 3), (1, 1, 1), (1, 1, 1), True, 100)
    _run(d3d, orc, outs, num_in, num_in, 100, 100, 16, 16, (3, 3, 3), False, "fp16", 2)


@pytest.mark.parametrize("cin,cout", [(16, 16), (16, 32), (32, 32), (32, 64), (64, 64), (64, 128), (128, 128),
                                      (128, 64), (64, 32), (32, 16), (64, 48), (128, 256), (256, 128), (256, 256),
                                      (16, 80)])
@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_channel_grid_subm(d3d, orc, cin, cout, dtype):
    coors = unique_coors(rng(3), 5000, [2, 24, 30, 20])
    outs, num_in = _rulebook(d3d, coors, [2, 24, 30, 20], (3, 3, 3), (1, 1, 1), (1, 1, 1), True, 5000)
    _run(d3d, orc, outs, num_in, num_in, 5000, 5000, cin, cout, (3, 3, 3), False, dtype, cin * 1000 + cout)


@pytest.mark.parametrize("ks,pd", [((3, 1, 3), (1, 0, 1)), ((1, 3, 3), (0, 1, 1)), ((3, 1, 1), (1, 0, 0)),
                                   ((1, 1, 1), (0, 0, 0))])
def test_asymmetric_kernels(d3d, orc, ks, pd):
    coors = unique_coors(rng(4), 9000, [2, 48, 36, 16])
    outs, num_in = _rulebook(d3d, coors, [2, 48, 36, 16], ks, (1, 1, 1), pd, True, 9100)
    _run(d3d, orc, outs, num_in, num_in, 9000, 9100, 32, 64, ks, False, "fp16", 5)


def test_strided_inverse_padded_and_epilogue(d3d, orc):
    """Strided conv with buffers larger than the live counts, its inverse, and the fused residual + ReLU epilogue."""
    coors = unique_coors(rng(6), 20000, [2, 120, 90, 8])
    outs, num_in = _rulebook(d3d, coors, [2, 120, 90, 8], (3, 3, 3), (2, 2, 1), (1, 1, 1), False, 50000)
    nout = int(outs[3].item())
    down = _run(d3d, orc, outs, num_in, outs[3], 20000, 50000, 32, 64, (3, 3, 3), False, "fp16", 7, relu=True)
    assert (down[nout:] == down[nout]).all()  # rows beyond numActOut hold relu(bias)
    _run(d3d, orc, outs, outs[3], num_in, 50000, 20000, 64, 32, (3, 3, 3), True, "fp16", 8, relu=True, residual=True)
    _run(d3d, orc, outs, outs[3], num_in, 50000, 20000, 64, 32, (3, 3, 3), True, "bf16", 9, relu=False, residual=True)


def test_config2_through_tensor_cores(d3d, orc):
    """benchmark config 2 at full size: 2 x 60 000 LiDAR-like voxels, 32 -> 64 strided then 64 -> 32 inverse."""
    from deploy3d_b200 import synth
    c = synth.config2()
    n = c["coors"].shape[0]
    outs, num_in = _rulebook(d3d, c["coors"], [2, 41, 1600, 1408], c["ksize"], c["stride"], c["padding"], False, n)
    _run(d3d, orc, outs, num_in, outs[3], n, n, 32, 64, c["ksize"], False, "fp16", 10)
    _run(d3d, orc, outs, outs[3], num_in, n, n, 64, 32, c["ksize"], True, "fp16", 11)


def test_ragged_and_empty_tiles(d3d, orc):
    """M not a multiple of 128, all-empty tiles in the middle (outputs without any neighbour), single row."""
    for n in (1, 127, 129, 1000):
        coors = unique_coors(rng(20 + n), n, [1, 40, 40, 40])
        outs, num_in = _rulebook(d3d, coors, [1, 40, 40, 40], (3, 3, 3), (1, 1, 1), (1, 1, 1), True, n + 300)
        _run(d3d, orc, outs, num_in, num_in, n, n + 300, 16, 32, (3, 3, 3), False, "fp16", 30 + n)


@pytest.mark.parametrize("ks,dil", [((3, 3, 3), (1, 1, 1)), ((3, 1, 3), (1, 1, 2)), ((5, 3, 3), (1, 1, 1))])
def test_mirror_table_build_gives_the_same_table(d3d, ks, dil):
    """A SubM rulebook with 'same' padding is mirror-symmetric; building the neighbour table in gather order from
    the mirrored entries must give exactly the table (ids, per-tile offset masks, row masks) of the generic scatter."""
    pad = tuple(d * (k // 2) for k, d in zip(ks, dil))
    shape = [2, 12, 30, 28]
    coors = unique_coors(rng(21), 3000, shape)
    outs, num_in = _rulebook(d3d, coors, shape, ks, (1, 1, 1), pad, True, 3000, dilation=dil)
    from deploy3d_b200.plugins import SPConvMMPlugin
    kvol = int(np.prod(ks))
    plain = SPConvMMPlugin.prepare(kvol, False, 3000, outs[0], outs[1])
    mirrored = SPConvMMPlugin.prepare(kvol, False, 3000, outs[0], outs[1], mirror=True)
    a, b = table_parts(plain, kvol, 3000), table_parts(mirrored, kvol, 3000)
    assert_tables_equal(a, b, "mirrored build vs generic scatter")
    assert_table_consistent(*a)
    assert int(table_row_bits(a[2]).sum()) == int((outs[0][2, :int(outs[1].item())] >= 0).sum())
    assert (a[1] != 0).any()


@pytest.mark.parametrize("case", ["subm", "strided", "inverse", "subm_313"])
def test_regrouped_table_same_pairs_same_bytes(d3d, orc, case):
    """d3d_spconv_mm_regroup: the regrouped table encodes exactly the (output, offset, input) triples of the plain
    one, its output map is a permutation, it has fewer (tile, offset) blocks on a LiDAR-like scene, and the
    convolution through it gives the same bytes as through the plain table (tensor-core and SIMT kernels, with
    residual and ReLU)."""
    from deploy3d_b200 import synth
    from deploy3d_b200.plugins import SPConvMMPlugin, deserialize_plugin
    r = rng(77)
    shape = [1, 21, 200, 200]
    vox = synth.lidar_like_voxels(r, 30000, tuple(shape[1:]))
    coors = np.concatenate([np.zeros((len(vox), 1), np.int32), vox], 1)
    n = len(coors)
    ks = (3, 1, 3) if case == "subm_313" else (3, 3, 3)
    subm = case.startswith("subm")
    st = (1, 1, 1) if subm else (2, 2, 2)
    pad = tuple(k // 2 for k in ks) if subm else (1, 1, 1)
    cap = n if subm else 4 * n
    outs, num_in = _rulebook(d3d, coors, shape, ks, st, pad, subm, cap)
    kvol = int(np.prod(ks))
    inverse = case == "inverse"
    m_max = n if (subm or inverse) else cap
    num_out = num_in if (subm or inverse) else outs[3]
    n_in_rows = cap if inverse else n
    plain = SPConvMMPlugin.prepare(kvol, inverse, m_max, outs[0], outs[1])
    grouped = SPConvMMPlugin.regroup(kvol, m_max, plain)
    pp, gp = table_parts(plain, kvol, m_max), table_parts(grouped, kvol, m_max)
    assert_table_consistent(*gp)
    assert torch.equal(table_pairs(pp), table_pairs(gp)), "the regrouped table encodes other pairs"
    perm = gp[3].flatten()
    live = perm[perm >= 0]
    assert live.numel() == m_max and torch.equal(torch.sort(live)[0], torch.arange(m_max, device=DEV, dtype=torch.int32))
    blocks = lambda parts: int(sum(bin(int(v) & 0xFFFFFFFF).count("1") for v in parts[1].cpu().numpy()))
    assert blocks(gp) < blocks(pp), (blocks(gp), blocks(pp))
    again = SPConvMMPlugin.regroup(kvol, m_max, plain)
    assert torch.equal(again, grouped) or all(torch.equal(x, y) for x, y in zip(table_parts(again, kvol, m_max)[1:], gp[1:]))
    cin, cout = 32, 64
    w = (r.standard_normal((kvol, cin, cout)) * np.sqrt(2.0 / (kvol * cin))).astype(np.float32)
    b = r.standard_normal(cout).astype(np.float32)
    x = torch.randn((n_in_rows, cin), device=DEV).half()
    res = torch.randn((m_max, cout), device=DEV).half()
    for which in (2, 3, 1):
        plug = deserialize_plugin("SPConvMM", d3d.data_s_spconv_mm(ks, cin, cout, m_max, subm, inverse, w, b))
        plug.configure(torch.float16)
        plug.set_kernel(which)
        y_plain = plug.run(x, num_out, plain, relu=True, residual=res).clone()
        y_grouped = plug.run(x, num_out, grouped, relu=True, residual=res)
        assert _kernel_error() == 0
        assert torch.equal(y_plain, y_grouped), "kernel choice %d: regrouped table changes the result" % which


def test_dependent_launch_is_bit_identical(d3d):
    """Three layers chained on one stream, launched with and without the programmatic stream-serialisation attribute:
    every layer waits for its predecessor before it reads, so the results are the same bit for bit."""
    from deploy3d_b200 import synth
    from deploy3d_b200.ops import data_s_spconv_index, data_s_spconv_mm
    from deploy3d_b200.plugins import SPConvMMPlugin, deserialize_plugin
    r = np.random.Generator(np.random.PCG64(321))
    vox = synth.lidar_like_voxels(r, 60000, (21, 400, 400))
    n = len(vox)
    coors = torch.from_numpy(np.concatenate([np.zeros((n, 1), np.int32), vox], 1)).cuda()
    num = torch.tensor([n], dtype=torch.int32, device="cuda")
    shape = torch.empty([1, 0, 21, 400, 400], dtype=torch.int32, device="cuda")
    ip = deserialize_plugin("SPConvIdx3d", data_s_spconv_index((3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0),
                                                                n, True, False))
    index, num_index = ip.enqueue(coors, num, shape)
    table = SPConvMMPlugin.prepare(27, False, n, index, num_index)
    chans = [(16, 32), (32, 32), (32, 64)]
    plugs = []
    for cin, cout in chans:
        w = synth.kaiming_weight(r, 27, cin, cout)
        b = (r.standard_normal(cout) * 0.1).astype(np.float32)
        pl = deserialize_plugin("SPConvMM", data_s_spconv_mm((3, 3, 3), cin, cout, n, True, False, w, b))
        pl.configure(torch.float16)
        plugs.append(pl)
    x0 = torch.randn((n, 16), device="cuda").half()
    outs = {}
    for enable in (False, True):
        for pl in plugs:
            pl.set_dependent_launch(enable)
        for _ in range(3):  # repeated: a layer must not overwrite what its predecessor still reads
            x = x0
            for pl in plugs:
                x = pl.run(x, num, table, relu=True)
        torch.cuda.synchronize()
        outs[enable] = x.clone()
    assert torch.equal(outs[False], outs[True])
