"""Helpers shared by the parity tests: seeded inputs, tolerances, canonical comparisons."""
import numpy as np


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def unique_coors(r, n, shape_b_spatial):
    """n distinct rows (b, d0, ..) in a grid [B, D0, ..] (the reference's _make_unique_coors,
    tests/spconv/test_spconv.py:8-21)."""
    dims = list(shape_b_spatial)
    total = int(np.prod(dims))
    ids = r.choice(total, size=n, replace=False)
    out = np.empty((n, len(dims)), dtype=np.int32)
    for d in range(len(dims) - 1, -1, -1):
        out[:, d] = ids % dims[d]
        ids = ids // dims[d]
    return out


def assert_feats_close(got, want, rtol, what=""):
    """|got - want| <= rtol * (|want| + rms(want)) element-wise: `rtol` relative to the value, with the RMS of the
    tensor as the floor so that entries that cancel to ~0 are judged at the scale of the data."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    if want.size == 0:
        return
    scale = float(np.sqrt(np.mean(want ** 2))) + 1e-30
    err = np.abs(got - want)
    lim = rtol * (np.abs(want) + scale)
    bad = err > lim
    assert not bad.any(), "%s: %d / %d elements off, worst err %.3e at limit %.3e (rms %.3e)" % (
        what, int(bad.sum()), want.size, float(err[bad].max()), float(lim[bad][np.argmax(err[bad])]), scale)


def round_to(a, dtype):
    """Round an fp32 array through fp16 / bf16 the way the device conversion does (round to nearest even)."""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32))
    if dtype == "fp16":
        return t.to(torch.float16).to(torch.float32).numpy()
    if dtype == "bf16":
        return t.to(torch.bfloat16).to(torch.float32).numpy()
    return t.numpy()


def pairs_equal(a, b, kvol):
    for k in range(kvol):
        assert a[k].shape == b[k].shape, "offset %d: %s vs %s pairs" % (k, a[k].shape, b[k].shape)
        assert (a[k] == b[k]).all(), "offset %d: pair lists differ" % k


def table_parts(table, kvol, max_num_act_out):
    """The three parts of SPConvMM's neighbour table (a uint8 tensor): ids int32 [tiles, kvol, 128], offset masks
    int32 [tiles], row masks int32 [tiles, kvol, 4]; every part starts on a multiple of 256 bytes."""
    import torch
    tiles = (max_num_act_out + 127) // 128
    up = lambda v: (v + 255) // 256 * 256
    ids_bytes, mask_bytes = kvol * tiles * 128 * 4, tiles * 4
    mask_off = up(ids_bytes)
    rows_off = mask_off + up(mask_bytes)
    ids = table[:ids_bytes].view(torch.int32).view(tiles, kvol, 128)
    mask = table[mask_off:mask_off + mask_bytes].view(torch.int32)
    rows = table[rows_off:rows_off + tiles * kvol * 16].view(torch.int32).view(tiles, kvol, 4)
    return ids, mask, rows


def assert_table_consistent(ids, mask, rows):
    """Row masks and offset masks say exactly what the ids say: bit r of word q <=> ids[.., 32 q + r] >= 0."""
    import torch
    tiles, kvol, _ = ids.shape
    have = (ids >= 0).view(tiles, kvol, 4, 32).long()
    weights = (1 << torch.arange(32, device=ids.device, dtype=torch.int64))
    want_rows = (have * weights).sum(-1)
    got_rows = rows.long() & 0xFFFFFFFF
    assert torch.equal(got_rows, want_rows), "row masks disagree with the ids"
    if kvol <= 32:
        any_k = (want_rows != 0).any(-1).long()
        want_mask = (any_k * (1 << torch.arange(kvol, device=ids.device, dtype=torch.int64))).sum(-1)
        assert torch.equal(mask.long() & 0xFFFFFFFF, want_mask), "offset masks disagree with the ids"
