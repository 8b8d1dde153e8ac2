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
    """The four parts of SPConvMM's neighbour table (a uint8 tensor): ids int32 [tiles, kvol, 128], offset masks
    int32 [tiles], row masks int32 [tiles, kvol, 4], output row of every tile row int32 [tiles, 128]; every part
    starts on a multiple of 256 bytes."""
    import torch
    tiles = (max_num_act_out + 127) // 128
    up = lambda v: (v + 255) // 256 * 256
    ids_bytes, mask_bytes, rows_bytes = kvol * tiles * 128 * 4, tiles * 4, tiles * kvol * 16
    mask_off = up(ids_bytes)
    rows_off = mask_off + up(mask_bytes)
    perm_off = rows_off + up(rows_bytes)
    ids = table[:ids_bytes].view(torch.int32).view(tiles, kvol, 128)
    mask = table[mask_off:mask_off + mask_bytes].view(torch.int32)
    rows = table[rows_off:rows_off + rows_bytes].view(torch.int32).view(tiles, kvol, 4)
    perm = table[perm_off:perm_off + tiles * 128 * 4].view(torch.int32).view(tiles, 128)
    return ids, mask, rows, perm


def table_row_bits(rows):
    """Row masks [tiles, kvol, 4] -> bool [tiles, kvol, 128]."""
    import torch
    tiles, kvol, _ = rows.shape
    bit = (rows.long().view(tiles, kvol, 4, 1) >> torch.arange(32, device=rows.device).view(1, 1, 1, 32)) & 1
    return bit.view(tiles, kvol, 128).bool()


def assert_tables_equal(a, b, what=""):
    """Same offset masks, row masks and output map; same ids wherever a row-mask bit is set (the others are
    unspecified)."""
    import torch
    (ids_a, mask_a, rows_a, perm_a), (ids_b, mask_b, rows_b, perm_b) = a, b
    assert torch.equal(mask_a, mask_b), what + ": offset masks differ"
    assert torch.equal(rows_a, rows_b), what + ": row masks differ"
    assert torch.equal(perm_a, perm_b), what + ": output maps differ"
    bits = table_row_bits(rows_a)
    assert torch.equal(ids_a[bits], ids_b[bits]), what + ": ids differ"


def assert_table_consistent(ids, mask, rows, perm=None):
    """Offset masks say what the row masks say, ids under a set bit are row indices, and a plain table maps tile row
    p to output p."""
    import torch
    tiles, kvol, _ = ids.shape
    bits = table_row_bits(rows)
    assert (ids[bits] >= 0).all(), "an id under a set row-mask bit is negative"
    if kvol <= 32:
        any_k = bits.any(-1).long()
        want_mask = (any_k * (1 << torch.arange(kvol, device=ids.device, dtype=torch.int64))).sum(-1)
        assert torch.equal(mask.long() & 0xFFFFFFFF, want_mask), "offset masks disagree with the row masks"


def table_pairs(parts):
    """The set of (output row, offset, input row) a table encodes, as a sorted int64 [n, 3] tensor."""
    import torch
    ids, mask, rows, perm = parts
    bits = table_row_bits(rows)
    t, k, r = bits.nonzero(as_tuple=True)
    out = perm[t, r].long()
    trip = torch.stack([out, k, ids[t, k, r].long()], 1)
    key = (trip[:, 0] * 64 + trip[:, 1]) * (1 << 32) + trip[:, 2]
    return trip[torch.argsort(key)]
