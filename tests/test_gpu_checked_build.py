"""The checked build of the library (-DDEPLOY3D_BOUNDS_CHECK, `python -m deploy3d_b200.build --checked`): every row id,
table entry and coordinate is range-checked before use and the first violation recorded.  Run in a child process
(the library choice is made when the package is imported): the small parity cases leave the record empty; ids that
point beyond the extent the caller declared are recorded and skipped.  The bad ids stay inside the allocations, so
the regular build would read valid memory too: nothing here can fault."""
import json
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECKED = os.path.join(ROOT, "deploy3d_b200", "libs", "libdeploy3d_b200_checked.so")

CHILD = textwrap.dedent("""
    import ctypes, json, sys
    sys.path.insert(0, %r)
    import numpy as np, torch
    from deploy3d_b200 import _lib, ops, synth
    from deploy3d_b200.plugins import SPConvMMPlugin, deserialize_plugin
    from deploy3d_b200.ops import data_s_spconv_index, data_s_spconv_mm
    assert _lib.LIB_PATH.endswith("_checked.so")
    L = _lib.lib()
    dev = "cuda:0"

    def take():
        rec = (ctypes.c_int32 * 4)()
        _lib.check("d3d_debug_take_bounds_violation", L.d3d_debug_take_bounds_violation(rec))
        return list(rec)

    out = {}
    r = np.random.Generator(np.random.PCG64(3))
    shape = (11, 60, 60)
    vox = synth.lidar_like_voxels(r, 5000, shape)
    n = len(vox)
    coors = torch.from_numpy(np.concatenate([np.zeros((n, 1), np.int32), vox], 1)).to(dev)
    num = torch.tensor([n], dtype=torch.int32, device=dev)
    shp = torch.empty([1, 0] + list(shape), dtype=torch.int32, device=dev)
    x = torch.randn((n, 32), device=dev).half()
    w = synth.kaiming_weight(r, 27, 32, 32)
    b = np.zeros(32, np.float32)
    results = {}
    for subm in (True, False):
        st = (1, 1, 1) if subm else (2, 2, 2)
        cap = n if subm else 8 * n
        ip = deserialize_plugin("SPConvIdx3d", data_s_spconv_index((3, 3, 3), st, (1, 1, 1), (1, 1, 1), (0, 0, 0), cap,
                                                                    subm, False))
        outs = ip.enqueue(coors, num, shp)
        num_out = num if subm else outs[3]
        table = SPConvMMPlugin.prepare(27, False, cap, outs[0], outs[1])
        for which in (2, 1):
            mm = deserialize_plugin("SPConvMM", data_s_spconv_mm((3, 3, 3), 32, 32, cap, subm, False, w, b))
            mm.configure(torch.float16)
            mm.set_kernel(which)
            y = mm.run(x, num_out, table, relu=True)
            results[(subm, which)] = y
        if subm:
            ops.bev_densify(results[(True, 2)], coors, num, shp, 32 * shape[0])
    out["clean"] = take()

    # ids beyond the rows the caller declares: the feature tensor is passed as its first half (same allocation)
    ip = deserialize_plugin("SPConvIdx3d", data_s_spconv_index((3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0), n,
                                                                True, False))
    outs = ip.enqueue(coors, num, shp)
    table = SPConvMMPlugin.prepare(27, False, n, outs[0], outs[1])
    for which, key in ((2, "tc"), (1, "simt")):
        mm = deserialize_plugin("SPConvMM", data_s_spconv_mm((3, 3, 3), 32, 32, n, True, False, w, b))
        mm.configure(torch.float16)
        mm.set_kernel(which)
        mm.run(x[: n // 2], num, table, relu=True)
        out[key] = take()

    # a voxel id beyond the number of voxels in ScatterTo / GatherBack
    pts = torch.randn((1000, 4), device=dev)
    ids = torch.arange(1000, dtype=torch.int32, device=dev) %% 50
    ids[7] = 60
    cnt = torch.ones(50, dtype=torch.int32, device=dev)
    ops.scatter_to(pts, ids, cnt, 0)
    out["scatter_to"] = take()
    red = torch.randn((50, 4), device=dev)
    ops.gather_back(red, ids, 0.0)
    out["gather_back"] = take()
    # a voxel coordinate outside the dense grid in BEVDensify
    bad = coors.clone()
    bad[3, 2] = shape[1] + 5
    ops.bev_densify(results[(True, 2)], bad, num, shp, 32 * shape[0])
    out["bev"] = take()
    # the mirror hint on a rulebook of duplicated coordinates (not mirror-symmetric): recorded at the centre offset
    dup = torch.cat([coors, coors[:40]])
    nd = torch.tensor([n + 40], dtype=torch.int32, device=dev)
    ip = deserialize_plugin("SPConvIdx3d", data_s_spconv_index((3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), (0, 0, 0),
                                                                n + 40, True, False))
    outs = ip.enqueue(dup, nd, shp)
    SPConvMMPlugin.prepare(27, False, n + 40, outs[0], outs[1], mirror=False)
    out["no_hint"] = take()
    SPConvMMPlugin.prepare(27, False, n + 40, outs[0], outs[1], mirror=True)
    out["mirror"] = take()
    print("RESULT " + json.dumps(out))
""") % ROOT


def test_checked_build_records_and_skips(tmp_path):
    if not os.path.exists(CHECKED):
        pytest.skip("the checked library was not built (python -m deploy3d_b200.build --checked)")
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    env = dict(os.environ, DEPLOY3D_B200_CHECKED="1")
    run = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert run.returncode == 0, run.stderr[-3000:]
    got = json.loads([ln for ln in run.stdout.splitlines() if ln.startswith("RESULT ")][-1][7:])
    assert got["clean"] == [0, 0, 0, 0], "valid inputs must leave no record: %s" % got["clean"]
    # {violations, site, value, limit}: sites 1 / 2 = SPConvMM tensor-core / SIMT kernel, 5 ScatterTo, 6 GatherBack, 4 BEV, 7 mirror hint
    for key, site in (("tc", 1), ("simt", 2)):
        count, where, value, limit = got[key]
        assert count > 0 and where == site and value >= limit > 0, (key, got[key])
    assert got["scatter_to"][1:] == [5, 60, 50] and got["scatter_to"][0] >= 1  # one thread per (point, channel group)
    assert got["gather_back"][1:] == [6, 60, 50] and got["gather_back"][0] >= 1
    assert got["bev"][0] == 1 and got["bev"][1] == 4
    assert got["no_hint"] == [0, 0, 0, 0]
    assert got["mirror"][0] == 40 and got["mirror"][1] == 7  # site 7: a row that is not its own centre neighbour
