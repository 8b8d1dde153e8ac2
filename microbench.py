"""Single-layer micro-benchmark of SPConvIdx + SPConvMM on synthetic LiDAR-like voxels.

    python microbench.py --cin 128 --cout 128 --voxels 66000 [--kernel 2] [--reps 20]

Builds one SubM 3x3x3 rulebook over `--voxels` LiDAR-like active voxels (or a strided one with --stride 2),
prepares the neighbour table once and times `--reps` launches of the convolution kernel with CUDA events.
Prints one JSON line: microseconds per launch, dense-equivalent and pair TFLOP/s, rulebook statistics.
Meant for per-layer tuning and for profiler captures of a single kernel (few launches, small problem).
"""
import argparse
import json

import numpy as np
import torch

from deploy3d_b200 import synth
from deploy3d_b200.ops import data_s_spconv_index, data_s_spconv_mm
from deploy3d_b200.plugins import SPConvMMPlugin, deserialize_plugin


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cin", type=int, default=128)
    ap.add_argument("--cout", type=int, default=128)
    ap.add_argument("--voxels", type=int, default=66000)
    ap.add_argument("--grid", type=int, nargs=3, default=[11, 360, 360], help="Z Y X of the voxel grid")
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--kernel", type=int, default=0, help="0 auto, 1 SIMT, 2 tcgen05, 3 tcgen05 with one CTA per SM")
    ap.add_argument("--dtype", default="fp16", choices=["fp16", "bf16"])
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--index-reps", type=int, default=0, help="also time the rulebook + table build this many times")
    ap.add_argument("--plan", type=int, nargs=3, default=None, metavar=("GROUP", "STAGES", "PRODUCER_WARPS"),
                    help="override the tensor-core kernel's pipeline plan (0 = automatic)")
    ap.add_argument("--regroup", action="store_true",
                    help="run on the neighbour table with its outputs grouped by offset mask (d3d_spconv_mm_regroup)")
    ap.add_argument("--lib", default=None, metavar="NAME",
                    help="load the tuning build libs/libdeploy3d_b200_NAME.so (python -m deploy3d_b200.build --tuning NAME ...)")
    ap.add_argument("--role-cycles", action="store_true",
                    help="after the timed launches, one more launch whose per-role cycle counts (CTA 0) are printed; "
                         "needs a tuning build with -DD3D_TC_PROFILE")
    args = ap.parse_args()
    if args.lib:
        from deploy3d_b200 import _lib
        _lib.use_tuning_build(args.lib)
    if args.plan:
        from deploy3d_b200 import _lib
        _lib.check("d3d_debug_set_tc_plan", _lib.lib().d3d_debug_set_tc_plan(*args.plan))
    dev = "cuda:0"
    rng = np.random.Generator(np.random.PCG64(77))
    vox = synth.lidar_like_voxels(rng, args.voxels, tuple(args.grid), sigma=6.0)
    coors = torch.from_numpy(np.concatenate([np.zeros((len(vox), 1), np.int32), vox], 1)).to(dev)
    n = coors.shape[0]
    num_in = torch.tensor([n], dtype=torch.int32, device=dev)
    subm = args.stride == 1
    ks, st, pd = (3, 3, 3), (args.stride,) * 3, (1, 1, 1)
    max_out = n if subm else 8 * n
    shape = torch.empty([1, 0] + list(args.grid), dtype=torch.int32, device=dev)
    idx_plug = deserialize_plugin("SPConvIdx3d", data_s_spconv_index(ks, st, pd, (1, 1, 1), (0, 0, 0), max_out, subm,
                                                                     False))
    outs = idx_plug.enqueue(coors, num_in, shape)
    num_out = num_in if subm else outs[3]
    m = int(num_out.item())
    table = SPConvMMPlugin.prepare(27, False, max_out, outs[0], outs[1], mirror=subm)
    blocks_plain = None
    if args.regroup:
        tiles = (max_out + 127) // 128
        mask_off = (27 * tiles * 128 * 4 + 255) // 256 * 256
        count = lambda t: int(sum(bin(int(v) & 0xFFFFFFFF).count("1")
                                  for v in t[mask_off:mask_off + 4 * tiles].view(torch.int32).cpu().numpy()))
        blocks_plain = count(table)
        plain = table
        table = SPConvMMPlugin.regroup(27, max_out, plain)
        blocks_grouped = count(table)
        scratch = torch.empty(max(SPConvMMPlugin.regroup_scratch_bytes(27, max_out), 16), dtype=torch.uint8, device=dev)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(10):
            SPConvMMPlugin.regroup(27, max_out, plain, table, scratch)
        t1.record()
        torch.cuda.synchronize()
        regroup_us = t0.elapsed_time(t1) * 100.0
    pairs = int((outs[0][2, :int(outs[1].item())] >= 0).sum().item())
    tdt = torch.float16 if args.dtype == "fp16" else torch.bfloat16
    w = synth.kaiming_weight(rng, 27, args.cin, args.cout)
    b = (rng.standard_normal(args.cout) * 0.1).astype(np.float32)
    mm = deserialize_plugin("SPConvMM", data_s_spconv_mm(ks, args.cin, args.cout, max_out, subm, False, w, b))
    mm.configure(tdt)
    mm.set_kernel(args.kernel)
    x = torch.randn((n, args.cin), device=dev).to(tdt)
    out = torch.empty((max_out, args.cout), dtype=tdt, device=dev)
    for _ in range(args.warmup):
        mm.run(x, num_out, table, out=out, relu=True)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.reps):
        mm.run(x, num_out, table, out=out, relu=True)
    e1.record()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) * 1e-3 / args.reps
    res = {"cin": args.cin, "cout": args.cout, "voxels_in": n, "voxels_out": m, "pairs": pairs, "kernel": args.kernel,
           "us_per_launch": sec * 1e6, "tflops_dense": 2.0 * m * 27 * args.cin * args.cout / sec / 1e12,
           "tflops_pair": 2.0 * pairs * args.cin * args.cout / sec / 1e12,
           "neighbours_per_output": pairs / max(m, 1)}
    if blocks_plain is not None:
        res["tile_offset_blocks"] = {"plain": blocks_plain, "regrouped": blocks_grouped}
        res["regroup_us"] = regroup_us
    if args.role_cycles:
        import ctypes
        from deploy3d_b200 import _lib
        mm.run(x, num_out, table, out=out, relu=True)
        buf = (ctypes.c_longlong * 24)()
        copy_prof = _lib.lib().d3d_debug_copy_prof  # AttributeError without -DD3D_TC_PROFILE
        copy_prof.restype, copy_prof.argtypes = ctypes.c_int, [ctypes.POINTER(ctypes.c_longlong)]
        _lib.check("d3d_debug_copy_prof", copy_prof(buf))
        c = np.array(list(buf)).reshape(3, 8)
        res["role_cycles"] = {
            "producer_warp0": {"other": int(c[0, 0]), "walk_and_id_loads": int(c[0, 1]), "wait_empty": int(c[0, 2]),
                               "address_and_copy_issue": int(c[0, 3])},
            "mma_warp": {"other": int(c[1, 0]), "wait_full": int(c[1, 1]), "proxy_fence": int(c[1, 2]),
                         "issue_and_commit": int(c[1, 3]), "wait_accumulator": int(c[1, 4])},
            "epilogue_warp0": {"other": int(c[2, 0]), "wait_accumulator_full": int(c[2, 1]), "work": int(c[2, 2])}}
    if args.index_reps:
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.index_reps):
            outs = idx_plug.enqueue(coors, num_in, shape, outputs=list(outs))
            SPConvMMPlugin.prepare(27, False, max_out, outs[0], outs[1], table=table, mirror=subm)
        e1.record()
        torch.cuda.synchronize()
        res["us_rulebook_and_table"] = e0.elapsed_time(e1) * 1e3 / args.index_reps
    print(json.dumps(res))


if __name__ == "__main__":
    main()
