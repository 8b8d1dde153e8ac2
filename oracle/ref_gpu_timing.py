"""TEST INFRASTRUCTURE ONLY -- the reference's GPU kernels, recompiled for sm_100a, timed beside the product's on
the benchmark frame (config 4: 300 000 points, VoxelResBackBone8x, fp16), one B200.

    python -m oracle.ref_gpu_timing [--reps 5]

For every rulebook of the backbone: the reference's createSparse{SubM,Conv}Index (trt/spconv/index.cu:253-476)
against the product's SPConvIdx3d enqueue + neighbour-table build; for every layer: the reference's indexedSpConv
(trt/spconv/mm.h:35-71: bias initialisation + gather / mma.sync GEMM / half atomic scatter) against the product's
SPConvMM launch, same rulebook, same features, same weights.  CUDA events on the launching stream, one untimed
launch first.  The reference's convolution has no fused ReLU / residual; the product's launch includes them.
Prints one table; it measures, it checks nothing (parity lives in tests/test_gpu_reference.py)."""
import argparse

import numpy as np


def _time(fn, reps):
    import torch
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fn()  # keeps the GPU busy while the host queues the timed calls: the events bracket device time
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps  # microseconds


def measure(reps=5, out=None):
    """Times both sides and returns {"rulebook_us": (reference, product), "conv_us": (reference, product)} per
    frame; prints the per-rulebook / per-layer table to `out` when given.  Raises RuntimeError when the reference
    library is not built."""
    import argparse as _argparse
    import torch
    from deploy3d_b200 import synth
    from deploy3d_b200.backbone import make_weights
    from deploy3d_b200.pipeline import DetectionPipeline
    from oracle import ref_gpu

    def print(*a):  # noqa: A001 -- the table goes to `out` or nowhere
        if out is not None:
            out.write(" ".join(str(x) for x in a) + "\n")

    args = _argparse.Namespace(reps=reps)
    L = ref_gpu.lib()
    if L is None or not L.has_mm:
        raise RuntimeError("oracle/_ref/libref_spconv.so (with the convolution) is not built")
    frame, boxes = synth.config4_points(), synth.config4_boxes()
    probe = DetectionPipeline("centerpoint", "cuda:0")
    probe.load_frame(frame, boxes)
    caps = probe.calibrate([frame])  # buffer capacities as the benchmark sizes them: live counts plus a margin
    del probe
    torch.cuda.empty_cache()
    pipe = DetectionPipeline("centerpoint", "cuda:0", caps=caps, overlap_rulebooks=False)
    pipe.load_frame(frame, boxes)
    pipe.enqueue()
    torch.cuda.synchronize()
    net = pipe.net
    counts = net.counts()
    print("voxel sets:", counts)

    print("\nrulebooks (microseconds per build)")
    print("%-8s %-7s %9s %9s | %12s %12s %7s" % ("key", "kind", "N in", "N out", "reference", "product", "ratio"))
    tot_ref = tot_our = 0.0
    for key, rb in net.rulebooks.items():
        src, dst = net.sets[rb.in_set], net.sets[rb.out_set]
        n = int(src["num"].item())
        coors = src["coors"][:n].contiguous()
        lay = next(l for l in net.layers if l.key == key)
        subm = rb.kind == "subm"
        t_ref = _time(lambda: ref_gpu.spconv_index(coors, src["cap"], dst["shape"], lay.ksize, lay.stride, lay.padding,
                                                   (1, 1, 1), dst["cap"], subm, False, sync=False), args.reps)
        t_our = _time(lambda: net._build_rulebook(rb), args.reps)
        tot_ref, tot_our = tot_ref + t_ref, tot_our + t_our
        print("%-8s %-7s %9d %9d | %12.1f %12.1f %6.1fx" % (key, rb.kind, n, counts[rb.out_set], t_ref, t_our,
                                                            t_ref / t_our))
    print("%-36s | %12.1f %12.1f %6.1fx" % ("all rulebooks of a frame", tot_ref, tot_our, tot_ref / tot_our))
    result = {"rulebook_us": (tot_ref, tot_our)}

    print("\nconvolution layers (microseconds per launch)")
    print("%-5s %-9s %9s | %12s %12s %7s" % ("layer", "channels", "M out", "reference", "product", "ratio"))
    weights = make_weights(net.layers, 0)
    saved, x = {}, pipe.vox_feats_lp
    tot_ref = tot_our = 0.0
    for li, (lay, (plug, out_buf, out_set)) in enumerate(zip(net.layers, net.mm)):
        if lay.source is not None:
            x = saved[lay.source]
        rb = net.rulebooks[lay.key]
        inverse = lay.kind == "inverse"
        table = rb.table_inv if inverse else rb.table_fwd
        res = saved[lay.residual] if lay.residual else None
        w, b = weights[li]
        if w.shape[1] != x.shape[1]:  # the first layer's input is zero-padded to 16 channels
            wp = np.zeros((w.shape[0], x.shape[1], w.shape[2]), dtype=np.float32)
            wp[:, :w.shape[1]] = w
            w = wp
        w_t = torch.from_numpy(w).to("cuda:0", torch.float16)
        b_t = torch.from_numpy(np.asarray(b, dtype=np.float32)).to("cuda:0", torch.float16)
        xin, cap = x, net.sets[out_set]["cap"]
        t_ref = _time(lambda: ref_gpu.spconv_mm(xin, w_t, b_t, rb.index, rb.num_index, inverse, cap, sync=False),
                      args.reps)
        t_our = _time(lambda: plug.run(xin, net.sets[out_set]["num"], table, out=out_buf, relu=lay.relu, residual=res),
                      args.reps)
        x = plug.run(xin, net.sets[out_set]["num"], table, out=out_buf, relu=lay.relu, residual=res)
        if lay.save:
            saved[lay.save] = x
        tot_ref, tot_our = tot_ref + t_ref, tot_our + t_our
        print("%-5d %3d->%-4d %9d | %12.1f %12.1f %6.1fx" % (li, w.shape[1], w.shape[2], counts[out_set], t_ref, t_our,
                                                             t_ref / t_our))
    print("%-25s | %12.1f %12.1f %6.1fx" % ("all layers of a frame", tot_ref, tot_our, tot_ref / tot_our))
    result["conv_us"] = (tot_ref, tot_our)
    return result


def main():
    import sys
    ap = argparse.ArgumentParser()
    ap.add_argument("--reps", type=int, default=5)
    args = ap.parse_args()
    try:
        measure(args.reps, sys.stdout)
    except RuntimeError as e:
        raise SystemExit(str(e))


if __name__ == "__main__":
    main()
