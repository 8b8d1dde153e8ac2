#!/usr/bin/env python
"""Benchmark of the sparse-convolution hot path: CenterPoint-shaped frames per second.

    python bench.py [--gpus N] [--steps K] [--warmup W]            this implementation (one process per GPU)
    python bench.py --impl reference [--steps K] [--warmup W]      the CPU restatement of the reference on host cores

One step = FRAMES_PER_STEP frames of benchmark config 4 (300 000 points x 5 channels -> mean voxel encoder ->
VoxelResBackBone8x 16/32/64/128 in fp16 -> BEV densify, plus rotated-BEV NMS over 10 x 1000 boxes at IoU 0.2) on
synthetic, seeded data.  Prints ONE JSON line (rank 0).  `value` is measured with the inputs resident in HBM (CUDA-graph replay,
CUDA events); `e2e` drives the same frames from pinned host memory through the public pipeline object, with the
H2D copy of every frame's inputs and the D2H read of its results inside the timed region.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "sparse backbone frames/s (CenterPoint-shaped frame, fp16)"
UNIT = "frames/s"
WORKLOAD = "config4: 300000 pts x5 -> mean VFE -> VoxelResBackBone8x 16/32/64/128 fp16 -> BEVDensify + NMS3d 10x1000 @0.2"
N_ROTATE = 4  # distinct synthetic frames cycled through the input buffers
FRAMES_PER_STEP = 10  # frames per GPU and step: 20 steps time 200 frames per GPU, about half a second
REFERENCE_BUDGET_S = 150.0  # the CPU arm stops adding timed steps once this much time has been spent
CPU_FRACTION = 1.0 / 16  # share of one frame (an azimuth sector) the CPU arm processes per thread and step
CPU_DENOM = 16


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], source="measured (MEASURED_PEAKS.json)")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback (MEASURED_PEAKS.json absent: earlier B200 measurement)")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------------------------
# CPU arm: the oracle restatement on host cores
# ------------------------------------------------------------------------------------------------------------------
def sector_sample(frame, fraction, which=0):
    """Points of an azimuth sector holding `fraction` of the frame: keeps local density and neighbourhoods intact,
    so the work per point matches the full frame."""
    pts = frame["points"]
    az = np.arctan2(pts[:, 1], pts[:, 0])
    edges = np.quantile(az, np.linspace(0, 1, int(round(1 / fraction)) + 1))
    lo, hi = edges[which % (len(edges) - 1)], edges[which % (len(edges) - 1) + 1]
    m = (az >= lo) & (az < hi)
    return pts[m], frame["batch"][m]


def cpu_frames_per_second(threads, fraction, steps, warmup, budget_s=None):
    """Runs `threads` sector samples concurrently per step; returns (frames/s, seconds per step, steps run).
    With `budget_s`, no further step is started once the timed steps have used that much time."""
    from concurrent.futures import ThreadPoolExecutor
    from deploy3d_b200 import synth
    from oracle import pipeline_cpu
    frame = synth.config4_points()
    boxes = synth.config4_boxes()
    nbox = max(1, int(round(10 * fraction)))  # the NMS rows are independent: take the same fraction of them
    sub_boxes = dict(scores=boxes["scores"][:nbox], boxes=boxes["boxes"][:nbox])
    samples = [sector_sample(frame, fraction, i) for i in range(threads)]

    def one(i):
        p, b = samples[i]
        pipeline_cpu.run_frame("centerpoint", p, b, frame["voxel_config"], frame["spatial_shape"], sub_boxes, 0.2)

    def step():
        with ThreadPoolExecutor(max_workers=threads) as ex:
            list(ex.map(one, range(threads)))

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    done = 0
    while done < steps:
        step()
        done += 1
        if budget_s is not None and time.perf_counter() - t0 > budget_s:
            break
    dt = (time.perf_counter() - t0) / done
    return threads * fraction / dt, dt, done


def run_reference(args):
    """The reference has no CPU implementation of its own; this arm times the CPU restatement of its algorithm
    (oracle/: scalar C, one thread per azimuth sector, one sector per host core and step).  It loads neither the
    product library nor a GPU."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = len(os.sched_getaffinity(0))
    fraction = CPU_FRACTION
    warmup = 1 if args.warmup > 0 else 0
    # every requested step is run unless the budget runs out first (a step is some 2-20 s, depending on the host)
    fps, dt, steps = cpu_frames_per_second(cores, fraction, max(1, args.steps), warmup, REFERENCE_BUDGET_S)
    line = {
        "impl": "reference", "metric": METRIC, "value": fps, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 accumulate over fp16-rounded operands", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": "1/%d azimuth sector of the frame per thread" % CPU_DENOM},
        "cpu_baseline": {"value": fps, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": "%d threads x (1/%d azimuth sector of one config-4 frame, 1 of the 10 NMS rows) "
                                   "per step, frames/s = threads/%d/t; %d of %d requested steps fit the %d s budget"
                                   % (cores, CPU_DENOM, CPU_DENOM, steps, args.steps, int(REFERENCE_BUDGET_S))},
        "e2e": {"value": fps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def reference_gpu_kernels():
    """Informational key of this implementation's line (`config.reference_gpu`): the reference's own CUDA kernels
    compile for sm_100a (oracle/_ref/libref_spconv.so).  When that library is present, its rulebook builders and
    convolution launches are timed on the benchmark frame, one after the other with CUDA events, after the timed
    regions of the benchmark.  Not a frames/s figure of a complete reference pipeline: its ReLU / add graph ops,
    encoder, densify, NMS and host synchronisations are not included, so 1 / (sum) bounds it from above."""
    try:
        from oracle import ref_gpu_timing
        r = ref_gpu_timing.measure(reps=5)
        ref_ms = (r["rulebook_us"][0] + r["conv_us"][0]) * 1e-3
        return {"rulebook_ms_per_frame": r["rulebook_us"][0] * 1e-3, "conv_ms_per_frame": r["conv_us"][0] * 1e-3,
                "frames_per_s_upper_bound": 1e3 / ref_ms,
                "product_rulebook_ms_per_frame": r["rulebook_us"][1] * 1e-3,
                "what": "reference CUDA kernels (trt/spconv/index.cu, trt/spconv/mm.h) recompiled for sm_100a, "
                        "rulebooks + 21 convolution launches of one config-4 frame, back to back on one B200"}
    except Exception as e:  # informational only
        sys.stderr.write("reference_gpu skipped: %s\n" % e)
        return None


# ------------------------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------------------------
DRAM_PROFILE = os.path.join(ROOT, "profiles", "spconv_mm_tc_bench_layers_dram.md")
INNER_LAUNCHES = 4  # timed launches per layer and frame in the per-layer pass


def conv_dram_bytes_per_frame():
    """dram__bytes_read.sum + dram__bytes_write.sum over the 21 SPConvMM launches of one config-4 frame, from the ncu
    capture summarised in profiles/spconv_mm_tc_bench_layers_dram.md (its `dram_bytes_per_frame:` line, which also
    names the kernel source revision it was captured at).  None when the summary is missing."""
    import re
    try:
        with open(DRAM_PROFILE) as f:
            m = re.search(r"^dram_bytes_per_frame:\s*([0-9.eE+]+)\s*\((.*)\)\s*$", f.read(), re.M)
        return (float(m.group(1)), m.group(2)) if m else None
    except OSError:
        return None


def conv_launch_times(pipe, frames, reps):
    """CUDA-event duration of every SPConvMM launch of a frame (eager replay of the layer list), averaged over
    `reps` frames.  Returns per-layer dicts with dense-equivalent and pair FLOPs."""
    import torch
    from deploy3d_b200.plugins import SPConvMMPlugin
    net = pipe.net
    n_layers = sum(1 for L in net.layers if L.kind != "ew")
    conv_layers = [L for L in net.layers if L.kind != "ew"]
    acc = np.zeros(n_layers)
    work = None
    for r in range(reps):
        pipe.load_frame(frames[r % len(frames)])
        pipe.enqueue()
        torch.cuda.synchronize()
        if work is None:
            work = net.layer_work()
        saved, x = {"input": pipe.vox_feats_lp}, pipe.vox_feats_lp
        ci = -1
        for L, (plug, out_buf, out_set) in zip(net.layers, net.mm):
            if L.kind == "ew":  # element-wise graph op between plugins: not a convolution launch
                from deploy3d_b200.backbone import ew_apply
                out_buf.copy_(ew_apply(L.ew[0], [saved[t].float() for t in L.ew[1]], torch))
                x = out_buf
                if L.save:
                    saved[L.save] = x
                continue
            ci += 1
            li = ci
            if L.source is not None:
                x = saved[L.source]
            rb = net.rulebooks[L.key]
            table = rb.table_inv if L.kind == "inverse" else rb.table_fwd
            res = saved[L.residual] if L.residual else None
            # an untimed launch first keeps the GPU busy while the host queues the timed ones, so that the events
            # bracket kernel time and not the host's launch path
            xin = x
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            hint = bool(getattr(rb, "regroup", False))
            x = plug.run(xin, net.sets[out_set]["num"], table, out=out_buf, relu=L.relu_mode, residual=res,
                         regrouped=hint)
            e0.record()
            for _ in range(INNER_LAUNCHES):
                x = plug.run(xin, net.sets[out_set]["num"], table, out=out_buf, relu=L.relu_mode, residual=res,
                             regrouped=hint)
            e1.record()
            e1.synchronize()
            acc[li] += e0.elapsed_time(e1) * 1e-3 / INNER_LAUNCHES
            if L.save:
                saved[L.save] = x
    out = []
    for li, (cin, cout, kvol, m, pairs) in enumerate(work):
        t = acc[li] / reps
        esz = 2
        out.append(dict(layer=li, cin=cin, cout=cout, kvol=kvol, m=m, pairs=pairs, seconds=t,
                        flops_dense=2.0 * m * kvol * cin * cout, flops_pair=2.0 * pairs * cin * cout,
                        bytes=m * cin * esz + m * cout * esz + kvol * cin * cout * esz + 4.0 * kvol * m +
                        (m * cout * esz if conv_layers[li].residual else 0)))
    return out


def run_ours(args):
    import torch
    from deploy3d_b200 import _lib, synth
    from deploy3d_b200.pipeline import DetectionPipeline

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus %d needs one process per GPU: launch with python -m torch.distributed.run "
                             "--nproc-per-node %d bench.py --gpus %d ..." % (args.gpus, args.gpus, args.gpus))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    _lib.lib()  # fails loudly when the CUDA library is missing
    if args.tc_plan:
        _lib.check("d3d_debug_set_tc_plan", _lib.lib().d3d_debug_set_tc_plan(*args.tc_plan))
    torch.cuda.set_device(local)
    dev = "cuda:%d" % local
    dist = None
    if world > 1:
        # The frames are independent replicas: no data crosses GPUs.  The ranks only meet at the barriers around the
        # timed regions and to exchange their elapsed times, which a host-side (gloo) group does.
        import torch.distributed as dist
        dist.init_process_group("gloo")

    frames = [synth.config4_points(i) for i in range(N_ROTATE)]
    boxes = synth.config4_boxes()
    probe = DetectionPipeline("centerpoint", dev, kernel=args.kernel, regroup=args.regroup)
    probe.load_frame(frames[0], boxes)
    caps = probe.calibrate(frames)
    del probe
    torch.cuda.empty_cache()
    # `in_flight` pipelines, each with its own buffers, CUDA graph and stream, take the frames in turn: frame i+1
    # starts (voxelisation, first rulebooks) while frame i runs its last, narrow layers -- what a serving loop over a
    # stream of frames does with two execution contexts.  Every frame still runs the whole path.
    n_pipes = max(1, args.in_flight)
    pipes = []
    for _ in range(n_pipes):
        q = DetectionPipeline("centerpoint", dev, caps=caps, kernel=args.kernel, regroup=args.regroup)
        q.load_frame(frames[0], boxes)
        q.capture()
        pipes.append(q)
    pipe = pipes[0]
    run_streams = [torch.cuda.Stream(device=dev) for _ in range(n_pipes)]
    torch.cuda.synchronize()
    dev_pts = [torch.from_numpy(f["points"]).to(dev) for f in frames]
    working_set = pipe.buffer_bytes()
    fps_step = FRAMES_PER_STEP

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()

    # ---- device-resident throughput: graph replay, inputs already in HBM ------------------------------------------
    main_stream = torch.cuda.current_stream()

    def fork():
        for st in run_streams:
            st.wait_stream(main_stream)

    def join():
        for st in run_streams:
            main_stream.wait_stream(st)

    def device_loop(n, marks=None):
        for i in range(n):
            k = i % n_pipes
            with torch.cuda.stream(run_streams[k]):
                if marks is not None:
                    marks.append((torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)))
                    marks[-1][0].record(run_streams[k])
                pipes[k].points.copy_(dev_pts[i % N_ROTATE], non_blocking=True)
                pipes[k].replay()
                if marks is not None:
                    marks[-1][1].record(run_streams[k])

    fork()
    device_loop(args.warmup * fps_step)
    join()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()  # on the launching stream; the run streams start after it and are joined before e1
    fork()
    device_loop(args.steps * fps_step)
    join()
    e1.record()
    barrier()
    elapsed = e0.elapsed_time(e1) * 1e-3
    clocks = sampler.stop() if rank == 0 else None
    # latency of one frame at that throughput (untimed extra pass: start and end events around every frame)
    marks = []
    fork()
    device_loop(4 * n_pipes + 4, marks)
    join()
    torch.cuda.synchronize()
    frame_latency_ms = float(np.median([a.elapsed_time(b) for a, b in marks[n_pipes:]]))

    # ---- end to end: pinned host -> device -> pipeline -> host ----------------------------------------------------
    host_pts = [torch.from_numpy(f["points"]).pin_memory() for f in frames]
    host_batch = torch.from_numpy(frames[0]["batch"]).pin_memory()
    host_scores = torch.from_numpy(boxes["scores"]).pin_memory()
    host_boxes = torch.from_numpy(boxes["boxes"]).pin_memory()
    count_tensors = [[q.vox_num] + [s["num"] for k, s in q.net.sets.items() if k != "in"] for q in pipes]
    h2d = host_pts[0].numel() * 4 + host_batch.numel() * 4 + host_scores.numel() * 4 + host_boxes.numel() * 4
    d2h = host_scores.numel() * 4 + 4 * len(count_tensors[0])
    # Two frames in flight, as a serving loop would run it: the host-to-device copy of frame i+1 (copy stream, into
    # one of two staging sets) overlaps the pipeline of frame i; the host picks up the result of frame i-1 while
    # frame i runs.  Every frame still pays its own H2D, device-to-device hand-over, graph replay and D2H.
    copy_stream = torch.cuda.Stream(device=dev)
    staging = [dict(points=torch.empty_like(pipe.points), batch=torch.empty_like(pipe.batch),
                    scores=torch.empty_like(pipe.scores), boxes=torch.empty_like(pipe.boxes)) for _ in range(2)]
    out_scores = [torch.empty_like(host_scores).pin_memory() for _ in range(2)]
    out_counts = [torch.zeros(8, dtype=torch.int32).pin_memory() for _ in range(2)]
    h2d_done = [torch.cuda.Event() for _ in range(2)]
    frame_done = [torch.cuda.Event() for _ in range(2)]

    def e2e_loop(n):
        for i in range(n):
            s = i % 2
            if i >= 2:
                frame_done[s].synchronize()  # frame i-2 is on the host: its staging set and result buffers are free
            with torch.cuda.stream(copy_stream):
                staging[s]["points"].copy_(host_pts[i % N_ROTATE], non_blocking=True)
                staging[s]["batch"].copy_(host_batch, non_blocking=True)
                staging[s]["scores"].copy_(host_scores, non_blocking=True)
                staging[s]["boxes"].copy_(host_boxes, non_blocking=True)
                h2d_done[s].record(copy_stream)
            q, comp_stream = pipes[s % n_pipes], run_streams[s % n_pipes]
            with torch.cuda.stream(comp_stream):
                comp_stream.wait_event(h2d_done[s])
                q.points.copy_(staging[s]["points"], non_blocking=True)
                q.batch.copy_(staging[s]["batch"], non_blocking=True)
                q.scores.copy_(staging[s]["scores"], non_blocking=True)
                q.boxes.copy_(staging[s]["boxes"], non_blocking=True)
                q.replay()
                out_scores[s].copy_(q.nms_scores, non_blocking=True)
                for j, t in enumerate(count_tensors[s % n_pipes]):
                    out_counts[s][j:j + 1].copy_(t, non_blocking=True)
                frame_done[s].record(comp_stream)
        for s in range(min(n, 2)):
            frame_done[s].synchronize()

    fork()
    e2e_loop(args.warmup * fps_step)
    join()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    fork()
    e2e_loop(args.steps * fps_step)
    join()
    f1.record()
    barrier()
    e2e_elapsed = f0.elapsed_time(f1) * 1e-3
    # the results that came back are real: both slots ran the same candidate boxes (same NMS decisions, some boxes
    # suppressed, some kept) and every voxel set of the last two frames is populated
    a, b = out_scores[0].numpy(), out_scores[1].numpy()
    if not ((a == b).all() and (a < 0).any() and (a > 0).any() and (out_counts[0][:len(count_tensors[0])] > 0).all()
            and (out_counts[1][:len(count_tensors[0])] > 0).all()):
        raise RuntimeError("end-to-end results look wrong: NMS scores or voxel counts of the last frames")

    per_rank = gather_ranks([elapsed, e2e_elapsed], dist)  # [rank][which]
    elapsed_all = [r[0] for r in per_rank]
    elapsed, e2e_elapsed = max(elapsed_all), max(r[1] for r in per_rank)

    line = None
    if rank == 0:
        peaks = measured_peaks()
        layers = conv_launch_times(pipe, frames, reps=3)
        tc = layers  # every layer runs the tensor-core kernel (the 5-channel input is zero-padded to 16)
        t_conv = sum(l["seconds"] for l in tc)
        f_dense = sum(l["flops_dense"] for l in tc)
        achieved = f_dense / t_conv / 1e12
        launches_per_frame = count_launches(pipe)
        traffic = conv_dram_bytes_per_frame()
        plugin_order = None
        if world == 1 and not args.no_plugin_order:
            plugin_order = plugin_order_rate(dev, caps, frames, boxes, dev_pts, args)
        ref_gpu = None
        if world == 1 and not args.no_reference_gpu and os.path.exists(os.path.join(ROOT, "oracle", "_ref",
                                                                                  "libref_spconv.so")):
            ref_gpu = reference_gpu_kernels()
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            # a quarter of a frame: some 10-20 s of single-core work, enough to time, short enough for a default run
            fps, dt, _ = cpu_frames_per_second(1, 0.25, 1, 0)
            cpu = {"value": fps, "unit": UNIT, "cores": 1, "kind": "port",
                   "sample": "one 1/4 azimuth sector of a config-4 frame (and 2 of the 10 NMS rows) on one core, "
                             "frames/s = (1/4)/t, t = %.1f s" % dt}
        frames_timed = args.steps * fps_step
        line = {
            "metric": METRIC, "value": aggregate_frames_per_second(world, args.steps, fps_step, elapsed),
            "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16 (fp32 accumulate)",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "frames_per_gpu_per_step": fps_step,
                       "ms_per_frame": elapsed / frames_timed * 1e3,
                       "parallelism": "frame replicas x%d (no collective; ranks meet at host-side barriers only)" % world,
                       "frames_in_flight_per_gpu": n_pipes, "frame_latency_ms": frame_latency_ms,
                       "voxels": {k: int(v) for k, v in pipe.net.counts().items()},
                       "l2": "no flush: a frame rewrites %.0f MB of rulebooks/tables/activations (> 126 MB L2) and "
                             "inputs rotate over %d frames" % (working_set / 1e6, N_ROTATE),
                       "kernel": {0: "auto", 1: "simt", 2: "tcgen05"}[args.kernel],
                       "regrouped_tables": bool(args.regroup),
                       "rank_seconds": {"min": min(elapsed_all), "median": float(np.median(elapsed_all)),
                                        "max": max(elapsed_all)},
                       "outputs": "NMS scores and voxel counts return to the host; the BEV map stays on the device, "
                                  "where the dense head of the engine reads it",
                       "plugin_order": plugin_order, "reference_gpu": ref_gpu},
            "clocks": clocks,
            "e2e": {"value": world * frames_timed / e2e_elapsed, "unit": UNIT, "h2d_bytes_per_step": h2d * fps_step,
                    "d2h_bytes_per_step": d2h * fps_step, "ms_per_step": e2e_elapsed / args.steps * 1e3},
            "gpu_launches": launches_per_frame * frames_timed,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["bf16_tflops"],
                         "traffic": traffic[0] / len(tc) if traffic else None,
                         "traffic_unit": ("bytes per launch (mean of the %d launches of a frame; ncu, L2 flushed before "
                                          "every launch; captured at %s)" % (len(tc), traffic[1])) if traffic else None,
                         "algorithmic_bytes": sum(l["bytes"] for l in tc) / len(tc),
                         "kernel": "SPConvMM (tcgen05) over all %d layers of the backbone, dense-equivalent FLOPs "
                                   "2*M*kVol*Cin*Cout per launch, time = sum of per-launch CUDA-event durations (each layer launched back to back)"
                                   % len(tc),
                         "peak_source": peaks["source"] + ", burst bf16",
                         "useful_tflops": sum(l["flops_pair"] for l in tc) / t_conv / 1e12,
                         "conv_ms_per_frame": t_conv * 1e3},
            "cpu_baseline": cpu,
        }
        if args.layers:
            for l in layers:
                sys.stderr.write("layer %2d  %3d->%3d k%2d  M=%7d P=%8d  %8.1f us  %7.2f TF/s dense  %6.2f TF/s pair\n"
                                 % (l["layer"], l["cin"], l["cout"], l["kvol"], l["m"], l["pairs"], l["seconds"] * 1e6,
                                    l["flops_dense"] / l["seconds"] / 1e12, l["flops_pair"] / l["seconds"] / 1e12))
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return line


METRIC5 = "sparse segmentation frames/s (Cylinder3D-shaped frame, fp16)"
WORKLOAD5 = ("config5: batch of 8 frames x 120000 pts x4 -> CylinderEncoder 480x360x32 -> ScatterTo(max) -> asymmetric "
             "3x1x3/1x3x3 SubM encoder-decoder 32/64/128/256 fp16 -> 20-class logits -> GatherBack -> argmax")
BATCH5 = 8


def run_config5(args):
    """Benchmark config 5: a batch of 8 Cylinder3D-shaped frames sharded over the GPUs (8, 4, 2 or 1 frames per GPU
    and step), one pipeline pair per GPU, no exchange between GPUs.  One step = the whole batch; `value` is the
    whole job's frames per second (strong scaling: the batch is fixed)."""
    import torch
    from deploy3d_b200 import _lib, synth
    from deploy3d_b200.pipeline import SegmentationPipeline
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if BATCH5 % world:
        raise SystemExit("config 5 shards a batch of %d frames: --gpus must divide it" % BATCH5)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    _lib.lib()
    torch.cuda.set_device(local)
    dev = "cuda:%d" % local
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("gloo")
    share = BATCH5 // world
    frames = [synth.config5_points(rank * share + i) for i in range(share)]
    all_frames = frames if world == 1 else [synth.config5_points(i) for i in range(BATCH5)]
    probe = SegmentationPipeline(dev)
    caps = {k: (probe.n_pts if k == "in" else 3 * probe.n_pts) for k in probe.set_names}
    del probe
    probe = SegmentationPipeline(dev, caps=caps, regroup=args.regroup)
    caps = probe.calibrate(all_frames)  # every rank sizes its buffers for the whole batch: identical engines
    del probe
    torch.cuda.empty_cache()
    n_pipes = max(1, args.in_flight)
    pipes = []
    for _ in range(n_pipes):
        q = SegmentationPipeline(dev, caps=caps, regroup=args.regroup)
        q.load_frame(frames[0])
        q.capture()
        pipes.append(q)
    streams = [torch.cuda.Stream(device=dev) for _ in range(n_pipes)]
    main = torch.cuda.current_stream()
    dev_pts = [torch.from_numpy(f["points"]).to(dev) for f in frames]
    host_pts = [torch.from_numpy(f["points"]).pin_memory() for f in frames]
    host_labels = [torch.zeros(pipes[0].n_pts, dtype=torch.int32).pin_memory() for _ in range(2)]
    torch.cuda.synchronize()

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()

    def loop(steps, e2e):
        for st in streams:
            st.wait_stream(main)
        for i in range(steps * share):
            k = i % n_pipes
            with torch.cuda.stream(streams[k]):
                if e2e:
                    pipes[k].points.copy_(host_pts[i % share], non_blocking=True)
                else:
                    pipes[k].points.copy_(dev_pts[i % share], non_blocking=True)
                pipes[k].replay()
                if e2e:
                    host_labels[k % 2].copy_(pipes[k].labels, non_blocking=True)
        for st in streams:
            main.wait_stream(st)

    results = []
    clocks = None
    for e2e in (False, True):
        loop(args.warmup, e2e)
        barrier()
        sampler = ClockSampler(local)
        if rank == 0 and not e2e:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        loop(args.steps, e2e)
        e1.record()
        barrier()
        results.append(e0.elapsed_time(e1) * 1e-3)
        if rank == 0 and not e2e:
            clocks = sampler.stop()
    per_rank = gather_ranks(results, dist)
    elapsed_all = [r[0] for r in per_rank]
    elapsed, e2e_elapsed = max(elapsed_all), max(r[1] for r in per_rank)
    if rank == 0:
        peaks = measured_peaks()
        pipe = pipes[0]
        layers = conv_launch_times(pipe, frames, reps=2)
        t_conv = sum(l["seconds"] for l in layers)
        achieved = sum(l["flops_dense"] for l in layers) / t_conv / 1e12
        labels = host_labels[0].numpy()
        if not (labels.max() > 0 and labels.min() >= 0 and labels.max() < pipe.n_class):
            raise RuntimeError("end-to-end labels look wrong")
        line = {
            "metric": METRIC5, "value": BATCH5 * args.steps / elapsed, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed / args.steps * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp16 (fp32 accumulate)",
            "data": "synthetic",
            "config": {"workload": WORKLOAD5, "frames_per_gpu_per_step": share, "batch": BATCH5,
                       "ms_per_frame_per_gpu": elapsed / (args.steps * share) * 1e3,
                       "parallelism": "batch of %d frames sharded %d per GPU (no collective)" % (BATCH5, share),
                       "frames_in_flight_per_gpu": n_pipes,
                       "voxels": {k: int(v) for k, v in pipe.net.counts().items()},
                       "conv_layers": len(layers), "regrouped_tables": bool(args.regroup),
                       "rank_seconds": {"min": min(elapsed_all), "median": float(np.median(elapsed_all)),
                                        "max": max(elapsed_all)}},
            "clocks": clocks,
            "e2e": {"value": BATCH5 * args.steps / e2e_elapsed, "unit": UNIT,
                    "h2d_bytes_per_step": host_pts[0].numel() * 4 * share,
                    "d2h_bytes_per_step": host_labels[0].numel() * 4 * share,
                    "ms_per_step": e2e_elapsed / args.steps * 1e3},
            "gpu_launches": count_launches(pipes[0], "segmentation") * args.steps * share,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["bf16_tflops"], "traffic": None,
                         "algorithmic_bytes": sum(l["bytes"] for l in layers) / len(layers),
                         "kernel": "SPConvMM (tcgen05) over the %d convolution layers of the network, dense-equivalent "
                                   "FLOPs, time = sum of per-launch CUDA-event durations" % len(layers),
                         "peak_source": peaks["source"] + ", burst bf16",
                         "useful_tflops": sum(l["flops_pair"] for l in layers) / t_conv / 1e12,
                         "conv_ms_per_frame": t_conv * 1e3},
            "cpu_baseline": None,
        }
        if args.layers:
            for l in layers:
                sys.stderr.write("layer %2d  %3d->%3d k%2d  M=%7d P=%8d  %8.1f us  %7.2f TF/s dense  %6.2f TF/s pair\n"
                                 % (l["layer"], l["cin"], l["cout"], l["kvol"], l["m"], l["pairs"], l["seconds"] * 1e6,
                                    l["flops_dense"] / l["seconds"] / 1e12, l["flops_pair"] / l["seconds"] / 1e12))
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def plugin_order_rate(dev, caps, frames, boxes, dev_pts, args):
    """What a TensorRT engine built from the reference's graph would get from this library: ONE pipeline on ONE
    stream, every node in ONNX order through the plugin-level entry points only (d3d_spconv_index_enqueue once per
    rulebook, d3d_spconv_mm_enqueue per layer -- which rebuilds its neighbour table in its own workspace every
    time --, ReLU / residual add as separate element-wise kernels, NMS after the backbone), captured in a CUDA graph
    with programmatic dependent launch on.  Frames per second with the inputs resident in HBM."""
    import torch
    from deploy3d_b200.pipeline import DetectionPipeline
    q = DetectionPipeline("centerpoint", dev, caps=caps, kernel=args.kernel, plugin_order=True)
    q.load_frame(frames[0], boxes)
    q.capture()
    n = max(20, min(args.steps * FRAMES_PER_STEP, 100))
    for i in range(5):
        q.points.copy_(dev_pts[i % N_ROTATE], non_blocking=True)
        q.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
        q.points.copy_(dev_pts[i % N_ROTATE], non_blocking=True)
        q.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    del q
    torch.cuda.empty_cache()
    return {"frames_per_s": 1e3 / ms, "ms_per_frame": ms, "frames": n,
            "what": "one pipeline, one stream, plugin-level enqueue of every node in graph order (neighbour table "
                    "rebuilt by each of the 21 SPConvMM nodes), separate ReLU / add kernels, CUDA graph, dependent launch"}


def gather_ranks(values, dist):
    """[rank][i] of `values` from every rank (identity without a process group).  The frames are independent
    replicas: this exchange of timings is the only inter-rank traffic, and it goes over the host."""
    if dist is None:
        return [[float(v) for v in values]]
    import torch
    mine = torch.tensor([float(v) for v in values], dtype=torch.float64)
    out = [torch.zeros_like(mine) for _ in range(dist.get_world_size())]
    dist.all_gather(out, mine)
    return [[float(v) for v in t] for t in out]


def aggregate_frames_per_second(world, steps, frames_per_step, elapsed_max):
    """Whole-job throughput: every rank processed steps x frames_per_step frames within the slowest rank's time."""
    return world * steps * frames_per_step / elapsed_max


def count_launches(pipe, kind="detection"):
    """Kernels of this library launched per frame, counted from the pipeline's plan (every enqueue is a fixed launch
    list: 105 launches per config-4 frame, as a profiler's launch list of this script shows)."""
    net = pipe.net
    n = 0
    for rb in net.rulebooks.values():
        # SubM: reset, insert, probe, segment scan, compact, padding fill; strided: reset, insert, count winners,
        # scan, assign, translate, segment scan, compact, padding fill
        n += 6 if rb.kind == "subm" else 9
        if not getattr(rb, "fused_table", False):
            n += 3  # neighbour table: fill, scatter, offset masks
        if getattr(rb, "table_inv", None) is not None:
            n += 3  # the inverse layers' table of the same rulebook
    n += sum(1 for L in net.layers if L.kind != "ew")  # SPConvMM
    if kind == "detection":
        n += 7  # SimpleMeanEncoder: reset, voxelize, owners, scan, number, accumulate, divide
        n += 3  # BEVDensify: map fill, map scatter, densify
        n += 2  # NMS3d: overlap mask, suppression
    else:
        n += 6  # CylinderEncoder: reset, cylinderize, owners, scan, number, scatter ids
        n += 2  # ScatterTo: fill, scatter-reduce
        n += 1  # GatherBack
    return n


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20, help="timed steps of %d frames per GPU each" % FRAMES_PER_STEP)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="config4", choices=["config4", "config5"],
                    help="config4: the headline CenterPoint-shaped frame; config5: the Cylinder3D-shaped batch of 8 "
                         "frames sharded over the GPUs (this implementation only)")
    ap.add_argument("--kernel", type=int, default=0, help="SPConvMM kernel: 0 auto, 1 SIMT, 2 tcgen05")
    ap.add_argument("--in-flight", type=int, default=2,
                    help="pipelines (buffers + CUDA graph + stream each) that take the frames in turn")
    ap.add_argument("--layers", action="store_true", help="print the per-layer SPConvMM table to stderr")
    ap.add_argument("--tc-plan", type=int, nargs=3, default=None, metavar=("GROUP", "STAGES", "PRODUCER_WARPS"),
                    help="override the tensor-core kernel's pipeline plan for every layer (0 = automatic)")
    ap.add_argument("--regroup", action="store_true",
                    help="rebuild every neighbour table with its outputs grouped by offset mask (d3d_spconv_mm_regroup): "
                         "fewer (tile, offset) blocks for the convolutions, three more kernels per rulebook")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-plugin-order", action="store_true", help="skip the single-stream plugin-order figure")
    ap.add_argument("--no-reference-gpu", action="store_true",
                    help="skip timing the reference's CUDA kernels (oracle/_ref) beside this library's")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "config5":
        run_config5(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
