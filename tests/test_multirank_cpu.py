"""The multi-GPU path is frame replication: ranks never exchange data, only the timings are gathered over the host
(the slowest rank decides) and the frame counts summed.  That host logic -- the very gloo group bench.py uses --
is exercised here with two ranks on the CPU."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys, json
    sys.path.insert(0, %r)
    import torch.distributed as dist
    import bench
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    # rank r pretends its timed region took (1 + r) seconds device-side and (2 + 3 r) seconds end to end
    per_rank = bench.gather_ranks([1.0 + rank, 2.0 + 3 * rank], dist)
    elapsed, e2e = max(r[0] for r in per_rank), max(r[1] for r in per_rank)
    fps = bench.aggregate_frames_per_second(world, steps=10, frames_per_step=bench.FRAMES_PER_STEP,
                                            elapsed_max=elapsed)
    dist.barrier()
    if rank == 0:
        print(json.dumps({"elapsed": elapsed, "e2e": e2e, "fps": fps, "world": world,
                          "fastest": min(r[0] for r in per_rank)}))
    dist.destroy_process_group()
""") % ROOT


def test_timings_reduce_to_the_slowest_rank(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                         capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    import json
    line = [ln for ln in out.stdout.splitlines() if ln.startswith("{")][-1]
    got = json.loads(line)
    assert got == {"elapsed": 2.0, "e2e": 5.0, "fps": 100.0, "world": 2, "fastest": 1.0}


def test_single_rank_is_identity():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.gather_ranks([1.5, 2.5], None) == [[1.5, 2.5]]
    assert bench.aggregate_frames_per_second(1, 20, 1, 0.5) == 40.0


def test_reference_arm_other_ranks_exit_quietly():
    """Under torchrun only rank 0 runs the CPU arm; the others print nothing and exit 0."""
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=120, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""
