"""World-size-2 gloo run of the benchmark's replica logic on CPU (no GPU), through bench.py's own functions: per-rank
prompts differ by rank, the step time is the maximum over ranks and the job throughput is the sum of the replicas' tokens
over it."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys, json
    sys.path.insert(0, %r)
    import numpy as np, torch, torch.distributed as dist
    import bench                                           # the benchmark's own helpers, not a copy of them
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    prompt = bench.prompt_for_rank(0, rank, 16)
    ms = bench.max_over_ranks(10.0 * (rank + 1), dist, "cpu")   # rank 1 is the slow replica
    gathered = [None] * world
    dist.all_gather_object(gathered, prompt.tolist())
    if rank == 0:
        K = 8
        print(json.dumps({"ms": ms, "value": bench.job_throughput(world, K, ms), "distinct": gathered[0] != gathered[1],
                          "rank0_is_reference_prompt": gathered[0] == bench.prompt_for_rank(0, 0, 16).tolist()}))
    dist.barrier()
    dist.destroy_process_group()
""") % ROOT


def test_replica_timing_is_max_over_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                          "--master-port", "29533", str(script)], capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    import json

    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    r = json.loads(line)
    assert r["ms"] == 20.0 and abs(r["value"] - 2 * 8 / 0.020) < 1e-6 and r["distinct"] and r["rank0_is_reference_prompt"]


def test_reference_arm_runs_on_rank0_only():
    """bench.py --impl reference under a 2-rank launch: rank 1 exits 0 without work."""
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"], capture_output=True,
                         text=True, env=env, timeout=120)
    assert out.returncode == 0 and out.stdout.strip() == ""
