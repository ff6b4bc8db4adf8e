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


def test_tensor_parallel_shards_add_up_to_the_block():
    """bench.tp_shards: rows of gate|up and the matching columns of down per rank; the ranks' partial outputs, summed in
    rank order (what the one-shot all-reduce does), are the unsharded MLP block.  CPU oracle arithmetic, two ranks."""
    import numpy as np

    sys.path.insert(0, ROOT)
    import bench
    from oracle import oracle as orc

    x = np.random.default_rng(5).standard_normal(4096).astype(np.float32)

    def mlp(gate, up, down, cols):
        g, u = orc.gemv_mlx(gate[0], gate[1], x), orc.gemv_mlx(up[0], up[1], x)
        act = (g / (1 + np.exp(-g)) * u).astype(np.float32)
        assert act.shape[0] == cols
        return orc.gemv_mlx(down[0], down[1], act)

    parts, full = [], None
    for rank in range(2):
        full, shard, per = bench.tp_shards(rank, 2, seed=3)
        assert per == 6144 and shard["gate"][0].shape == (6144, 512) and shard["down"][0].shape == (4096, 768) and shard["down"][1].shape == (4096, 192)
        parts.append(mlp(shard["gate"], shard["up"], shard["down"], per))
    want = mlp(full["gate"], full["up"], full["down"], 12288)
    got = (parts[0] + parts[1]).astype(np.float32)
    assert np.max(np.abs(got - want)) <= 1e-5 * np.abs(want).max()
