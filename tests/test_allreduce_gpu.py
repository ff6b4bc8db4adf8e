"""The one-shot all-reduce over peer memory (insg_comm_*, insg_allreduce_oneshot*).

On one GPU all ranks of a communicator run as one cooperative launch (kernels that wait on one another may not be
separate launches on one GPU); with two or more GPUs the real form is also run: one process per GPU, exchange buffers
mapped through CUDA IPC, one kernel per rank, checked against torch.distributed's all-reduce.  The failure-detection
test makes a wait run out on a flag that nothing sets (a silent rank) and reads the status; nothing is hung or faulted.
"""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

ROOT = os.path.join(os.path.dirname(__file__), "..")
sys.path.insert(0, ROOT)

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def rank_order_sum(xs):
    acc = np.zeros_like(xs[0])
    for x in xs:
        acc = (acc + x).astype(np.float32)
    return acc


@pytest.mark.parametrize("world,count", [(2, 4096), (4, 4096), (8, 4096), (8, 1000), (3, 12288), (1, 64)])
def test_local_ranks_sum_in_rank_order(cuda, world, count):
    from insignia_b200 import ops

    rng = np.random.default_rng(world * 100 + count)
    comms = ops.Comm.local(world, 12288)
    try:
        for call in range(5):  # both slot sets, several epochs
            xs = [(rng.standard_normal(count) * 10 ** rng.uniform(-3, 3)).astype(np.float32) for _ in range(world)]
            ts = [torch.from_numpy(x).cuda() for x in xs]
            ops.Comm.allreduce_local(comms, ts, count)
            want = rank_order_sum(xs)
            for t in ts:  # bit-identical on every rank, and to the sum in rank order
                assert np.array_equal(t.cpu().numpy(), want), call
        assert all(c.error() == 0 for c in comms)
    finally:
        for c in comms:
            c.close()


def test_silent_rank_makes_the_wait_run_out(cuda):
    from insignia_b200 import ops

    comms = ops.Comm.local(3, 4096)
    try:
        for c in comms:
            c.set_timeout(2_000_000)  # 2 ms
        ts = [torch.ones(4096, device="cuda") for _ in range(3)]
        ops.Comm.allreduce_local(comms, ts, 4096, skip_rank=1)  # rank 1 never raises its flags
        torch.cuda.synchronize()
        assert comms[0].error() == 1 and comms[2].error() == 1 and comms[1].error() == 0
        # the context is still usable: reset every rank, and the next call is right
        for c in comms:
            c.reset()
        ts = [torch.full((4096,), float(r + 1), device="cuda") for r in range(3)]
        ops.Comm.allreduce_local(comms, ts, 4096)
        assert all(c.error() == 0 for c in comms) and all(bool((t == 6).all()) for t in ts)
    finally:
        for c in comms:
            c.close()


def test_argument_checks(cuda):
    from insignia_b200 import ops

    with pytest.raises(RuntimeError, match="world"):
        ops.Comm(0, 9, 4096)
    c = ops.Comm(0, 2, 4096)
    try:
        with pytest.raises(Exception, match="not connected"):
            c.allreduce(torch.zeros(4096, device="cuda"))
    finally:
        c.close()
    comms = ops.Comm.local(2, 4096)
    try:
        with pytest.raises(Exception, match="multiple of 4"):
            ops.Comm.allreduce_local(comms, [torch.zeros(4098, device="cuda")] * 2, 4098)
    finally:
        for c in comms:
            c.close()


WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, %r)
    import numpy as np, torch, torch.distributed as dist
    from insignia_b200 import ops
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    comm = ops.Comm(rank, world, 4096)
    mine = torch.frombuffer(bytearray(comm.handle()), dtype=torch.uint8).cuda()
    every = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(every, mine)
    comm.connect([bytes(h.cpu().numpy().tobytes()) for h in every])
    ok = True
    for call in range(6):
        g = torch.Generator(device="cuda").manual_seed(1000 * call + rank)
        x = torch.randn(4096, device="cuda", generator=g)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        want = torch.zeros_like(x)
        for q in range(world):
            want = want + parts[q]          # rank order
        got = comm.allreduce(x.clone())
        torch.cuda.synchronize()
        ok = ok and bool(torch.equal(got, want))
    ok = ok and comm.error() == 0
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    if rank == 0:
        print("ALLREDUCE_OK" if int(flag.item()) == 1 else "ALLREDUCE_MISMATCH")
""") % os.path.abspath(ROOT)


def test_two_processes_two_gpus(cuda, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                          "--master-port", "29541", str(script)], capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "ALLREDUCE_OK" in out.stdout, out.stdout[-2000:]
