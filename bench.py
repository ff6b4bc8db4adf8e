#!/usr/bin/env python3
"""Decode benchmark: batch-1 greedy tok/s of the 32-layer MXFP4 hybrid on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (BASELINE.json configs[3]): the full 32-layer model (24 gated-DeltaNet + 8 gated-GQA
layers, hidden 4096, FFN 12288, vocab 248320), every linear weight MXFP4 quantised from seeded
N(0, 0.02); a 512-token prompt of seeded uniform-random ids is ingested token by token (the
reference has no prefill: src/generate_ids.cu:4), then tokens are decoded greedily.  A "step" is
one decoded token = one pass of the hot path.  Weights are synthetic (the real checkpoint is not
available offline) and are written to a RAM-backed file once, then loaded through the same
ModelFile -> TieredStorage path a real checkpoint takes.

* ``value``  tok/s with everything resident in HBM: K tokens generated back to back with the
  arg-max fed back on the device (Qwen35Decode::generate), CUDA events on the engine's stream.
* ``e2e``    tok/s through the reference-facing call Qwen35Decode::decode_token(int) -> int: the
  token id goes host -> device and the result device -> host every step.
* ``roofline``  the fused GEMV kernel: algorithmic weight bytes per launch / its mean launch
  duration, taken from one eager step with a CUDA-event pair around every launch, against the
  measured HBM copy bandwidth of MEASURED_PEAKS.json.
* ``cpu_baseline``  the CPU oracle port (oracle/, C + OpenMP) decoding a few tokens of the same
  model on the host cores.

N > 1 (torchrun): independent replicas, one per GPU, no collective on the data path; ``value`` is
the sum over ranks divided by the slowest rank's time (weak scaling).

``--impl reference`` runs the reference's own engine: its unmodified CUDA sources compiled for
sm_100a under oracle/_ref (see oracle/Makefile), driven through its public decode_token loop on the
same checkpoint and prompt.  If that library is absent it falls back to the CPU oracle port.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

HIDDEN, VOCAB = 4096, 248320
WEIGHT_BYTES_PER_TOKEN = 4_217_924_096  # 24 DeltaNet + 8 attention layers + lm_head, 17 bytes / 32 weights
STATE_BYTES_PER_TOKEN = 24 * 2 * (32 * 128 * 128 * 4 + 8192 * 3 * 4)
# dram__bytes_read+write of the GEMV kernel / its algorithmic bytes, from the ncu capture summarised in
# profiles/gemv_fused_kernel_65536x4096.md (scaled per launch by the bytes processed)
GEMV_TRAFFIC_RATIO = 1.03


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--kv-bf16", action="store_true", help="bf16 KV cache (the default is the reference's fp32 cache)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gemv", default="mma", choices=["mma", "tcgen05"], help="GEMV kernel family of the engine")
    ap.add_argument("--tune", action="append", default=[], help="kernel tuning knob key=value (insg_tune_set)")
    ap.add_argument("--persistent", action="store_true", help="the persistent token kernel (one cooperative launch per token) instead of the graph of launches")
    ap.add_argument("--prefetch", type=int, default=-1, help="persistent kernel: weight records per warp kept prefetched into L2 (-1 = default)")
    return ap.parse_args()


def workdir() -> str:
    for base in ("/dev/shm", "/tmp"):
        try:
            if shutil.disk_usage(base).free > (8 << 30):
                d = os.path.join(base, "insignia_b200_bench")
                os.makedirs(d, exist_ok=True)
                return d
        except OSError:
            pass
    raise RuntimeError("no scratch directory with 8 GiB free")


def ensure_checkpoint(seed: int, use_cuda: bool) -> tuple[str, str]:
    from insignia_b200 import synth

    d = workdir()
    st, idx = os.path.join(d, f"qwen35_synth_seed{seed}.safetensors"), os.path.join(d, f"qwen35_synth_seed{seed}.idx")
    if not (os.path.exists(st) and os.path.exists(idx)):
        tmp = st + ".tmp"
        cfg = synth.SynthConfig(seed=seed, norms="ones", backend="torch" if use_cuda else "numpy")
        synth.write_checkpoint(cfg, tmp)
        os.replace(tmp, st)
        from insignia_b200.checkpoint_io import write_index

        write_index(st, idx)
    return st, idx


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu: int):
        self.gpu, self.rows, self.proc = gpu, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            self.t.join(timeout=2)

    def summary(self) -> dict:
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def measured_hbm_peak() -> tuple[float, str]:
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def cpu_port_baseline(st_path: str, prompt: np.ndarray, budget_s: float = 20.0) -> dict:
    """Times the CPU oracle port on the first tokens of the same workload (all host threads)."""
    from insignia_b200.checkpoint_io import SafetensorsReader
    from oracle import oracle as orc

    m = orc.OracleModel(SafetensorsReader(st_path), max_context=64, gate="broadcast", fast_gemv=True)
    t0 = time.perf_counter()
    m.decode_token(int(prompt[0]))
    t1 = time.perf_counter() - t0
    n = int(max(1, min(8, budget_s / max(t1, 1e-3))))
    t0 = time.perf_counter()
    for i in range(n):
        m.decode_token(int(prompt[1 + i]))
    dt = time.perf_counter() - t0
    return {"value": n / dt, "unit": "tok/s", "cores": orc.num_threads(), "kind": "port",
            "sample": f"{n} greedy tokens of the full 32-layer model from position 1 (after one warm-up token)"}


def run_native(args, rank, world, local_rank):
    import torch

    from insignia_b200.engine import Engine

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if rank == 0:
        st, idx = ensure_checkpoint(args.seed, True)
    if dist:
        dist.barrier()
    st, idx = ensure_checkpoint(args.seed, True)

    K, W = args.steps, args.warmup
    ctx = args.prompt + W + 2 * K + 32
    from insignia_b200 import ops

    for kv in args.tune:
        k, v = kv.split("=")
        ops.tune(k, int(v))
    eng = Engine(idx, max_context=ctx, budget_bytes=16 << 30, kv_bf16=args.kv_bf16, device=local_rank, gemv_tcgen05=args.gemv == "tcgen05",
                 persistent=args.persistent)
    if args.prefetch >= 0:
        eng.set_program_option("prefetch_records", args.prefetch)
    rng = np.random.default_rng(args.seed + 1000 * rank)
    prompt = rng.integers(0, VOCAB, args.prompt)
    stream = torch.cuda.ExternalStream(eng.stream, device=local_rank)
    # the prompt goes in by forward_tokens (not part of the metric; reported as "prefill")
    PRE = 40 if args.prompt >= 80 else min(8, args.prompt - 1)
    eng.forward_tokens([int(t) for t in prompt[:PRE]])  # loads and repacks every weight, in both layouts
    torch.cuda.synchronize()
    pa, pb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pa.record(stream)
    eng.forward_tokens([int(t) for t in prompt[PRE:]])
    pb.record(stream)
    torch.cuda.synchronize()
    prefill_ms = pa.elapsed_time(pb)
    tok = eng.logits_argmax()

    def timed(fn):
        if dist:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        out = fn()
        b.record(stream)
        torch.cuda.synchronize()
        ms = torch.tensor([a.elapsed_time(b)], device="cuda")
        if dist:
            dist.barrier()
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), out

    if W > 0:
        tok = eng.generate(tok, W)[-1]
    with ClockSampler(local_rank) as clocks:
        l0 = eng.launch_count
        ms, toks = timed(lambda: eng.generate(tok, K))
        launches = eng.launch_count - l0
        tok = toks[-1]

        def e2e_loop():
            t = tok
            for _ in range(K):
                t = eng.decode_token(t)
            return t

        ms_e2e, tok = timed(e2e_loop)
    final_ctx = eng.position
    # the dominant kernel in its own flow: the token's fused-GEMV launches alone, replayed as a graph between two events
    chain = eng.profile_gemv_chain(replays=8)
    gemv = {"bytes": chain["bytes"], "ms": chain["ms_per_token"], "launches": chain["launches"]}
    peak, peak_kind = measured_hbm_peak()
    gemv_gbs = gemv["bytes"] / (gemv["ms"] * 1e-3) / 1e9
    kv_bytes = 8 * 1024 * 2 * (2 if args.kv_bf16 else 4) * (args.prompt + W + K // 2)
    token_bytes = WEIGHT_BYTES_PER_TOKEN + STATE_BYTES_PER_TOKEN + kv_bytes
    value = world * K / (ms * 1e-3)
    out = {
        "metric": "9B MXFP4 hybrid decode tok/s (bs1)", "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "impl": "native",
        "config": {"workload": "configs[3]: 32-layer hybrid (24 DeltaNet + 8 GQA), MXFP4 weights, batch-1 greedy decode after a "
                               f"{args.prompt}-token prompt", "prompt_tokens": args.prompt, "context_at_end": final_ctx,
                   "kv_cache": "bf16" if args.kv_bf16 else "f32", "gemv": args.gemv, "tune": args.tune, "weights": "seeded N(0,0.02) -> MXFP4, norms 1.0",
                   "parallelism": f"replica x{world}" if world > 1 else "single GPU",
                   "l2": "weights streamed per token (4.2 GB) exceed the 126 MB L2; no flush needed"},
        "e2e": {"value": world * K / (ms_e2e * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 4},
        "gpu_launches": int(launches),
        "token_hbm": {"algorithmic_bytes_per_token": token_bytes, "achieved_gbs": token_bytes / (ms / K * 1e-3) / 1e9,
                      "frac_of_measured_peak": token_bytes / (ms / K * 1e-3) / 1e9 / peak,
                      "frac_of_8tbs": token_bytes / (ms / K * 1e-3) / 1e9 / 8000.0},
        "roofline": {"bound": "hbm", "kernel": "gemv_fused_kernel", "achieved": gemv_gbs, "peak": peak, "unit": "GB/s",
                     "frac": gemv_gbs / peak, "traffic": gemv["bytes"] / gemv["launches"] * GEMV_TRAFFIC_RATIO,
                     "peak_source": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs, burst copy)",
                     "bytes_per_launch": gemv["bytes"] / gemv["launches"], "us_per_launch": gemv["ms"] * 1e3 / gemv["launches"],
                     "launches_per_token": gemv["launches"],
                     "timing": "CUDA events around 8 replays of a graph holding only this kernel's launches of one token "
                               "(dependent-launch overlap on, weights exceed L2)"},
        "clocks": clocks.summary(),
        "prefill": {"value": world * (args.prompt - PRE) / (prefill_ms * 1e-3), "unit": "tok/s", "tokens": args.prompt - PRE,
                    "how": "forward_tokens: passes of up to 32 tokens through the tcgen05 kernel (eight tokens per kind::mxf4 "
                           "instruction), DeltaNet and attention steps token by token; outside the timed metric"},
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_port_baseline(st, prompt)
    eng.close()
    if rank == 0:
        print(json.dumps(out), flush=True)
    if dist:
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args, rank, world, local_rank):
    if rank != 0:
        return  # the reference is single-GPU, single-sequence: rank 0 alone runs it
    K, W = args.steps, args.warmup
    rng = np.random.default_rng(args.seed)
    prompt = rng.integers(0, VOCAB, args.prompt)
    base = {"metric": "9B MXFP4 hybrid decode tok/s (bs1)", "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "impl": "reference"}
    from oracle import ref_engine

    if ref_engine.available():
        import torch

        torch.cuda.set_device(local_rank)
        st, idx = ensure_checkpoint(args.seed, True)
        eng = ref_engine.RefEngine(idx, max_context=args.prompt + W + K + 8, budget=16 << 30)
        for t in prompt:
            eng.forward_token(int(t))
        tok = eng.logits_argmax()
        for _ in range(W):
            tok = eng.decode_token(tok)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as clocks:
            a.record()
            for _ in range(K):
                tok = eng.decode_token(tok)
            b.record()
            torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        eng.close()
        v = K / (ms * 1e-3)
        base.update({"value": v, "ms_per_step": ms / K, "clocks": clocks.summary(),
                     "config": {"workload": "configs[3]: same checkpoint, prompt and decode loop through the reference's "
                                            "Qwen35Decode::decode_token (src/decode.cu:23)", "prompt_tokens": args.prompt,
                                "engine": "reference CUDA sources, unmodified, compiled for sm_100a with its own flags "
                                          "(-O3 --use_fast_math), run on this GPU"},
                     "cpu_baseline": {"value": v, "unit": "tok/s", "cores": 1, "kind": "reference",
                                      "sample": f"{K} greedy tokens after a {args.prompt}-token prompt; one host thread drives "
                                                "the reference's GPU kernels (it has no multi-token CPU path)"},
                     "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    else:
        st, idx = ensure_checkpoint(args.seed, False)
        cb = cpu_port_baseline(st, prompt)
        base.update({"value": cb["value"], "ms_per_step": 1e3 / cb["value"], "cpu_baseline": cb,
                     "config": {"workload": "configs[3] on the CPU oracle port (oracle/_ref not built)", "prompt_tokens": 0},
                     "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    print(json.dumps(base), flush=True)


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world, local_rank)
    else:
        run_native(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
