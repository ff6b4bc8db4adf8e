"""TEST INFRASTRUCTURE ONLY.  Times the REFERENCE's own NumPy tools (tools/reference_all_layers.py: first token, position 0,
every matrix dequantised on every call) where the reference checkout is mounted, on the seeded 4-layer full-size synthetic
checkpoint (layers 0-2 DeltaNet, layer 3 attention), and extrapolates to the 32-layer model (24 DeltaNet + 8 attention
blocks; the tool has no lm_head).  The reference tools cannot travel to the GPU box, so the figure is recorded in the
repository's baseline notes together with the core count printed here.

    python oracle/time_reference_tools.py --reference /path/to/insignia
"""
import argparse
import os
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from insignia_b200 import synth  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    src = open(os.path.join(args.reference, "tools", "reference_all_layers.py")).read()
    prefix = src.split("x=dq('language_model.model.embed_tokens')[42]")[0]
    with tempfile.TemporaryDirectory() as tmp:
        st = os.path.join(tmp, "golden4.safetensors")
        synth.write_checkpoint(synth.SynthConfig(layers=(0, 1, 2, 3), vocab_rows=64, mtp=False, lm_head=True, seed=7, norms="random"), st)
        ns = {}
        old = sys.argv
        sys.argv = ["reference_all_layers.py", st]
        try:
            exec(compile(prefix, "reference_all_layers.py(prefix)", "exec"), ns)
        finally:
            sys.argv = old
        ns["states"] = [np.zeros((32, 128, 128), np.float32) for _ in range(24)]
        x = ns["dq"]("language_model.model.embed_tokens")[42]
        times = []
        for l in range(4):
            t0 = time.perf_counter()
            x = ns["attn"](x, l) if l % 4 == 3 else ns["delta"](x, l)
            times.append(time.perf_counter() - t0)
        # pre-dequantised variant of the same arithmetic: the matrix products alone (what remains when dq() is hoisted)
        w = ns["dq"]("language_model.model.layers.0.mlp.gate_proj")
        t0 = time.perf_counter()
        for _ in range(5):
            w @ x
        matvec = (time.perf_counter() - t0) / 5
    delta, attn = float(np.mean(times[:3])), times[3]
    total = 24 * delta + 8 * attn
    print(f"cores {os.cpu_count()}  numpy {np.__version__}")
    print(f"DeltaNet block {delta:.3f} s, attention block {attn:.3f} s (per-call dequantisation, as the tool does)")
    print(f"32 layers, first token: {total:.1f} s = {1.0 / total:.4f} tok/s (no lm_head in the tool)")
    print(f"pre-dequantised 12288 x 4096 fp32 matvec: {matvec * 1e3:.2f} ms")


if __name__ == "__main__":
    main()
