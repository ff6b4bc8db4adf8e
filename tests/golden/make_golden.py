"""Generates the golden vectors under tests/golden/ by running the REFERENCE's own NumPy tools.

Run where the reference checkout is mounted:

    python tests/golden/make_golden.py --reference /path/to/reference-checkout

It writes a seeded 4-layer synthetic checkpoint (the model's layers 0-3: three
DeltaNet blocks and one attention block, full-size matrices, 64 embedding rows),
imports the functions of ``tools/reference_all_layers.py`` exactly the way the
reference's own ``tools/reference_attention_seams.py:1`` does (exec of the file
up to its driver line) and stores what they return for token 42 at position 0:

* ``layers_tok42.npy``   fp32 [4][4096]: residual stream after layers 0..3
* ``index_small.bin`` / ``index_small.json``: the INSIDX01 index written by the
  reference's ``tools/index_safetensors.py`` for a tiny safetensors file, and that
  file's header, for the index-format test.

The checkpoint itself is NOT committed: tests regenerate it bit-identically from
the same seed (numpy Generator streams are platform independent).
"""
import argparse
import json
import os
import runpy
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from insignia_b200 import synth  # noqa: E402

GOLDEN_CFG = dict(layers=(0, 1, 2, 3), vocab_rows=64, mtp=False, lm_head=True, seed=7, norms="random")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    args = ap.parse_args()
    tools = os.path.join(args.reference, "tools")
    with tempfile.TemporaryDirectory() as tmp:
        st = os.path.join(tmp, "golden4.safetensors")
        synth.write_checkpoint(synth.SynthConfig(**GOLDEN_CFG), st)
        src = open(os.path.join(tools, "reference_all_layers.py")).read()
        prefix = src.split("x=dq('language_model.model.embed_tokens')[42]")[0]
        ns = {}
        old_argv = sys.argv
        sys.argv = ["reference_all_layers.py", st]
        try:
            exec(compile(prefix, "reference_all_layers.py(prefix)", "exec"), ns)
        finally:
            sys.argv = old_argv
        ns["states"] = [np.zeros((32, 128, 128), np.float32) for _ in range(24)]
        x = ns["dq"]("language_model.model.embed_tokens")[42]
        out = []
        for l in range(4):
            x = ns["attn"](x, l) if l % 4 == 3 else ns["delta"](x, l)
            out.append(np.asarray(x, np.float32))
        np.save(os.path.join(HERE, "layers_tok42.npy"), np.stack(out))
        print("layers_tok42.npy", np.stack(out).shape, [float(np.abs(o).max()) for o in out])

        # index-format fixture from the reference's own index builder
        small = os.path.join(tmp, "small.safetensors")
        cfg = synth.SynthConfig(layers=(), vocab_rows=32, mtp=False, lm_head=False, seed=1)
        synth.write_checkpoint(cfg, small)
        idx = os.path.join(tmp, "small.idx")
        subprocess.check_call([sys.executable, os.path.join(tools, "index_safetensors.py"), small, idx])
        blob = open(idx, "rb").read()
        # the index embeds the absolute payload path; store it with a placeholder so the fixture is location-free
        real = os.path.realpath(small).encode()
        assert blob.count(real) == 1
        open(os.path.join(HERE, "index_small.bin"), "wb").write(blob.replace(real, b"@PAYLOAD@"))
        import struct

        with open(small, "rb") as f:
            (n,) = struct.unpack("<Q", f.read(8))
            header = json.loads(f.read(n))
        json.dump({"header": header, "header_len": n, "path_len": len(real)}, open(os.path.join(HERE, "index_small.json"), "w"),
                  indent=1, sort_keys=True)
        print("index_small.bin", len(blob))


if __name__ == "__main__":
    main()
