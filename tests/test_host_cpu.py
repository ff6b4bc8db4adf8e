"""Host-side logic that needs no GPU: file formats, quantiser, library symbols, C-ABI argument checks."""
import ctypes as C
import json
import os
import re
import struct
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_library_exports_every_declared_symbol():
    from insignia_b200 import _lib

    header = open(os.path.join(ROOT, "include", "insignia_b200.h")).read()
    declared = set(re.findall(r"INSG_API[^;]*?\b(insg_\w+)\s*\(", header))
    assert len(declared) >= 45
    L = _lib.lib()
    for name in declared:
        assert hasattr(L, name), name
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert L.insg_version() == 100


def test_cabi_rejects_bad_arguments_without_gpu():
    from insignia_b200 import _lib

    L = _lib.lib()
    assert L.insg_mxfp4_packed_bytes(4096, 4096) == 4096 * 4096 * 17 // 32
    assert L.insg_mxfp4_packed_bytes(4097, 4096) == 0 and L.insg_mxfp4_packed_bytes(4096, 4100) == 0
    assert L.insg_mxfp4_gemv_mlx(None, None, None, None, 16, 4096, None) == -3
    assert L.insg_mxfp4_gemv_mlx(1, 1, 1, 1, 16, 4097, None) == -1
    assert b"cols" in L.insg_last_error()
    assert L.insg_gemv_fused(None, None) == -3
    assert L.insg_deltanet_decode(None, None, None, None, None, None, None, 0, None) == -3
    assert L.insg_gqa_decode(None, None, None, None, 0, 0, None, 0, None) == 0  # tokens <= 0 returns silently (src/attention.cu:5)
    assert L.insg_gqa_decode(None, None, None, None, 5, 0, None, 0, None) == -3
    assert L.insg_tune_set(b"nonsense", 1) == -3
    assert L.insg_engine_create(b"/nonexistent/index", None) is None
    assert b"cannot open Insignia index" in L.insg_last_error()


def test_quantiser_round_trip_and_ties():
    from insignia_b200 import mxfp4

    v = np.zeros((1, 32), np.float32)
    v[0, :16] = [0, .25, .75, 1.25, 1.75, 2.5, 3.5, 5, 6, 7.9, -0.25, -0.75, -5, -6, 0.26, 0.74]
    v[0, 16] = 4.0  # group maximum decides the scale: floor(log2(7.9)) - 2 = 0
    p, s = mxfp4.quantize_rows(v)
    assert s[0, 0] == 127
    d = mxfp4.dequantize(p, s)[0]
    assert list(d[:16]) == [0, 0, 1, 1, 2, 2, 4, 4, 6, 6, -0.0, -1, -4, -6, .5, .5]
    rng = np.random.default_rng(0)
    x = (rng.standard_normal((64, 256)) * 0.02).astype(np.float32)
    p, s = mxfp4.quantize_rows(x)
    assert s.min() >= 1 and s.max() <= 254
    d = mxfp4.dequantize(p, s)
    assert np.max(np.abs(d - x)) <= np.abs(x).max() / 4 + 1e-9
    # quantising representable values is the identity
    p2, s2 = mxfp4.quantize_rows(d)
    assert np.array_equal(mxfp4.dequantize(p2, s2), d)


def test_quantiser_torch_matches_numpy():
    import torch

    from insignia_b200 import mxfp4, synth

    rng = np.random.default_rng(3)
    x = (rng.standard_normal((128, 512)) * rng.uniform(1e-3, 10, (128, 1))).astype(np.float32)
    x[5] = 0
    p, s = mxfp4.quantize_rows(x)
    pt, st = synth.quantize_rows_torch(torch.from_numpy(x))
    assert np.array_equal(p, pt.numpy().view(np.uint32)) and np.array_equal(s, st.numpy())


def test_index_writer_is_byte_identical_to_reference_tool(tmp_path):
    from insignia_b200 import checkpoint_io as io, synth

    meta = json.load(open(os.path.join(GOLD, "index_small.json")))
    small = str(tmp_path / "small.safetensors")
    synth.write_checkpoint(synth.SynthConfig(layers=(), vocab_rows=32, mtp=False, lm_head=False, seed=1), small)
    with open(small, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
    assert header == meta["header"] and n == meta["header_len"]
    idx = str(tmp_path / "small.idx")
    assert io.write_index(small, idx) == 3
    want = open(os.path.join(GOLD, "index_small.bin"), "rb").read()
    real = os.path.realpath(small).encode()
    want = want.replace(b"@PAYLOAD@", real)
    # the reference tool stored len(path) of ITS temp file; patch the length field for ours
    want = want[:24] + struct.pack("<I", len(real)) + want[28:]
    assert open(idx, "rb").read() == want
    info = io.load_index(idx)
    assert info["payload_offset"] == 8 + n and [t["name"] for t in info["tensors"]] == sorted(header)


def test_synth_full_model_tensor_inventory():
    from insignia_b200 import synth

    specs = synth.file_specs(synth.SynthConfig())
    assert len(specs) == 699  # src/test_model.cpp:4
    names = {n: (d, s) for n, d, s in specs}
    assert names["language_model.model.layers.3.self_attn.q_proj.weight"] == ("U32", (8192, 512))  # src/test_qwen35.cu:5
    assert names["language_model.model.layers.0.linear_attn.in_proj_qkv.scales"] == ("U8", (8192, 128))
    assert names["language_model.mtp.fc.weight"] == ("BF16", (4096, 8192))
    assert sum(1 for n in names if ".linear_attn." in n) == 24 * 14


def test_golden_checkpoint_is_reproducible(golden_ckpt):
    import hashlib

    from insignia_b200.checkpoint_io import SafetensorsReader

    t = SafetensorsReader(golden_ckpt[0])
    h = hashlib.sha256(t.get("language_model.model.layers.0.linear_attn.in_proj_qkv.weight").tobytes()).hexdigest()
    assert h == open(os.path.join(GOLD, "golden4_qkv_sha256.txt")).read().strip()


def test_dropin_headers_compile_standalone(tmp_path):
    """Every header of include/ compiles on its own and together (the kernel-level ones are inline wrappers over the C ABI)."""
    import shutil
    import subprocess

    if not shutil.which("nvcc"):
        pytest.skip("nvcc not on PATH")
    inc = os.path.join(ROOT, "include")
    headers = sorted(f for f in os.listdir(inc) if f != "insignia_posix_shim.hpp")
    assert {"insignia_layout.cuh", "insignia_attention.cuh", "insignia_deltanet.cuh", "insignia_ops.cuh", "insignia_qwen_kernels.cuh",
            "insignia_model.hpp", "insignia_storage.hpp", "insignia_qwen35.hpp", "insignia_decode.hpp", "insignia_b200.h"} <= set(headers)
    src = tmp_path / "all.cu"
    src.write_text("".join(f'#include "{h}"\n' for h in headers) + """
static_assert(sizeof(insignia::MxFp4Block) == 17, "block size");
int probe() {
    insignia::MxFp4Block b{127, {0x21}};
    return insignia::mxfp4_value(b, 0) == 0.5f && insignia::mxfp4_value(b, 16) == 1.0f && insignia::fp4_e2m1(15) == -6.0f
        && insignia::e8m0(0) == 0.0f && insignia::e8m0(255) != insignia::e8m0(255);
}
int main() { return probe() ? 0 : 1; }
""")
    exe = tmp_path / "all"
    subprocess.check_call(["nvcc", "-std=c++20", "-gencode", "arch=compute_100a,code=sm_100a", "-I", inc, str(src),
                           "-L", os.path.join(ROOT, "insignia_b200", "lib"), "-linsignia_b200", "-o", str(exe)])
    env = dict(os.environ, LD_LIBRARY_PATH=os.path.join(ROOT, "insignia_b200", "lib") + ":" + os.environ.get("LD_LIBRARY_PATH", ""))
    assert subprocess.run([str(exe)], env=env).returncode == 0  # host-only helpers: runs without a GPU
