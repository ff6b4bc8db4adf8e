"""The reference's own console drivers, compiled unmodified against this repository's headers and library.

`make -C oracle drivers` builds every driver of the reference (src/test_*.cu, src/generate_ids.cu,
src/dump_*.cu, src/bench_mxfp4_mlx.cu, src/test_model.cpp) twice: "new" = this repository's include/ +
libinsignia_b200.so, "ref" = the reference's headers + its own sources.  The kernel-level drivers carry
their own CPU check and thresholds and must exit 0; the model-level drivers are run on the same synthetic
full-size checkpoint in both builds and what they print (token ids, checksums) or dump (layer seams) is compared.
"""
import os
import re
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.join(os.path.dirname(__file__), "..")
sys.path.insert(0, ROOT)
NEW = os.path.join(ROOT, "oracle", "_ref", "drivers", "new")
REF = os.path.join(ROOT, "oracle", "_ref", "drivers", "ref")

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not os.path.exists(os.path.join(NEW, "test_generate")),
                                 reason="reference drivers not built (make -C oracle drivers needs the reference checkout)")]


def run(path, *args, timeout=600):
    p = subprocess.run([path, *args], capture_output=True, text=True, timeout=timeout)
    return p.returncode, p.stdout + p.stderr


@pytest.fixture(scope="module")
def index(cuda):
    import bench

    return bench.ensure_checkpoint(0, True)[1]


@pytest.mark.parametrize("name", ["test_mxfp4", "test_deltanet", "test_attention", "test_ops"])
def test_kernel_driver_passes_its_own_check(cuda, name):
    """Tier-A fixtures of the reference: closed-form inputs, CPU loop inside the driver, its own thresholds."""
    rc, out = run(os.path.join(NEW, name))
    print(out)
    assert rc == 0, out


def test_microbenchmark_driver_runs(cuda):
    """src/bench_mxfp4_mlx.cu: prints max relative error of the MLX-layout GEMV and of the int8 path against its CPU loop."""
    rc, out = run(os.path.join(NEW, "bench_mxfp4_mlx"))
    print(out)
    assert rc == 0, out
    errs = [float(x) for x in re.findall(r"max_rel=([0-9.eE+-]+)", out)]
    assert errs and errs[0] < 1e-4, out  # fp32 path; the int8 path is approximate by design


def both(name, *args):
    rn, on = run(os.path.join(NEW, name), *args)
    rr, orf = run(os.path.join(REF, name), *args)
    print("new:", on, "\nref:", orf)
    assert rn == 0, on
    assert rr == 0, orf
    return on, orf


def test_model_file_driver(index):
    rc, out = run(os.path.join(NEW, "test_model"), index)
    print(out)
    assert rc == 0 and "mapped 699 tensors" in out, out


def test_generate_driver_tokens_identical(index):
    on, orf = both("test_generate", index)
    pat = r"step=(\d+) token=(\d+) -> (\d+)"
    assert re.findall(pat, on) == re.findall(pat, orf) and len(re.findall(pat, on)) == 3


def test_generate_ids_driver_tokens_identical(index):
    prompt = [str(t) for t in (42, 1000, 248319, 7, 123456, 99)]
    on, orf = both("generate_ids", index, *prompt)
    ints = lambda s: [int(x) for x in re.findall(r"-?\d+", s)]
    assert ints(on) == ints(orf) and len(ints(on)) == 3 + 8


def test_mtp_driver_drafts_identical(index):
    on, orf = both("test_mtp", index)
    pat = r"input=(\d+) cold_draft=(\d+) draft=(\d+)"
    assert re.findall(pat, on) == re.findall(pat, orf) and re.findall(pat, on)


def floats_after(s, keys):
    return [float(re.search(key + r"=([-+0-9.eE]+|nan|inf)", s).group(1)) for key in keys]


@pytest.mark.parametrize("name", ["test_full_model", "test_layer"])
def test_hidden_checksum_drivers_agree(index, name):
    on, orf = both(name, index)
    (sn, mn), (sr, mr) = floats_after(on, ["sum", "max"]), floats_after(orf, ["sum", "max"])
    assert abs(mn - mr) <= 1e-3 * abs(mr)
    assert abs(sn - sr) <= 1e-3 * 4096 ** 0.5 * abs(mr)  # a sum of 4096 terms of that size


def test_weights_driver_agrees(index):
    on, orf = both("test_qwen35", index)
    assert floats_after(on, ["sum", "max"]) == floats_after(orf, ["sum", "max"])  # a dequantised row: exact
    assert "q_proj=8192x4096" in on


def test_checkpoint_driver_agrees(index):
    on, orf = both("test_checkpoint", index)
    (cn, mn), (cr, mr) = floats_after(on, ["checksum", "max_abs"]), floats_after(orf, ["checksum", "max_abs"])
    assert abs(mn - mr) <= 1e-5 * abs(mr) and abs(cn - cr) <= 1e-4 * 8192 ** 0.5 * abs(mr)
    assert "LRU eviction/reload" in on


@pytest.mark.parametrize("name", ["dump_layers", "dump_layer0", "dump_layer3", "dump_attention"])
def test_dump_drivers_agree(index, tmp_path, name):
    """Seam dumps (the files the reference compares with its NumPy tools): cosine >= 0.9999 and
    max-abs-rel <= 2e-2 per 1024-float piece."""
    fn, fr = str(tmp_path / "new.f32"), str(tmp_path / "ref.f32")
    rn, on = run(os.path.join(NEW, name), index, fn)
    rr, orf = run(os.path.join(REF, name), index, fr)
    assert rn == 0, on
    assert rr == 0, orf
    a, b = np.fromfile(fn, np.float32), np.fromfile(fr, np.float32)
    assert a.size == b.size and a.size >= 4096 and a.size % 1024 == 0
    worst = 0.0
    for i in range(0, a.size, 1024):
        x, y = a[i:i + 1024].astype(np.float64), b[i:i + 1024].astype(np.float64)
        if not np.any(y):
            assert not np.any(x)
            continue
        assert x @ y / np.linalg.norm(x) / np.linalg.norm(y) >= 0.9999, (name, i)
        rel = float(np.max(np.abs(x - y)) / np.abs(y).max())
        assert rel <= 2e-2, (name, i, rel)
        worst = max(worst, rel)
    print(name, "worst max-abs-rel", worst)
