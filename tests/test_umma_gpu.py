"""The tcgen05 (kind::mxf4 block-scaled MMA) GEMV kernel, through the C ABI, against the CPU oracle."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
from oracle import oracle as orc  # noqa: E402
from tests import fixtures as fx  # noqa: E402
from tests.test_kernels_gpu import bf16, dev, host, rand_matrix  # noqa: E402

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def umma(ops, w, s):
    return ops.repack_umma(dev(w), dev(s))


def run_store(ops, P, x, rows, **kw):
    out = torch.zeros(rows, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.gemv_fused(dev(x), [dict(packed=P, out=out, rows=rows, epilogue="store")], layout=1, error_flag=err, **kw)
    assert int(err.item()) == 0
    return host(out)


def test_umma_reference_fixture(cuda):
    from insignia_b200 import ops

    w, s, x, expected = fx.mxfp4_mlx(rows=4096)
    y = run_store(ops, umma(ops, w, s), x, 4096)
    assert fx.max_rel(y, expected, 1e-5) <= 3e-4  # src/bench_mxfp4_mlx.cu:10
    y64 = orc.gemv_mlx_f64(w, s, x)
    assert np.max(np.abs(y - y64)) <= 1e-5 * np.abs(y64).max()


@pytest.mark.parametrize("rows,cols", [(4096, 4096), (1024, 12288), (32, 4096), (16, 128), (48, 1152), (2048, 8192), (12352, 4096),
                                       (128 * 149 + 16, 256)])
def test_umma_shapes_vs_oracle(cuda, rows, cols):
    from insignia_b200 import ops

    rng = np.random.default_rng(rows + cols)
    w, s = rand_matrix(rng, rows, cols)
    x = (rng.standard_normal(cols) * 3).astype(np.float32)
    y = run_store(ops, umma(ops, w, s), x, rows)
    y64 = orc.gemv_mlx_f64(w, s, x)
    assert np.max(np.abs(y - y64)) <= 4e-6 * np.abs(y64).max() + 1e-7


def test_umma_extreme_inputs(cuda):
    from insignia_b200 import ops

    rng = np.random.default_rng(5)
    rows, cols = 256, 1024
    w, s = rand_matrix(rng, rows, cols)
    P = umma(ops, w, s)
    for x in (np.zeros(cols, np.float32), np.eye(1, cols, 7, dtype=np.float32)[0] * 3e4, (rng.standard_normal(cols) * 1e-12).astype(np.float32),
              np.where(np.arange(cols) % 97 == 0, 1000.0, 1e-3).astype(np.float32)):
        y = run_store(ops, P, x, rows)
        y64 = orc.gemv_mlx_f64(w, s, x)
        assert np.all(np.isfinite(y))
        assert np.max(np.abs(y - y64)) <= 4e-6 * max(np.abs(y64).max(), 1e-30)


def test_umma_inproj_epilogues_over_tokens(cuda):
    """in_proj(qkv|z|a|b): conv+SiLU with history, store, decay, beta; three tokens (src/decode.cu:14-16)."""
    from insignia_b200 import mxfp4, ops

    rng = np.random.default_rng(21)
    nq = 384
    wq, sq = rand_matrix(rng, nq, 4096)
    wz, sz = rand_matrix(rng, 256, 4096)
    wa, sa = rand_matrix(rng, 32, 4096, std=0.05)
    wb, sb = rand_matrix(rng, 32, 4096, std=0.05)
    conv_w = mxfp4.f32_to_bf16_bits((0.5 * rng.standard_normal((nq, 4))).astype(np.float32))
    A_log = rng.uniform(-1, 1, 32).astype(np.float32)
    dt = mxfp4.f32_to_bf16_bits((0.5 * rng.standard_normal(32)).astype(np.float32))
    nw = bf16(rng, 4096)
    P = [umma(ops, w, s) for w, s in ((wq, sq), (wz, sz), (wa, sa), (wb, sb))]
    conv_state = torch.zeros(nq * 3, device="cuda")
    o_q, o_z = torch.zeros(nq, device="cuda"), torch.zeros(256, device="cuda")
    o_a, o_b = torch.zeros(32, device="cuda"), torch.zeros(32, device="cuda")
    ref_state = np.zeros(nq * 3, np.float32)
    d_nw, d_cw, d_A, d_dt = dev(nw), dev(conv_w), dev(A_log), dev(dt)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    for step in range(3):
        hidden = (rng.standard_normal(4096) * 3).astype(np.float32)
        ops.gemv_fused(dev(hidden), [
            dict(packed=P[0], out=o_q, rows=nq, epilogue="conv_silu", conv_state=conv_state, conv_w=d_cw),
            dict(packed=P[1], out=o_z, rows=256, epilogue="store"),
            dict(packed=P[2], out=o_a, rows=32, epilogue="decay", A_log=d_A, dt_bias=d_dt),
            dict(packed=P[3], out=o_b, rows=32, epilogue="beta")], prologue="rmsnorm", norm_w=d_nw, layout=1, error_flag=err)
        n = orc.rmsnorm_bf16(hidden, nw)
        q = orc.gemv_mlx(wq, sq, n)
        orc.causal_conv4_silu(q, ref_state, conv_w)
        a, b = orc.gemv_mlx(wa, sa, n), orc.gemv_mlx(wb, sb, n)
        orc.deltanet_parameters(a, b, A_log, dt)
        assert np.max(np.abs(host(o_q) - q)) <= 2e-5 * max(1.0, np.abs(q).max())
        assert np.max(np.abs(host(conv_state) - ref_state)) <= 2e-5 * np.abs(ref_state).max()
        assert np.max(np.abs(host(o_z) - orc.gemv_mlx(wz, sz, n))) <= 2e-5
        assert np.max(np.abs(host(o_a) - a)) <= 2e-5 * max(1.0, np.abs(a).max())
        assert np.max(np.abs(host(o_b) - b)) <= 2e-6
    assert int(err.item()) == 0


def test_umma_swiglu_down_residual_and_gates(cuda):
    from insignia_b200 import ops

    rng = np.random.default_rng(22)
    wg, sg = rand_matrix(rng, 768, 4096)
    wu, su = rand_matrix(rng, 768, 4096)
    wd, sd = rand_matrix(rng, 256, 12288)
    hidden = (rng.standard_normal(4096) * 3).astype(np.float32)
    nw = bf16(rng, 4096)
    act = torch.zeros(768, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.gemv_fused(dev(hidden), [dict(packed=umma(ops, wg, sg), packed2=umma(ops, wu, su), out=act, rows=768, epilogue="swiglu")],
                   prologue="rmsnorm", norm_w=dev(nw), layout=1, error_flag=err)
    n = orc.rmsnorm_bf16(hidden, nw)
    g, u = orc.gemv_mlx(wg, sg, n), orc.gemv_mlx(wu, su, n)
    want = (g / (1 + np.exp(-g)) * u).astype(np.float32)
    assert np.max(np.abs(host(act) - want)) <= 2e-5 * np.abs(want).max()
    big = (rng.standard_normal(12288) * 2).astype(np.float32)
    res0 = rng.standard_normal(256).astype(np.float32)
    out = dev(res0.copy())
    ops.gemv_fused(dev(big), [dict(packed=umma(ops, wd, sd), out=out, rows=256, epilogue="residual")], layout=1, error_flag=err)
    y = orc.gemv_mlx_f64(wd, sd, big)
    assert np.max(np.abs(host(out) - (res0 + y))) <= 6e-6 * np.abs(y).max()
    # gated RMSNorm and the attention output gates
    w, s = rand_matrix(rng, 128, 4096)
    P = umma(ops, w, s)
    core = rng.standard_normal(4096).astype(np.float32)
    z = rng.standard_normal(4096).astype(np.float32) * 2
    hw = bf16(rng, 128)
    y = run_store(ops, P, core, 128, prologue="gated_rmsnorm", aux=dev(z), norm_w=dev(hw))
    y64 = orc.gemv_mlx_f64(w, s, orc.rmsnorm_bf16(core.reshape(32, 128), hw, gate=z.reshape(32, 128)).reshape(-1))
    assert np.max(np.abs(y - y64)) <= 1e-5 * np.abs(y64).max()
    qraw = rng.standard_normal(8192).astype(np.float32)
    gate = qraw.reshape(16, 512)[:, 256:].reshape(-1).copy()
    for mode, gg in (("sigmoid_gate_qproj", gate), ("sigmoid_gate_head0", np.repeat(gate.reshape(16, 256)[:, :1], 256, 1).reshape(-1))):
        y = run_store(ops, P, core, 128, prologue=mode, aux=dev(qraw))
        y64 = orc.gemv_mlx_f64(w, s, (core * (1 / (1 + np.exp(-gg)))).astype(np.float32))
        assert np.max(np.abs(y - y64)) <= 1e-5 * np.abs(y64).max()
    assert int(err.item()) == 0


def test_umma_logits_argmax_feedback(cuda):
    from insignia_b200 import ops

    rng = np.random.default_rng(24)
    rows = 128 * 300 + 64
    w, s = rand_matrix(rng, rows, 4096)
    P = umma(ops, w, s)
    nw = bf16(rng, 4096)
    logits = torch.zeros(rows, device="cuda")
    scratch = ops.argmax_scratch("cuda")
    tok = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    fb = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    log = torch.full((16,), -1, dtype=torch.int32, device="cuda")
    pos = torch.tensor([5], dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    for it in range(2):
        hidden = (rng.standard_normal(4096) * 3).astype(np.float32)
        ops.gemv_fused(dev(hidden), [dict(packed=P, out=logits, rows=rows, epilogue="logits")], prologue="rmsnorm", norm_w=dev(nw),
                       argmax=dict(scratch=scratch, token_out=tok, token_feedback=fb, token_log=log, position=pos), layout=1, error_flag=err)
        got = host(logits)
        y = orc.gemv_mlx_f64(w, s, orc.rmsnorm_bf16(hidden, nw))
        assert np.max(np.abs(got - y)) <= 6e-6 * np.abs(y).max()
        assert int(tok.item()) == int(np.argmax(got)) == int(fb.item())
        assert int(pos.item()) == 6 + it and int(log[5 + it].item()) == int(tok.item())
    assert int(err.item()) == 0
