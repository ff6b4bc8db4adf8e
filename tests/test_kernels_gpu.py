"""CUDA kernels, called through the C ABI, against the CPU oracle (and the compiled reference kernels)."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
from oracle import oracle as orc  # noqa: E402
from oracle import ref_engine as refengine  # noqa: E402
from tests import fixtures as fx  # noqa: E402

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if a.dtype == np.uint32:
        t = torch.from_numpy(np.ascontiguousarray(a).view(np.int32))
    if a.dtype == np.uint16:
        t = torch.from_numpy(np.ascontiguousarray(a).view(np.int16))
    return t.cuda()


def host(t):
    return t.detach().cpu().numpy()


def rand_matrix(rng, rows, cols, std=0.02):
    from insignia_b200 import mxfp4

    return mxfp4.quantize_rows((rng.standard_normal((rows, cols)) * std).astype(np.float32))


def bf16(rng, n, mean=1.0, std=0.1):
    from insignia_b200 import mxfp4

    return mxfp4.f32_to_bf16_bits((mean + std * rng.standard_normal(n)).astype(np.float32))


# ------------------------------------------------------------------------ codec
def test_dequant_bit_exact_all_codes_and_scales(cuda):
    from insignia_b200 import ops

    # every E2M1 code under every scale byte, 0 and 255 included (src/mxfp4.cu:52 semantics)
    rows, cols = 256, 32
    codes = (np.arange(32) % 16).astype(np.uint32)
    word = np.zeros((rows, 4), np.uint32)
    for i in range(4):
        for j in range(8):
            word[:, i] |= codes[i * 8 + j] << np.uint32(4 * j)
    word[1::2] = np.roll(word[1::2], 1, axis=1)
    scales = np.arange(256, dtype=np.uint8).reshape(rows, 1)
    got = host(ops.dequant_mlx(dev(word), dev(scales)))
    want = orc.dequant_mlx(word, scales)
    nan = np.isnan(want)  # 0 * Inf under scale byte 255: a NaN on both sides, payload bits are not specified
    assert np.array_equal(np.isnan(got), nan) and nan.sum() == 2 * 2
    assert np.array_equal(got.view(np.uint32)[~nan], want.view(np.uint32)[~nan])
    row = host(ops.get_row_mlx(dev(word), dev(scales), 131))
    assert np.array_equal(row.view(np.uint32), want[131].view(np.uint32))


def test_dequant_bit_exact_random_matrix(cuda):
    from insignia_b200 import ops

    rng = np.random.default_rng(1)
    w, s = rand_matrix(rng, 512, 4096)
    got = host(ops.dequant_mlx(dev(w), dev(s)))
    assert np.array_equal(got.view(np.uint32), orc.dequant_mlx(w, s).view(np.uint32))


# ------------------------------------------------------------------------- GEMV
def test_gemv_mlx_reference_fixture(cuda):
    from insignia_b200 import ops

    w, s, x, expected = fx.mxfp4_mlx(rows=4096)
    y = host(ops.gemv_mlx(dev(w), dev(s), dev(x)))
    assert fx.max_rel(y, expected, 1e-5) <= 3e-4  # src/bench_mxfp4_mlx.cu:10


def test_gemv_mlx_ragged_rows(cuda):
    from insignia_b200 import ops

    rng = np.random.default_rng(2)
    for rows, cols in ((1, 32), (257, 4096), (33, 96)):
        w, s = rand_matrix(rng, rows, cols)
        x = rng.standard_normal(cols).astype(np.float32)
        y = host(ops.gemv_mlx(dev(w), dev(s), dev(x)))
        y64 = orc.gemv_mlx_f64(w, s, x)
        assert np.max(np.abs(y - y64)) <= 2e-6 * max(1.0, np.abs(y64).max()) * np.sqrt(cols)


def test_gemv_packed_reference_fixture(cuda):
    from insignia_b200 import ops

    w, s, x, expected = fx.mxfp4_mlx(rows=4096)
    packed = ops.repack(dev(w), dev(s))
    y = host(ops.gemv_packed(packed, dev(x)))
    assert fx.max_rel(y, expected, 1e-5) <= 3e-4
    y64 = orc.gemv_mlx_f64(w, s, x)
    assert np.max(np.abs(y - y64)) <= 1e-5 * np.abs(y64).max()


@pytest.mark.parametrize("rows,cols", [(4096, 4096), (1024, 12288), (32, 4096), (16, 128), (48, 1152), (2048, 8192), (12352, 4096),
                                       (16 * 149, 256), (16 * 7, 128)])
def test_gemv_packed_shapes_vs_oracle(cuda, rows, cols):
    from insignia_b200 import ops

    rng = np.random.default_rng(rows + cols)
    w, s = rand_matrix(rng, rows, cols)
    x = rng.standard_normal(cols).astype(np.float32)
    packed = ops.repack(dev(w), dev(s))
    y = host(ops.gemv_packed(packed, dev(x)))
    y64 = orc.gemv_mlx_f64(w, s, x)
    yref = orc.gemv_mlx(w, s, x, warps=2)
    tol = 4e-6 * np.abs(y64).max() + 1e-7
    assert np.max(np.abs(y - y64)) <= tol
    assert np.array_equal(host(ops.gemv_packed(packed, dev(x))), y)  # the same sums on every launch
    # the restated reference order is itself this close to the exact sum
    assert np.max(np.abs(yref - y64)) <= tol * 4


@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 8])
def test_gemv_packed_multi_token(cuda, M):
    from insignia_b200 import ops

    rng = np.random.default_rng(10 + M)
    rows, cols = 256, 4096
    w, s = rand_matrix(rng, rows, cols)
    x = (rng.standard_normal((M, cols)) * rng.uniform(0.01, 30, (M, 1))).astype(np.float32)
    packed = ops.repack(dev(w), dev(s))
    y = host(ops.gemv_packed(packed, dev(x)))
    for m in range(M):
        y64 = orc.gemv_mlx_f64(w, s, x[m])
        assert np.max(np.abs(y[m] - y64)) <= 4e-6 * np.abs(y64).max()


def test_gemv_packed_extreme_inputs(cuda):
    from insignia_b200 import ops

    rng = np.random.default_rng(5)
    rows, cols = 64, 1024
    w, s = rand_matrix(rng, rows, cols)
    packed = ops.repack(dev(w), dev(s))
    # all-zero activations, a single huge element, tiny activations
    for x in (np.zeros(cols, np.float32), np.eye(1, cols, 7, dtype=np.float32)[0] * 3e4,
              (rng.standard_normal(cols) * 1e-12).astype(np.float32)):
        y = host(ops.gemv_packed(packed, dev(x)))
        y64 = orc.gemv_mlx_f64(w, s, x)
        assert np.all(np.isfinite(y))
        assert np.max(np.abs(y - y64)) <= 4e-6 * max(np.abs(y64).max(), 1e-30)


def _fused_setup(rng, cols=4096):
    hidden = rng.standard_normal(cols).astype(np.float32) * 3
    return hidden


def test_gemv_fused_rmsnorm_store_and_residual(cuda):
    from insignia_b200 import ops

    rng = np.random.default_rng(20)
    w1, s1 = rand_matrix(rng, 512, 4096)
    w2, s2 = rand_matrix(rng, 32, 4096)
    hidden = _fused_setup(rng)
    nw = bf16(rng, 4096)
    p1, p2 = ops.repack(dev(w1), dev(s1)), ops.repack(dev(w2), dev(s2))
    out1 = torch.zeros(512, device="cuda")
    res0 = rng.standard_normal(32).astype(np.float32)
    out2 = dev(res0.copy())
    xo = torch.zeros(4096, device="cuda")
    ops.gemv_fused(dev(hidden), [dict(packed=p1, out=out1, rows=512, epilogue="store"),
                                 dict(packed=p2, out=out2, rows=32, epilogue="residual")],
                   prologue="rmsnorm", norm_w=dev(nw), x_out=xo)
    n = orc.rmsnorm_bf16(hidden, nw)
    assert np.max(np.abs(host(xo) - n)) <= 2e-6 * np.abs(n).max()
    y1, y2 = orc.gemv_mlx_f64(w1, s1, n), orc.gemv_mlx_f64(w2, s2, n)
    assert np.max(np.abs(host(out1) - y1)) <= 6e-6 * np.abs(y1).max()
    assert np.max(np.abs(host(out2) - (res0 + y2))) <= 6e-6 * np.abs(y2).max()


def test_gemv_fused_inproj_conv_decay_beta(cuda):
    """in_proj(qkv|z|a|b) with the conv+SiLU, decay and beta epilogues over two tokens (src/decode.cu:14-16)."""
    from insignia_b200 import mxfp4, ops

    rng = np.random.default_rng(21)
    nq = 256  # channels of the conv segment in this test
    wq, sq = rand_matrix(rng, nq, 4096)
    wz, sz = rand_matrix(rng, 64, 4096)
    wa, sa = rand_matrix(rng, 32, 4096, std=0.05)
    wb, sb = rand_matrix(rng, 32, 4096, std=0.05)
    conv_w = mxfp4.f32_to_bf16_bits((0.5 * rng.standard_normal((nq, 4))).astype(np.float32))
    A_log = rng.uniform(-1, 1, 32).astype(np.float32)
    dt = mxfp4.f32_to_bf16_bits((0.5 * rng.standard_normal(32)).astype(np.float32))
    nw = bf16(rng, 4096)
    P = [ops.repack(dev(w), dev(s)) for w, s in ((wq, sq), (wz, sz), (wa, sa), (wb, sb))]
    conv_state = torch.zeros(nq * 3, device="cuda")
    o_q, o_z = torch.zeros(nq, device="cuda"), torch.zeros(64, device="cuda")
    o_a, o_b = torch.zeros(32, device="cuda"), torch.zeros(32, device="cuda")
    ref_state = np.zeros(nq * 3, np.float32)
    d_nw, d_cw, d_A, d_dt = dev(nw), dev(conv_w), dev(A_log), dev(dt)
    for step in range(3):
        hidden = _fused_setup(rng)
        ops.gemv_fused(dev(hidden), [
            dict(packed=P[0], out=o_q, rows=nq, epilogue="conv_silu", conv_state=conv_state, conv_w=d_cw),
            dict(packed=P[1], out=o_z, rows=64, epilogue="store"),
            dict(packed=P[2], out=o_a, rows=32, epilogue="decay", A_log=d_A, dt_bias=d_dt),
            dict(packed=P[3], out=o_b, rows=32, epilogue="beta")], prologue="rmsnorm", norm_w=d_nw)
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


def test_gemv_fused_swiglu_and_down(cuda):
    from insignia_b200 import ops

    rng = np.random.default_rng(22)
    wg, sg = rand_matrix(rng, 768, 4096)
    wu, su = rand_matrix(rng, 768, 4096)
    wd, sd = rand_matrix(rng, 64, 12288)
    hidden = _fused_setup(rng)
    nw = bf16(rng, 4096)
    act = torch.zeros(768, device="cuda")
    ops.gemv_fused(dev(hidden), [dict(packed=ops.repack(dev(wg), dev(sg)), packed2=ops.repack(dev(wu), dev(su)), out=act,
                                      rows=768, epilogue="swiglu")], prologue="rmsnorm", norm_w=dev(nw))
    n = orc.rmsnorm_bf16(hidden, nw)
    g, u = orc.gemv_mlx(wg, sg, n), orc.gemv_mlx(wu, su, n)
    want = (g / (1 + np.exp(-g)) * u).astype(np.float32)
    assert np.max(np.abs(host(act) - want)) <= 2e-5 * np.abs(want).max()
    big = (rng.standard_normal(12288) * 2).astype(np.float32)
    res0 = rng.standard_normal(64).astype(np.float32)
    out = dev(res0.copy())
    ops.gemv_fused(dev(big), [dict(packed=ops.repack(dev(wd), dev(sd)), out=out, rows=64, epilogue="residual")])
    y = orc.gemv_mlx_f64(wd, sd, big)
    assert np.max(np.abs(host(out) - (res0 + y))) <= 6e-6 * np.abs(y).max()


def test_gemv_fused_gated_rmsnorm_and_gate_prologues(cuda):
    from insignia_b200 import ops

    rng = np.random.default_rng(23)
    w, s = rand_matrix(rng, 128, 4096)
    P = ops.repack(dev(w), dev(s))
    core = rng.standard_normal(4096).astype(np.float32)
    z = rng.standard_normal(4096).astype(np.float32) * 2
    nw = bf16(rng, 128)
    out = torch.zeros(128, device="cuda")
    ops.gemv_fused(dev(core), [dict(packed=P, out=out, rows=128, epilogue="store")], prologue="gated_rmsnorm", aux=dev(z),
                   norm_w=dev(nw))
    n = orc.rmsnorm_bf16(core.reshape(32, 128), nw, gate=z.reshape(32, 128)).reshape(-1)
    y = orc.gemv_mlx_f64(w, s, n)
    assert np.max(np.abs(host(out) - y)) <= 1e-5 * np.abs(y).max()
    # attention output gates read from the interleaved q_proj buffer [16][q256|gate256]
    qraw = rng.standard_normal(8192).astype(np.float32)
    gate = qraw.reshape(16, 512)[:, 256:].reshape(-1).copy()
    for mode, g in (("sigmoid_gate_qproj", gate), ("sigmoid_gate_head0", np.repeat(gate.reshape(16, 256)[:, :1], 256, 1).reshape(-1))):
        ops.gemv_fused(dev(core), [dict(packed=P, out=out, rows=128, epilogue="store")], prologue=mode, aux=dev(qraw))
        xg = (core * (1 / (1 + np.exp(-g)))).astype(np.float32)
        y = orc.gemv_mlx_f64(w, s, xg)
        assert np.max(np.abs(host(out) - y)) <= 1e-5 * np.abs(y).max()
    ops.gemv_fused(dev(core), [dict(packed=P, out=out, rows=128, epilogue="store")], prologue="sigmoid_gate", aux=dev(gate))
    y = orc.gemv_mlx_f64(w, s, (core * (1 / (1 + np.exp(-gate)))).astype(np.float32))
    assert np.max(np.abs(host(out) - y)) <= 1e-5 * np.abs(y).max()


def test_gemv_fused_logits_argmax_feedback(cuda):
    from insignia_b200 import ops

    rng = np.random.default_rng(24)
    rows = 16 * 700
    w, s = rand_matrix(rng, rows, 4096)
    P = ops.repack(dev(w), dev(s))
    nw = bf16(rng, 4096)
    logits = torch.zeros(rows, device="cuda")
    scratch = ops.argmax_scratch("cuda")
    tok = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    fb = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    log = torch.full((16,), -1, dtype=torch.int32, device="cuda")
    pos = torch.tensor([5], dtype=torch.int32, device="cuda")
    for it in range(2):  # twice: the ticket must be left reset
        hidden = _fused_setup(rng)
        ops.gemv_fused(dev(hidden), [dict(packed=P, out=logits, rows=rows, epilogue="logits")], prologue="rmsnorm",
                       norm_w=dev(nw), argmax=dict(scratch=scratch, token_out=tok, token_feedback=fb, token_log=log, position=pos))
        got = host(logits)
        n = orc.rmsnorm_bf16(hidden, nw)
        y = orc.gemv_mlx_f64(w, s, n)
        assert np.max(np.abs(got - y)) <= 6e-6 * np.abs(y).max()
        assert int(tok.item()) == int(np.argmax(got)) == int(fb.item())
        assert int(pos.item()) == 6 + it and int(log[5 + it].item()) == int(tok.item())
    assert int(torch.from_numpy(host(scratch)[:4].copy()).view(torch.int32).item()) == 0


# --------------------------------------------------------------------- DeltaNet
def test_deltanet_reference_fixture_with_state(cuda):
    from insignia_b200 import ops

    s, q, k, v, g, b, ref, state_after = fx.deltanet()
    st = dev(s.copy())
    out = host(ops.deltanet_decode(st, dev(q), dev(k), dev(v), dev(g), dev(b)))
    assert fx.max_rel(out, ref, 1e-5) < 3e-3  # src/test_deltanet.cu:9
    assert np.max(np.abs(host(st) - state_after)) < 1e-6


def test_deltanet_random_multi_step_vs_oracle(cuda):
    from insignia_b200 import ops

    rng = np.random.default_rng(30)
    state_ref = (rng.standard_normal(32 * 128 * 128) * 0.05).astype(np.float32)
    st = dev(state_ref.copy())
    for step in range(4):
        q = rng.standard_normal(2048).astype(np.float32)
        k = rng.standard_normal(2048).astype(np.float32)
        v = rng.standard_normal(4096).astype(np.float32)
        g = -rng.uniform(0.001, 2.0, 32).astype(np.float32)
        b = rng.uniform(0, 1, 32).astype(np.float32)
        out = host(ops.deltanet_decode(st, dev(q), dev(k), dev(v), dev(g), dev(b)))
        want = orc.deltanet_decode(state_ref, q, k, v, g, b)
        assert np.max(np.abs(out - want)) <= 2e-5 * max(1.0, np.abs(want).max())
        assert np.max(np.abs(host(st) - state_ref)) <= 2e-5 * np.abs(state_ref).max()


# -------------------------------------------------------------------- attention
def test_gqa_reference_fixture(cuda):
    from insignia_b200 import ops

    q, k, v, ref = fx.attention()
    out = host(ops.gqa_decode(dev(q), dev(k), dev(v), 257))
    assert np.max(np.abs(out - ref)) < 2e-5  # src/test_attention.cu:7


@pytest.mark.parametrize("tokens", [1, 2, 63, 64, 65, 1024, 2369, 9000])
def test_gqa_lengths_vs_oracle(cuda, tokens):
    from insignia_b200 import ops

    rng = np.random.default_rng(tokens)
    q = rng.standard_normal(4096).astype(np.float32)
    k = rng.standard_normal(tokens * 1024).astype(np.float32)
    v = rng.standard_normal(tokens * 1024).astype(np.float32)
    scratch = ops.gqa_scratch("cuda")
    for _ in range(2):  # scratch counters must come back to zero
        out = host(ops.gqa_decode(dev(q), dev(k), dev(v), tokens, scratch))
    want = orc.gqa_decode(q, k, v, tokens)
    assert np.max(np.abs(out - want)) <= 3e-5
    kb, vb = dev(k).to(torch.bfloat16), dev(v).to(torch.bfloat16)
    outb = host(ops.gqa_decode(dev(q), kb, vb, tokens, scratch))
    wantb = orc.gqa_decode(q, host(kb.float()), host(vb.float()), tokens)
    assert np.max(np.abs(outb - wantb)) <= 3e-5


@pytest.mark.parametrize("kv_bf16", [False, True])
def test_attention_step_sequence_vs_oracle(cuda, kv_bf16):
    """Fused norm+RoPE+store+attention over consecutive positions against the unfused oracle chain."""
    from insignia_b200 import ops

    rng = np.random.default_rng(40)
    ctx = 96
    qw, kw = bf16(rng, 256), bf16(rng, 256)
    kc = torch.zeros(ctx * 1024, device="cuda", dtype=torch.bfloat16 if kv_bf16 else torch.float32)
    vc = torch.zeros_like(kc)
    kc_ref, vc_ref = np.zeros(ctx * 1024, np.float32), np.zeros(ctx * 1024, np.float32)
    scratch = ops.gqa_scratch("cuda")
    pos_dev = torch.zeros(1, dtype=torch.int32, device="cuda")
    for pos in list(range(0, 70)):
        qraw = rng.standard_normal(8192).astype(np.float32)
        kraw = rng.standard_normal(1024).astype(np.float32)
        v = rng.standard_normal(1024).astype(np.float32)
        pos_dev.fill_(pos)
        out = host(ops.attention_step(dev(qraw), dev(kraw), dev(v), dev(qw), dev(kw), kc, vc, pos_dev, ctx, scratch,
                                      fast_trig=False))
        q = np.ascontiguousarray(qraw.reshape(16, 512)[:, :256]).reshape(-1)
        k = kraw.copy()
        orc.qk_norm_rope(q, k, qw, kw, pos)
        if kv_bf16:
            k = host(dev(k).to(torch.bfloat16).float())
            v = host(dev(v).to(torch.bfloat16).float())
        orc.lib().orc_store_kv(k, v, kc_ref, vc_ref, pos)
        want = orc.gqa_decode(q, kc_ref, vc_ref, pos + 1)
        assert np.max(np.abs(out - want)) <= 5e-5, pos
    # fp32 cache: rounding only; bf16 cache: at most one bf16 ulp where the fp32 values straddle a rounding boundary
    assert np.max(np.abs(host(kc.float())[:70 * 1024] - kc_ref[:70 * 1024])) <= (2.0 ** -7 * np.abs(kc_ref).max() if kv_bf16 else 1e-5)


@pytest.mark.parametrize("kv_bf16", [False, True])
def test_attention_chunk_equals_token_steps_bitwise(cuda, kv_bf16):
    """A chunk of consecutive tokens in two launches (keys and values of the chunk stored first, then every token's
    attention over the rows up to its own) against the same tokens fed one insg_attention_step at a time."""
    from insignia_b200 import ops

    rng = np.random.default_rng(41)
    ctx, start, T = 400, 37, 32
    qw, kw = bf16(rng, 256), bf16(rng, 256)
    dt = torch.bfloat16 if kv_bf16 else torch.float32
    history_k, history_v = torch.randn(ctx * 1024, device="cuda").to(dt), torch.randn(ctx * 1024, device="cuda").to(dt)
    qraw = dev(rng.standard_normal((T, 8192)).astype(np.float32))
    kraw = dev(rng.standard_normal((T, 1024)).astype(np.float32))
    v = dev(rng.standard_normal((T, 1024)).astype(np.float32))
    pos_dev = torch.zeros(1, dtype=torch.int32, device="cuda")
    kc1, vc1 = history_k.clone(), history_v.clone()
    scratch = ops.gqa_scratch("cuda")
    want = []
    for m in range(T):
        pos_dev.fill_(start + m)
        want.append(host(ops.attention_step(qraw[m], kraw[m], v[m], dev(qw), dev(kw), kc1, vc1, pos_dev, ctx, scratch)))
    kc2, vc2 = history_k.clone(), history_v.clone()
    pos_dev.fill_(start)
    big = torch.zeros(T * scratch.numel(), dtype=torch.uint8, device="cuda")
    got = host(ops.attention_chunk(qraw, kraw, v, dev(qw), dev(kw), kc2, vc2, pos_dev, ctx, big, T))
    assert np.array_equal(got, np.stack(want))
    assert torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    # the scratch heads are left zero: a second chunk right behind the first gives the same again; with the host's hint of
    # the context length fewer CTAs start, and the result is the same
    kc3, vc3 = history_k.clone(), history_v.clone()
    assert np.array_equal(host(ops.attention_chunk(qraw, kraw, v, dev(qw), dev(kw), kc3, vc3, pos_dev, ctx, big, T, rows_hint=start + T)), got)
    with pytest.raises(Exception, match="scratch"):
        ops.attention_chunk(qraw, kraw, v, dev(qw), dev(kw), kc3, vc3, pos_dev, ctx, scratch, T)


@pytest.mark.parametrize("kv_bf16", [False, True])
def test_attention_batch_equals_sequence_steps_bitwise(cuda, kv_bf16):
    """Five independent sequences at the same position in one launch against one insg_attention_step per sequence."""
    from insignia_b200 import ops

    rng = np.random.default_rng(43)
    ctx, pos, B = 300, 211, 5
    qw, kw = bf16(rng, 256), bf16(rng, 256)
    dt = torch.bfloat16 if kv_bf16 else torch.float32
    kc, vc = torch.randn(B, ctx * 1024, device="cuda").to(dt), torch.randn(B, ctx * 1024, device="cuda").to(dt)
    qraw = dev(rng.standard_normal((B, 8192)).astype(np.float32))
    kraw = dev(rng.standard_normal((B, 1024)).astype(np.float32))
    v = dev(rng.standard_normal((B, 1024)).astype(np.float32))
    pos_dev = torch.full((1,), pos, dtype=torch.int32, device="cuda")
    kc1, vc1 = kc.clone(), vc.clone()
    scratch = ops.gqa_scratch("cuda")
    want = [host(ops.attention_step(qraw[s], kraw[s], v[s], dev(qw), dev(kw), kc1[s], vc1[s], pos_dev, ctx, scratch)) for s in range(B)]
    kc2, vc2 = kc.clone(), vc.clone()
    big = torch.zeros(B * scratch.numel(), dtype=torch.uint8, device="cuda")
    got = host(ops.attention_batch(qraw, kraw, v, dev(qw), dev(kw), kc2, vc2, pos_dev, ctx, big, B))
    assert np.array_equal(got, np.stack(want))
    assert torch.equal(kc1, kc2) and torch.equal(vc1, vc2)


# -------------------------------------------------------------------- small ops
def test_small_ops_vs_oracle(cuda):
    from insignia_b200 import mxfp4, ops

    rng = np.random.default_rng(50)
    x, w, ref = fx.rmsnorm()
    assert np.max(np.abs(host(ops.rmsnorm_zero_centered(dev(x), dev(w))) - ref)) < 2e-6  # src/test_ops.cu:7
    h = rng.standard_normal((3, 4096)).astype(np.float32)
    nw = bf16(rng, 4096)
    for zc in (False, True):
        assert np.max(np.abs(host(ops.rmsnorm_bf16(dev(h), dev(nw), zc)) - orc.rmsnorm_bf16(h, nw, zc))) <= 3e-6 * 8
    g = rng.standard_normal(12288).astype(np.float32) * 3
    u = rng.standard_normal(12288).astype(np.float32)
    want = np.empty_like(g)
    orc.lib().orc_silu_mul(g, u, want, g.size)
    assert np.max(np.abs(host(ops.silu_mul(dev(g), dev(u))) - want)) <= 1e-5
    a = dev(g[:4096].copy())
    ops.residual_add(a, dev(u[:4096].copy()))
    assert np.array_equal(host(a), g[:4096] + u[:4096])
    a = dev(g[:4096].copy())
    ops.sigmoid_mul(a, dev(u[:4096].copy()))
    assert np.max(np.abs(host(a) - g[:4096] / (1 + np.exp(-u[:4096])))) <= 1e-5
    qraw = rng.standard_normal(8192).astype(np.float32)
    q, gate = ops.split_q_gate(dev(qraw))
    assert np.array_equal(host(q), qraw.reshape(16, 512)[:, :256].reshape(-1))
    assert np.array_equal(host(gate), qraw.reshape(16, 512)[:, 256:].reshape(-1))
    assert np.array_equal(host(ops.expand_gate_heads(gate)), np.repeat(host(gate).reshape(16, 256)[:, :1], 256, 1).reshape(-1))
    assert np.array_equal(host(ops.concat(q, gate)), np.concatenate([host(q), host(gate)]))
    logits = rng.standard_normal(248320).astype(np.float32)
    logits[[77, 200000]] = 9.0
    assert int(ops.argmax_logits(dev(logits)).item()) == 77
    wbf = mxfp4.f32_to_bf16_bits((0.02 * rng.standard_normal((128, 8192))).astype(np.float32))
    xx = rng.standard_normal(8192).astype(np.float32)
    got = host(ops.bf16_gemv(dev(wbf), dev(xx)))
    assert np.max(np.abs(got - orc.bf16_gemv(wbf, xx))) <= 2e-5
    # conv + params
    n = 512
    cw = mxfp4.f32_to_bf16_bits((0.5 * rng.standard_normal((n, 4))).astype(np.float32))
    st_ref, st = np.zeros(n * 3, np.float32), torch.zeros(n * 3, device="cuda")
    for _ in range(5):
        xv = rng.standard_normal(n).astype(np.float32)
        xd, xr = dev(xv.copy()), xv.copy()
        ops.causal_conv4_silu(xd, st, dev(cw))
        orc.causal_conv4_silu(xr, st_ref, cw)
        assert np.max(np.abs(host(xd) - xr)) <= 1e-5 and np.array_equal(host(st), st_ref)
    aa, bb = rng.standard_normal(32).astype(np.float32) * 8, rng.standard_normal(32).astype(np.float32)
    aa[0] = 25.0
    A, dt = rng.uniform(-1, 1, 32).astype(np.float32), mxfp4.f32_to_bf16_bits(rng.standard_normal(32).astype(np.float32))
    ad, bd = dev(aa.copy()), dev(bb.copy())
    ops.deltanet_parameters(ad, bd, dev(A), dev(dt))
    orc.deltanet_parameters(aa, bb, A, dt)
    assert np.max(np.abs(host(ad) - aa)) <= 2e-5 * np.abs(aa).max() and np.max(np.abs(host(bd) - bb)) <= 1e-6
    # q/k norm + RoPE, accurate and fast trigonometry
    for pos in (0, 1, 777):
        q0, k0 = rng.standard_normal(4096).astype(np.float32), rng.standard_normal(1024).astype(np.float32)
        qw, kw = bf16(rng, 256), bf16(rng, 256)
        qr, kr = q0.copy(), k0.copy()
        orc.qk_norm_rope(qr, kr, qw, kw, pos)
        for fast, tol in ((False, 3e-6), (True, 2e-3)):
            qd, kd = dev(q0.copy()), dev(k0.copy())
            ops.qk_norm_rope(qd, kd, dev(qw), dev(kw), pos, fast)
            assert np.max(np.abs(host(qd) - qr)) <= tol * 8 and np.max(np.abs(host(kd) - kr)) <= tol * 8


@pytest.mark.skipif(not refengine.available(), reason="compiled reference (oracle/_ref) not built")
def test_kernels_vs_compiled_reference(cuda):
    """The reference's own CUDA kernels (unmodified sources, sm_100a) on the same device buffers."""
    from insignia_b200 import ops

    rng = np.random.default_rng(60)
    w, s = rand_matrix(rng, 4096, 4096)
    x = rng.standard_normal(4096).astype(np.float32)
    dw, ds, dx = dev(w), dev(s), dev(x)
    yref = torch.zeros(4096, device="cuda")
    refengine.call("ref_mxfp4_gemv_mlx", dw.data_ptr(), ds.data_ptr(), dx.data_ptr(), yref.data_ptr(), 4096, 4096, 2)
    y = ops.gemv_packed(ops.repack(dw, ds), dx)
    assert float((y - yref).abs().max()) <= 6e-6 * float(yref.abs().max())
    # the CPU restatement of the reference order agrees with the reference kernel to rounding
    assert np.max(np.abs(orc.gemv_mlx(w, s, x, warps=2) - host(yref))) <= 2e-6 * float(yref.abs().max())
    # DeltaNet
    st0 = (rng.standard_normal(32 * 128 * 128) * 0.05).astype(np.float32)
    q, k, v = (rng.standard_normal(n).astype(np.float32) for n in (2048, 2048, 4096))
    g, b = -rng.uniform(0.01, 1, 32).astype(np.float32), rng.uniform(0, 1, 32).astype(np.float32)
    s1, s2 = dev(st0.copy()), dev(st0.copy())
    oref = torch.zeros(4096, device="cuda")
    dq, dk, dv, dg, db = dev(q), dev(k), dev(v), dev(g), dev(b)
    refengine.call("ref_deltanet_decode", s1.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dg.data_ptr(),
                   db.data_ptr(), oref.data_ptr())
    o = ops.deltanet_decode(s2, dq, dk, dv, dg, db)
    assert float((o - oref).abs().max()) <= 2e-5 * max(1.0, float(oref.abs().max()))
    assert float((s1 - s2).abs().max()) <= 2e-5 * float(s1.abs().max())
    # attention
    T = 300
    qq = dev(rng.standard_normal(4096).astype(np.float32))
    kk, vv = dev(rng.standard_normal(T * 1024).astype(np.float32)), dev(rng.standard_normal(T * 1024).astype(np.float32))
    refengine.call("ref_gqa_decode", qq.data_ptr(), kk.data_ptr(), vv.data_ptr(), oref.data_ptr(), T)
    o = ops.gqa_decode(qq, kk, vv, T)
    assert float((o - oref).abs().max()) <= 3e-5


# ------------------------------------------------------------------------ launchers outside the token loop
def test_block_layout_gemv_vs_scalar_decode(cuda):
    """include/insignia_layout.cuh:11-15 blocks: low nibbles are elements 0..15, high nibbles 16..31."""
    from insignia_b200 import _lib

    rng = np.random.default_rng(11)
    rows, cols = 37, 256
    blocks = rng.integers(0, 256, (rows, cols // 32, 17), dtype=np.uint8)
    blocks[:, :, 0] = rng.integers(118, 132, (rows, cols // 32))
    x = rng.standard_normal(cols).astype(np.float32)
    lut = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], np.float64)
    codes = np.concatenate([blocks[:, :, 1:] & 15, blocks[:, :, 1:] >> 4], axis=2)  # [rows][blocks][32]
    w = lut[codes] * np.exp2(blocks[:, :, :1].astype(np.float64) - 127)
    expected = (w.reshape(rows, cols) * x).sum(1)
    y, db, dx = torch.zeros(rows, device="cuda"), dev(blocks), dev(x)
    _lib.check(_lib.lib().insg_mxfp4_gemv_blocks(db.data_ptr(), dx.data_ptr(), y.data_ptr(), rows, cols, None))
    assert np.max(np.abs(host(y) - expected)) <= 1e-5 * np.abs(expected).max()
    assert _lib.lib().insg_mxfp4_gemv_blocks(db.data_ptr(), dx.data_ptr(), y.data_ptr(), rows, 48, None) < 0


def test_int8_activation_path(cuda):
    """src/mxfp4.cu:83-127: per-32 absmax int8 quantisation, then integer dot products with doubled E2M1 codes."""
    from insignia_b200 import _lib, mxfp4

    rng = np.random.default_rng(12)
    rows, cols = 130, 512
    w, s = rand_matrix(rng, rows, cols)
    x = rng.standard_normal(cols).astype(np.float32)
    x[64:96] = 0.0  # an all-zero group keeps scale 1
    L = _lib.lib()
    dx, qx, qs, y = dev(x), torch.zeros(cols, dtype=torch.int8, device="cuda"), torch.zeros(cols // 32, device="cuda"), torch.zeros(rows, device="cuda")
    _lib.check(L.insg_quantize_q8_groups(dx.data_ptr(), qx.data_ptr(), qs.data_ptr(), cols, None))
    g = x.reshape(-1, 32)
    amax = np.abs(g).max(1)
    scale = np.where(amax > 0, amax * np.float32(1.0 / 127.0), np.float32(1.0)).astype(np.float32)
    q = np.rint(g / scale[:, None]).astype(np.int8)
    assert np.array_equal(host(qs), scale)
    assert np.max(np.abs(host(qx).astype(np.int32) - q.reshape(-1).astype(np.int32))) <= 1  # division rounding at exact halves
    dw, ds = dev(w), dev(s)
    _lib.check(L.insg_mxfp4_gemv_dp4a(dw.data_ptr(), ds.data_ptr(), qx.data_ptr(), qs.data_ptr(), y.data_ptr(), rows, cols, None))
    deq = mxfp4.dequantize(w, s).astype(np.float64)
    xq = (host(qx).astype(np.float64).reshape(-1, 32) * host(qs).astype(np.float64)[:, None]).reshape(-1)
    expected = deq @ xq  # exact given the quantised activations
    assert np.max(np.abs(host(y) - expected)) <= 1e-5 * np.abs(expected).max()
    assert np.max(np.abs(host(y) - deq @ x)) <= 3e-2 * np.abs(deq @ x).max()  # int8 rounding of x


def test_gemv_fused_prepared_chain_matches_in_kernel_prologues(cuda):
    """out_proj (residual, leaves the next RMSNorm's input ready) -> gate|up (prepared input, leaves its SwiGLU output
    ready) -> down (prepared input, residual): against the oracle chain and against the same three launches with the
    in-kernel prologues.  At scales the fixed-scale image cannot hold (tiny or huge residual stream) the consumer must
    notice from the producer's sums and read the fp32 vector instead."""
    from insignia_b200 import _lib, ops

    rng = np.random.default_rng(31)
    wo, so = rand_matrix(rng, 4096, 4096)
    wg, sg = rand_matrix(rng, 12288, 4096)
    wu, su = rand_matrix(rng, 12288, 4096)
    wd, sd = rand_matrix(rng, 4096, 12288)
    po, pg, pu, pd = (ops.repack(dev(w), dev(s)) for w, s in ((wo, so), (wg, sg), (wu, su), (wd, sd)))
    nw = bf16(rng, 4096)
    x0 = rng.standard_normal(4096).astype(np.float32)

    def run(h0, prepared):
        hidden = dev(h0.copy())
        act_d = torch.zeros(12288, device="cuda")
        img_h = torch.zeros(2 * 4096, dtype=torch.float16, device="cuda")
        img_a = torch.zeros(2 * 12288, dtype=torch.float16, device="cuda")
        parts = torch.full((2, 296), 7.0, device="cuda")  # stale values must be overwritten
        if prepared:
            ops.gemv_fused(dev(x0), [dict(packed=po, out=hidden, rows=4096, epilogue="residual", prep=img_h, prep_w=dev(nw),
                                          prep_partials=parts[0])])
            ops.gemv_fused(img_h, [dict(packed=pg, packed2=pu, out=act_d, rows=12288, epilogue="swiglu", prep=img_a,
                                        prep_partials=parts[1])],
                           prologue="prepared", prep_partials=parts[0], prep_rms=True, aux=hidden, norm_w=dev(nw), cols=4096)
            ops.gemv_fused(img_a, [dict(packed=pd, out=hidden, rows=4096, epilogue="residual")], prologue="prepared",
                           prep_partials=parts[1], aux=act_d, cols=12288)
        else:
            ops.gemv_fused(dev(x0), [dict(packed=po, out=hidden, rows=4096, epilogue="residual")])
            ops.gemv_fused(hidden, [dict(packed=pg, packed2=pu, out=act_d, rows=12288, epilogue="swiglu")], prologue="rmsnorm",
                           norm_w=dev(nw))
            ops.gemv_fused(act_d, [dict(packed=pd, out=hidden, rows=4096, epilogue="residual")])
        return host(hidden), host(act_d), host(parts)

    for scale, outlier in ((3.0, 250.0), (1e-6, 0.0), (3e6, 0.0), (3.0, 4e7)):
        h0 = (rng.standard_normal(4096) * scale).astype(np.float32)
        if outlier:
            h0[7] = outlier  # an outlier in the residual stream (the second one is beyond what the image can hold)
        h1 = h0 + orc.gemv_mlx_f64(wo, so, x0)
        n = orc.rmsnorm_bf16(h1.astype(np.float32), nw)
        g, u = orc.gemv_mlx_f64(wg, sg, n), orc.gemv_mlx_f64(wu, su, n)
        act = g / (1 + np.exp(-g)) * u
        h2 = h1 + orc.gemv_mlx_f64(wd, sd, act.astype(np.float32))
        hp, ap, parts = run(h0, True)
        hn, an, _ = run(h0, False)
        assert np.max(np.abs(ap - act)) <= 3e-5 * np.abs(act).max(), (scale, outlier)
        assert np.max(np.abs(hp - h2)) <= 2e-5 * np.abs(h2).max(), (scale, outlier)
        assert np.max(np.abs(ap - an)) <= 2e-5 * np.abs(an).max() and np.max(np.abs(hp - hn)) <= 1e-5 * np.abs(hn).max()
        if outlier > 1e7 or scale > 1e6:
            assert np.isinf(parts[0].sum())  # the producer flagged values that did not fit the image
        else:
            assert abs(parts[0].sum() - float((h1.astype(np.float64) ** 2).sum())) <= 1e-5 * float((h1.astype(np.float64) ** 2).sum())
        assert np.count_nonzero(parts[0]) <= 148
    # a prepared input is one token wide, and only residual / SwiGLU rows can be left prepared
    with pytest.raises(_lib.InsigniaError):
        ops.gemv_fused(dev(x0), [dict(packed=po, out=torch.zeros(4096, device="cuda"), rows=4096, epilogue="store",
                                      prep=torch.zeros(8192, dtype=torch.float16, device="cuda"))])


@pytest.mark.parametrize("tokens", [2, 4])
def test_gemv_fused_consecutive_tokens_equal_single_token_launches(cuda, tokens):
    """A launch over 2 or 4 consecutive tokens of one sequence (weights streamed once) gives, bit for bit, what one
    launch per token gives, including the convolution history that is carried from token to token."""
    from insignia_b200 import mxfp4, ops

    rng = np.random.default_rng(41)
    nq = 256
    wq, sq = rand_matrix(rng, nq, 4096)
    wz, sz = rand_matrix(rng, 64, 4096)
    wa, sa = rand_matrix(rng, 32, 4096, std=0.05)
    wb, sb = rand_matrix(rng, 32, 4096, std=0.05)
    P = [ops.repack(dev(w), dev(s)) for w, s in ((wq, sq), (wz, sz), (wa, sa), (wb, sb))]
    d_cw = dev(mxfp4.f32_to_bf16_bits((0.5 * rng.standard_normal((nq, 4))).astype(np.float32)))
    d_A = dev(rng.uniform(-1, 1, 32).astype(np.float32))
    d_dt = dev(mxfp4.f32_to_bf16_bits((0.5 * rng.standard_normal(32)).astype(np.float32)))
    d_nw = dev(bf16(rng, 4096))
    hidden = dev(np.stack([_fused_setup(rng) for _ in range(tokens)]))
    state0 = (rng.standard_normal(nq * 3)).astype(np.float32)

    def segs(o, conv):
        return [dict(packed=P[0], out=o[0], rows=nq, epilogue="conv_silu", conv_state=conv, conv_w=d_cw),
                dict(packed=P[1], out=o[1], rows=64, epilogue="store"),
                dict(packed=P[2], out=o[2], rows=32, epilogue="decay", A_log=d_A, dt_bias=d_dt),
                dict(packed=P[3], out=o[3], rows=32, epilogue="beta")]

    rows = (nq, 64, 32, 32)
    together = [torch.zeros(tokens, r, device="cuda") for r in rows]
    conv_a = dev(state0.copy())
    ops.gemv_fused(hidden, segs(together, conv_a), prologue="rmsnorm", norm_w=d_nw, cols=4096, tokens=tokens)
    conv_b = dev(state0.copy())
    for m in range(tokens):
        single = [torch.zeros(r, device="cuda") for r in rows]
        ops.gemv_fused(hidden[m], segs(single, conv_b), prologue="rmsnorm", norm_w=d_nw)
        for o, t in zip(single, together):
            assert np.array_equal(host(o), host(t[m])), m
    assert np.array_equal(host(conv_a), host(conv_b))
    # residual and SwiGLU rows, gated prologue with a per-token operand
    wg, sg = rand_matrix(rng, 256, 4096)
    wu, su = rand_matrix(rng, 256, 4096)
    pg, pu = ops.repack(dev(wg), dev(sg)), ops.repack(dev(wu), dev(su))
    z = dev(rng.standard_normal((tokens, 4096)).astype(np.float32))
    gw = dev(bf16(rng, 128))
    res0 = rng.standard_normal((tokens, 256)).astype(np.float32)
    act_t, res_t = torch.zeros(tokens, 256, device="cuda"), dev(res0.copy())
    ops.gemv_fused(hidden, [dict(packed=pg, packed2=pu, out=act_t, rows=256, epilogue="swiglu")], prologue="gated_rmsnorm", aux=z,
                   norm_w=gw, cols=4096, tokens=tokens)
    ops.gemv_fused(hidden, [dict(packed=pg, out=res_t, rows=256, epilogue="residual")], cols=4096, tokens=tokens)
    for m in range(tokens):
        act_1, res_1 = torch.zeros(256, device="cuda"), dev(res0[m].copy())
        ops.gemv_fused(hidden[m], [dict(packed=pg, packed2=pu, out=act_1, rows=256, epilogue="swiglu")], prologue="gated_rmsnorm",
                       aux=z[m], norm_w=gw)
        ops.gemv_fused(hidden[m], [dict(packed=pg, out=res_1, rows=256, epilogue="residual")])
        assert np.array_equal(host(act_1), host(act_t[m])) and np.array_equal(host(res_1), host(res_t[m])), m


@pytest.mark.parametrize("T", [2, 4, 32, 33, 70])
def test_deltanet_several_steps_in_one_launch(cuda, T):
    """Consecutive steps in one launch (state kept on chip, inputs prepared per block of 32 steps, outputs folded one
    step late) equal single-step launches, bit for bit."""
    from insignia_b200 import ops

    rng = np.random.default_rng(51 + T)
    state0 = (rng.standard_normal(32 * 128 * 128) * 0.05).astype(np.float32)
    qkv = rng.standard_normal((T, 8192)).astype(np.float32)
    g = -rng.uniform(0.01, 1, (T, 32)).astype(np.float32)
    b = rng.uniform(0, 1, (T, 32)).astype(np.float32)
    d_qkv, d_g, d_b = dev(qkv), dev(g), dev(b)
    sa = dev(state0.copy())
    flat = d_qkv.reshape(-1)  # step m's q, k, v start at m * 8192 + {0, 2048, 4096}
    together = host(ops.deltanet_decode_tokens(sa, flat, flat[2048:], flat[4096:], d_g, d_b, T, 8192))
    sb = dev(state0.copy())
    for m in range(T):
        one = host(ops.deltanet_decode(sb, d_qkv[m, :2048], d_qkv[m, 2048:4096], d_qkv[m, 4096:], d_g[m], d_b[m]))
        assert np.array_equal(one, together[m]), m
    assert np.array_equal(host(sa), host(sb))
