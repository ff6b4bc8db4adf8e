"""The persistent token kernel (insg_program_*): a recorded sequence of fused operations run by one cooperative launch,
checked against the same operations launched one by one, against the CPU oracle, and for its bounded barrier wait."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
from oracle import oracle as orc  # noqa: E402
from tests.test_kernels_gpu import bf16, dev, host, rand_matrix  # noqa: E402

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _mlp_ops(rng, rows_inter=1536, rows_out=4096):
    """post-norm + gate|up + SwiGLU (leaves its output prepared) -> down + residual (leaves the hidden vector prepared)."""
    from insignia_b200 import ops

    wg, sg = rand_matrix(rng, rows_inter, 4096)
    wu, su = rand_matrix(rng, rows_inter, 4096)
    wd, sd = rand_matrix(rng, rows_out, rows_inter)
    t = dict(pg=ops.repack(dev(wg), dev(sg)), pu=ops.repack(dev(wu), dev(su)), pd=ops.repack(dev(wd), dev(sd)),
             nw=dev(bf16(rng, 4096)), nw2=dev(bf16(rng, rows_out)), hidden0=(rng.standard_normal(4096) * 3).astype(np.float32))
    t["raw"] = (wg, sg, wu, su, wd, sd)
    return t


def _mlp_buffers(t, rows_inter, rows_out):
    return dict(hidden=dev(t["hidden0"].copy()), act=torch.zeros(rows_inter, device="cuda"),
                prep_act=torch.zeros(2 * rows_inter, dtype=torch.float16, device="cuda"),
                prep_hidden=torch.zeros(2 * rows_out, dtype=torch.float16, device="cuda"),
                sums_act=torch.zeros(296, device="cuda"), sums_hidden=torch.zeros(296, device="cuda"))


def _mlp_calls(t, b, rows_inter, rows_out):
    """(input, segments, keywords) of the two GEMVs, for ops.gemv_fused or Program.add_gemv."""
    up = (b["hidden"], [dict(packed=t["pg"], packed2=t["pu"], out=b["act"], rows=rows_inter, epilogue="swiglu", prep=b["prep_act"],
                             prep_partials=b["sums_act"])], dict(prologue="rmsnorm", norm_w=t["nw"]))
    down = (b["prep_act"], [dict(packed=t["pd"], out=b["hidden"], rows=rows_out, epilogue="residual", prep=b["prep_hidden"],
                                 prep_w=t["nw2"], prep_partials=b["sums_hidden"])],
            dict(prologue="prepared", prep_partials=b["sums_act"], aux=b["act"], cols=rows_inter))
    return up, down


def test_program_mlp_pair_bitwise_equals_launches(cuda):
    """Two dependent GEMV phases (SwiGLU pair -> down + residual, with prepared inputs) in one persistent launch give the
    same bits as the two stand-alone launches, three token steps in a row."""
    from insignia_b200 import ops

    rng = np.random.default_rng(100)
    ri, ro = 1536, 4096
    t = _mlp_ops(rng, ri, ro)
    a, b = _mlp_buffers(t, ri, ro), _mlp_buffers(t, ri, ro)
    prog = ops.Program()
    for inp, segs, kw in _mlp_calls(t, b, ri, ro):
        prog.add_gemv(inp, segs, **kw)
    prog.finalize()
    assert prog.phase_count == 2 and prog.weight_bytes == (2 * ri * 4096 + ro * ri) * 17 // 32
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    for step in range(3):
        for inp, segs, kw in _mlp_calls(t, a, ri, ro):
            ops.gemv_fused(inp, segs, **kw)
        prog.run(error_flag=err)
        torch.cuda.synchronize()
        assert int(err.item()) == 0
        for name in ("hidden", "act", "prep_act", "prep_hidden", "sums_act", "sums_hidden"):
            assert torch.equal(a[name], b[name]), (step, name)
    # and the result is the oracle's
    wg, sg, wu, su, wd, sd = t["raw"]
    h = t["hidden0"].copy()
    for step in range(3):
        n = orc.rmsnorm_bf16(h, host(t["nw"]).view(np.uint16))
        g, u = orc.gemv_mlx(wg, sg, n), orc.gemv_mlx(wu, su, n)
        act = (g / (1 + np.exp(-g)) * u).astype(np.float32)
        h = h + orc.gemv_mlx_f64(wd, sd, act).astype(np.float32)
    assert np.max(np.abs(host(b["hidden"]) - h)) <= 2e-5 * np.abs(h).max()


@pytest.mark.parametrize("prefetch", [0, 8, 200])
def test_program_many_tokens_one_launch(cuda, prefetch):
    """n_tokens > 1: the kernel loops over the program itself; the L2 prefetch cursor (any distance, also beyond the
    program's length) changes nothing in the results."""
    from insignia_b200 import ops

    rng = np.random.default_rng(101)
    ri, ro = 768, 4096
    t = _mlp_ops(rng, ri, ro)
    a, b = _mlp_buffers(t, ri, ro), _mlp_buffers(t, ri, ro)
    prog = ops.Program()
    for inp, segs, kw in _mlp_calls(t, b, ri, ro):
        prog.add_gemv(inp, segs, **kw)
    prog.finalize()
    prog.set_option("prefetch_records", prefetch)
    for _ in range(5):
        for inp, segs, kw in _mlp_calls(t, a, ri, ro):
            ops.gemv_fused(inp, segs, **kw)
    prog.run(n_tokens=5)
    torch.cuda.synchronize()
    assert torch.equal(a["hidden"], b["hidden"]) and torch.equal(a["act"], b["act"])


def test_program_inproj_deltanet_outproj(cuda):
    """A DeltaNet block's first three operations as phases: in_proj with conv / decay / beta epilogues, the recurrent
    step, out_proj with the gated-norm prologue and the residual epilogue; two tokens, against the launches."""
    from insignia_b200 import mxfp4, ops

    rng = np.random.default_rng(102)
    wq, sq = rand_matrix(rng, 8192, 4096)
    wz, sz = rand_matrix(rng, 4096, 4096)
    wa, sa = rand_matrix(rng, 32, 4096, std=0.05)
    wb, sb = rand_matrix(rng, 32, 4096, std=0.05)
    wo, so = rand_matrix(rng, 4096, 4096)
    P = [ops.repack(dev(w), dev(s)) for w, s in ((wq, sq), (wz, sz), (wa, sa), (wb, sb), (wo, so))]
    conv_w = dev(mxfp4.f32_to_bf16_bits((0.5 * rng.standard_normal((8192, 4))).astype(np.float32)))
    A_log = dev(rng.uniform(-1, 1, 32).astype(np.float32))
    dt = dev(mxfp4.f32_to_bf16_bits((0.5 * rng.standard_normal(32)).astype(np.float32)))
    nw, dn_w = dev(bf16(rng, 4096)), dev(bf16(rng, 128))
    hidden0 = (rng.standard_normal(4096) * 2).astype(np.float32)
    state0 = (rng.standard_normal(32 * 128 * 128) * 0.05).astype(np.float32)

    def buffers():
        return dict(hidden=dev(hidden0.copy()), qkv=torch.zeros(8192, device="cuda"), z=torch.zeros(4096, device="cuda"),
                    a=torch.zeros(32, device="cuda"), b=torch.zeros(32, device="cuda"), core=torch.zeros(4096, device="cuda"),
                    conv=torch.zeros(8192 * 3, device="cuda"), state=dev(state0.copy()))

    def in_proj(x):
        return (x["hidden"], [dict(packed=P[0], out=x["qkv"], rows=8192, epilogue="conv_silu", conv_state=x["conv"], conv_w=conv_w),
                              dict(packed=P[1], out=x["z"], rows=4096, epilogue="store"),
                              dict(packed=P[2], out=x["a"], rows=32, epilogue="decay", A_log=A_log, dt_bias=dt),
                              dict(packed=P[3], out=x["b"], rows=32, epilogue="beta")], dict(prologue="rmsnorm", norm_w=nw))

    def out_proj(x):
        return (x["core"], [dict(packed=P[4], out=x["hidden"], rows=4096, epilogue="residual")],
                dict(prologue="gated_rmsnorm", aux=x["z"], norm_w=dn_w))

    a, b = buffers(), buffers()
    prog = ops.Program()
    inp, segs, kw = in_proj(b)
    prog.add_gemv(inp, segs, **kw)
    prog.add_deltanet(b["state"], b["qkv"], b["qkv"][2048:], b["qkv"][4096:], b["a"], b["b"], b["core"])
    inp, segs, kw = out_proj(b)
    prog.add_gemv(inp, segs, **kw)
    prog.finalize()
    for step in range(2):
        # the same inputs on both sides at every step (after a step they agree only to rounding, see below)
        b["hidden"].copy_(a["hidden"]), b["state"].copy_(a["state"])
        inp, segs, kw = in_proj(a)
        ops.gemv_fused(inp, segs, **kw)
        core = ops.deltanet_decode(a["state"], a["qkv"], a["qkv"][2048:], a["qkv"][4096:], a["a"], a["b"])
        a["core"].copy_(core)
        inp, segs, kw = out_proj(a)
        ops.gemv_fused(inp, segs, **kw)
        prog.run()
        torch.cuda.synchronize()
        for name in ("qkv", "z", "a", "b", "conv"):  # GEMV phases: the same bits
            assert torch.equal(a[name], b[name]), (step, name)
        for name in ("core", "state", "hidden"):  # the recurrent step sums over 16 warps instead of 8
            x, y = host(a[name]), host(b[name])
            assert np.max(np.abs(x - y)) <= 1e-5 * max(1.0, np.abs(x).max()), (step, name)
    # the DeltaNet phase against the oracle, from the launch path's inputs of the last step
    st = state0.copy()
    # (state after two steps was compared to the launch path above, which has its own oracle tests)
    assert np.all(np.isfinite(host(b["state"]))) and not np.array_equal(host(b["state"]), st)


@pytest.mark.parametrize("kv_bf16", [False, True])
def test_program_attention_phase_sequence_vs_oracle(cuda, kv_bf16):
    """The attention phase (norm + RoPE + cache write + split-K attention) over consecutive positions, run as a one-phase
    program whose launch sets the position every CTA then reads, against the unfused oracle chain."""
    from insignia_b200 import ops

    rng = np.random.default_rng(103)
    ctx = 160
    qw, kw = bf16(rng, 256), bf16(rng, 256)
    kc = torch.zeros(ctx * 1024, device="cuda", dtype=torch.bfloat16 if kv_bf16 else torch.float32)
    vc = torch.zeros_like(kc)
    kc_ref, vc_ref = np.zeros(ctx * 1024, np.float32), np.zeros(ctx * 1024, np.float32)
    scratch = ops.gqa_scratch("cuda")
    pos_dev = torch.zeros(1, dtype=torch.int32, device="cuda")
    qraw_d, kraw_d, v_d = torch.zeros(8192, device="cuda"), torch.zeros(1024, device="cuda"), torch.zeros(1024, device="cuda")
    out = torch.zeros(4096, device="cuda")
    prog = ops.Program()
    prog.add_attention(qraw_d, kraw_d, v_d, dev(qw), dev(kw), kc, vc, out, pos_dev, ctx, scratch, fast_trig=False)
    prog.finalize()
    for pos in range(0, 150):
        qraw = rng.standard_normal(8192).astype(np.float32)
        kraw = rng.standard_normal(1024).astype(np.float32)
        v = rng.standard_normal(1024).astype(np.float32)
        qraw_d.copy_(dev(qraw)), kraw_d.copy_(dev(kraw)), v_d.copy_(dev(v))
        prog.run(position=pos, device_position=pos_dev)
        q = np.ascontiguousarray(qraw.reshape(16, 512)[:, :256]).reshape(-1)
        k = kraw.copy()
        orc.qk_norm_rope(q, k, qw, kw, pos)
        if kv_bf16:
            k = host(dev(k).to(torch.bfloat16).float())
            v = host(dev(v).to(torch.bfloat16).float())
        orc.lib().orc_store_kv(k, v, kc_ref, vc_ref, pos)
        if pos % 7 == 0 or pos > 140 or pos < 40:
            want = orc.gqa_decode(q, kc_ref, vc_ref, pos + 1)
            assert np.max(np.abs(host(out) - want)) <= 5e-5, pos
    assert np.max(np.abs(host(kc.float())[:150 * 1024] - kc_ref[:150 * 1024])) <= (2.0 ** -7 * np.abs(kc_ref).max() if kv_bf16 else 5e-5)
    assert int(scratch[:16].view(torch.int32).abs().sum().item()) == 0  # tickets left at zero


def test_program_embed_and_logits_feedback(cuda):
    """Embedding lookup -> lm_head-style GEMV with arg-max feedback, three tokens in one launch: token ids, log and position
    as from the launches."""
    from insignia_b200 import ops

    rng = np.random.default_rng(104)
    vocab = 16 * 40
    we, se = rand_matrix(rng, vocab, 4096, std=1.0)
    wl, sl = rand_matrix(rng, vocab, 4096)
    Pl = ops.repack(dev(wl), dev(sl))
    nw = dev(bf16(rng, 4096))
    d_we, d_se = dev(we), dev(se)

    def buffers():
        return dict(hidden=torch.zeros(4096, device="cuda"), logits=torch.zeros(vocab, device="cuda"), scratch=ops.argmax_scratch("cuda"),
                    tok=torch.tensor([17], dtype=torch.int32, device="cuda"), nxt=torch.full((1,), -1, dtype=torch.int32, device="cuda"),
                    log=torch.full((8,), -1, dtype=torch.int32, device="cuda"), pos=torch.tensor([2], dtype=torch.int32, device="cuda"))

    def head(x):
        return (x["hidden"], [dict(packed=Pl, out=x["logits"], rows=vocab, epilogue="logits")],
                dict(prologue="rmsnorm", norm_w=nw, argmax=dict(scratch=x["scratch"], token_out=x["nxt"], token_feedback=x["tok"],
                                                                 token_log=x["log"], position=x["pos"])))

    a, b = buffers(), buffers()
    for _ in range(3):
        a["hidden"].copy_(ops.get_row_mlx(d_we, d_se, int(a["tok"].item())))
        inp, segs, kw = head(a)
        ops.gemv_fused(inp, segs, **kw)
    prog = ops.Program()
    prog.add_embed(d_we, d_se, b["hidden"], b["tok"])
    inp, segs, kw = head(b)
    prog.add_gemv(inp, segs, **kw)
    prog.finalize()
    b["tok"].fill_(99)  # overwritten by the kernel: the first token comes in as an argument
    b["pos"].fill_(0)
    prog.run(n_tokens=3, token=17, position=2, device_token=b["tok"], device_position=b["pos"])
    torch.cuda.synchronize()
    for name in ("hidden", "logits", "tok", "nxt", "log", "pos"):
        assert torch.equal(a[name], b[name]), name
    assert int(b["pos"].item()) == 5 and host(b["log"])[2:5].min() >= 0 and int(host(b["log"])[5]) == -1


def test_program_barrier_wait_runs_out(cuda):
    """A grid barrier that can never be met (it waits for one CTA more than the grid has) gives up after its time limit,
    raises the error status and every CTA returns; after recover() the program runs normally again."""
    from insignia_b200 import ops

    rng = np.random.default_rng(105)
    ri, ro = 768, 4096
    t = _mlp_ops(rng, ri, ro)
    a, b = _mlp_buffers(t, ri, ro), _mlp_buffers(t, ri, ro)
    prog = ops.Program()
    for inp, segs, kw in _mlp_calls(t, b, ri, ro):
        prog.add_gemv(inp, segs, **kw)
    prog.finalize()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    prog.selftest_barrier_timeout(1_000_000, err)  # 1 ms
    torch.cuda.synchronize()
    assert int(err.item()) == 1
    err.zero_()
    prog.recover()
    b["hidden"].copy_(dev(t["hidden0"]))
    for inp, segs, kw in _mlp_calls(t, a, ri, ro):
        ops.gemv_fused(inp, segs, **kw)
    prog.run(error_flag=err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0 and torch.equal(a["hidden"], b["hidden"])


def test_engine_selftest_and_recovery(cuda, golden_ckpt):
    """The engine reports the expired wait and decodes correctly afterwards."""
    from insignia_b200.engine import Engine

    with Engine(golden_ckpt[1], n_layers=4, vocab=64, max_context=64, persistent=True) as e, \
            Engine(golden_ckpt[1], n_layers=4, vocab=64, max_context=64, persistent=True) as ref:
        want = [ref.decode_token(t) for t in (42, 7, 63)]
        assert e.decode_token(42) == want[0]
        assert e.selftest_barrier_timeout() is True
        e.reset()
        assert [e.decode_token(t) for t in (42, 7, 63)] == want
        assert np.array_equal(e.read("hidden"), ref.read("hidden"))
