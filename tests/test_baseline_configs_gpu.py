"""The benchmark's named configurations 0-2 as parity cases (seeded synthetic inputs of their shapes).

0: one gated-DeltaNet layer with the model's layer-0 shapes, norms 1, 64 bf16 N(0,1) hidden vectors fed one after the
   other: every output and the final recurrent state against the CPU oracle.
1: MXFP4 weight x activation products for the four shapes and M = 1, 4, 16, 64: sampled rows against double
   accumulation, the full product through linearity.
2: the layer-3 attention decode at contexts 1024 / 8192 / 32768 over a bf16 cache, one and eight sequences.
"""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
from oracle import oracle as orc  # noqa: E402

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def bf16_round(a):
    from insignia_b200 import mxfp4

    return mxfp4.bf16_bits_to_f32(mxfp4.f32_to_bf16_bits(np.asarray(a, np.float32)))


def dev(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).cuda()
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).cuda()
    return torch.from_numpy(a).cuda()


# ---------------------------------------------------------------------------------------------- configs[0]
def test_config0_deltanet_layer_64_tokens(cuda, workdir):
    from insignia_b200 import synth
    from insignia_b200.checkpoint_io import SafetensorsReader
    from insignia_b200.engine import Engine

    st, idx = os.path.join(workdir, "cfg0.safetensors"), os.path.join(workdir, "cfg0.idx")
    synth.write_checkpoint(synth.SynthConfig(layers=(0,), vocab_rows=64, mtp=False, lm_head=True, seed=0, norms="ones"), st, idx)
    rng = np.random.default_rng(0)
    xs = bf16_round(rng.standard_normal((64, 4096)))
    ref = orc.OracleModel(SafetensorsReader(st), max_context=8, n_layers=1)
    worst = 0.0
    with Engine(idx, max_context=8, n_layers=1, vocab=64, use_graph=False) as e:
        for t in range(64):
            e.write("hidden", xs[t])
            e.layer(0)
            ref.hidden = xs[t].copy()
            ref.layer(0)
            got, want = e.read("hidden"), ref.hidden
            cosv = float(got @ want / np.linalg.norm(got) / np.linalg.norm(want))
            rel = float(np.max(np.abs(got - want)) / np.abs(want).max())
            assert cosv >= 0.9999 and rel <= 2e-2, (t, cosv, rel)
            worst = max(worst, rel)
        state, conv = e.read("delta_state", 32 * 128 * 128), e.read("conv_state", 8192 * 3)
    assert worst <= 2e-4, worst  # measured: a few 1e-6
    assert np.max(np.abs(state - ref.delta_state[0])) <= 1e-4 * np.abs(ref.delta_state[0]).max()
    assert np.max(np.abs(conv - ref.conv_state[0])) <= 1e-5 * np.abs(ref.conv_state[0]).max()


# ---------------------------------------------------------------------------------------------- configs[1]
def _quantised(rows, cols, seed):
    """rows x cols N(0, 0.02) -> MXFP4 on the GPU (a 248320 x 4096 matrix takes seconds there, minutes in NumPy)."""
    from insignia_b200 import synth

    g = torch.Generator(device="cuda").manual_seed(seed)
    v = torch.randn(rows, cols, generator=g, device="cuda") * 0.02
    w, s = synth.quantize_rows_torch(v)
    return w, s


@pytest.mark.parametrize("rows,cols", [(24576, 4096), (4096, 12288), (4096, 4096), (248320, 4096)])
def test_config1_matmul_shapes_and_token_counts(cuda, rows, cols):
    from insignia_b200 import mxfp4, ops

    w, s = _quantised(rows, cols, seed=rows + cols)
    packed = ops.repack(w, s)
    tiles = ops.repack_umma(w, s)  # the same matrix in the tcgen05 kernel's layout (16 and 64 tokens go through it too)
    rng = np.random.default_rng(1)
    sample = np.sort(rng.choice(rows, 512, replace=False))
    pick = torch.from_numpy(sample).cuda()
    wn = np.ascontiguousarray(w[pick].cpu().numpy()).view(np.uint32)
    sn = np.ascontiguousarray(s[pick].cpu().numpy())
    deq = mxfp4.dequantize(wn, sn).astype(np.float64)
    del w, s
    for M in (1, 4, 16, 64):
        x = bf16_round(rng.standard_normal((M, cols)))
        y = ops.gemv_packed(packed, dev(x)).cpu().numpy().reshape(M, rows)
        want = x.astype(np.float64) @ deq.T  # [M][512]
        err = np.max(np.abs(y[:, sample] - want)) / np.abs(want).max()
        assert err <= 4e-6, (M, err)  # fp32 accumulation of exact products
        # "bf16 out": rounded to bf16 the two agree to one unit in the last place of the largest value
        assert np.max(np.abs(bf16_round(y[:, sample]) - bf16_round(want.astype(np.float32)))) <= 2.0 ** -7 * np.abs(want).max()
        if M >= 4:
            # linearity over the whole matrix: W(x0 + x1) = W x0 + W x1 (bf16 inputs whose sum is exact in fp32)
            z = ops.gemv_packed(packed, dev(x[0] + x[1])).cpu().numpy()
            assert np.max(np.abs(z - (y[0] + y[1]))) <= 1e-5 * np.abs(z).max()
        # a token's result does not depend on how many tokens travel with it
        y1 = ops.gemv_packed(packed, dev(x[M - 1])).cpu().numpy()
        assert np.array_equal(y1, y[M - 1])
        if M >= 16:
            # the tcgen05 kind::mxf4 kernel (sixteen tokens per instruction, stream-K shares): same bar on the sampled rows,
            # and the whole matrix against the mma.sync kernel's result
            yt = ops.gemm_umma(tiles, dev(x)).cpu().numpy().reshape(M, rows)
            err_t = np.max(np.abs(yt[:, sample] - want)) / np.abs(want).max()
            assert err_t <= 4e-6, (M, err_t)
            assert np.max(np.abs(yt - y)) <= 4e-6 * np.abs(y).max()


# ---------------------------------------------------------------------------------------------- configs[2]
@pytest.mark.parametrize("ctx", [1024, 8192, 32768])
def test_config2_attention_decode_bf16_cache(cuda, ctx):
    from insignia_b200 import ops

    rng = np.random.default_rng(ctx)
    B = 8 if ctx <= 8192 else 2  # eight sequences at the two shorter contexts; the CPU check of 32768 x 8 would take minutes
    for b in range(B):
        kc, vc = bf16_round(rng.standard_normal(ctx * 1024)), bf16_round(rng.standard_normal(ctx * 1024))
        q = rng.standard_normal(4096).astype(np.float32)
        got = ops.gqa_decode(dev(q), dev(kc).to(torch.bfloat16), dev(vc).to(torch.bfloat16), ctx).cpu().numpy()
        want = orc.gqa_decode(q, kc, vc, ctx)
        assert np.max(np.abs(got - want)) <= 3e-5 * max(1.0, np.abs(want).max()), (ctx, b)
        if b == 0:  # the fp32 cache holds the same (bf16-exact) values: the two cache types must agree closely
            # (from 2048 cached rows on the bf16 cache runs on the tensor cores with the query and the weights as two bf16
            # pieces each: a different rounding than the fp32 loop, far inside the bar above)
            got32 = ops.gqa_decode(dev(q), dev(kc), dev(vc), ctx).cpu().numpy()
            assert np.max(np.abs(got32 - got)) <= (1e-6 if ctx < 2048 else 2e-5) * max(1.0, np.abs(got).max())


@pytest.mark.parametrize("kv_bf16", [True, False])
@pytest.mark.parametrize("ctx", [2048, 2049, 2063, 4100, 6001])
def test_attention_tensor_core_loop_ragged_lengths(cuda, ctx, kv_bf16):
    """The tensor-core loop of the bf16 cache (from 2048 rows on, 16 rows per warp step) at lengths that leave ragged last
    tiles and idle warps, with large scores (sharp softmax) in one head, against the CPU oracle; the row past the end must
    not leak in.  The fp32 cache (scalar loop at every length) runs the same cases."""
    from insignia_b200 import ops

    rng = np.random.default_rng(ctx)
    kc, vc = rng.standard_normal(ctx * 1024).astype(np.float32), (rng.standard_normal(ctx * 1024) * 3).astype(np.float32)
    if kv_bf16:
        kc, vc = bf16_round(kc), bf16_round(vc)
    dt = torch.bfloat16 if kv_bf16 else torch.float32
    q = rng.standard_normal(4096).astype(np.float32)
    q[:256] *= 6.0  # head 0: scores spread over +-6, the softmax picks a few rows
    kbig = torch.full(((ctx + 8) * 1024,), 1.0e4, device="cuda").to(dt)  # what lies past the end is poison
    vbig = torch.full(((ctx + 8) * 1024,), 1.0e4, device="cuda").to(dt)
    kbig[: ctx * 1024] = dev(kc).to(dt)
    vbig[: ctx * 1024] = dev(vc).to(dt)
    got = ops.gqa_decode(dev(q), kbig, vbig, ctx).cpu().numpy()
    want = orc.gqa_decode(q, kc, vc, ctx)
    assert np.all(np.isfinite(got))
    err = float(np.max(np.abs(got - want)) / max(1.0, np.abs(want).max()))
    print(f"ctx {ctx} {'bf16' if kv_bf16 else 'fp32'} cache: max error {err:.2e}")
    assert err <= 3e-5


def test_attention_step_bf16_long_context_fused_equals_unfused(cuda):
    """The fused step (norm, RoPE, cache write, attention) beyond 2048 rows on a bf16 cache: the row it has just written is
    fetched from the cache like every other; result against the unfused kernels on the updated cache."""
    from insignia_b200 import mxfp4, ops

    rng = np.random.default_rng(11)
    ctx, pos = 2600, 2500
    qw = mxfp4.f32_to_bf16_bits((1 + 0.1 * rng.standard_normal(256)).astype(np.float32))
    kw = mxfp4.f32_to_bf16_bits((1 + 0.1 * rng.standard_normal(256)).astype(np.float32))
    kc = torch.randn(ctx * 1024, device="cuda").to(torch.bfloat16)
    vc = torch.randn(ctx * 1024, device="cuda").to(torch.bfloat16)
    qraw, kraw, v = (dev(rng.standard_normal(n).astype(np.float32)) for n in (8192, 1024, 1024))
    pos_dev = torch.full((1,), pos, dtype=torch.int32, device="cuda")
    got = ops.attention_step(qraw, kraw, v, dev(qw), dev(kw), kc, vc, pos_dev, ctx, ops.gqa_scratch("cuda")).cpu().numpy()
    q = qraw.reshape(16, 512)[:, :256].contiguous().reshape(-1).clone()
    k = kraw.clone()
    ops.qk_norm_rope(q, k, dev(qw), dev(kw), pos)
    row = slice(pos * 1024, (pos + 1) * 1024)
    assert torch.equal(kc[row], k.to(torch.bfloat16)) and torch.equal(vc[row], v.to(torch.bfloat16))
    want = ops.gqa_decode(q, kc, vc, pos + 1).cpu().numpy()
    assert np.max(np.abs(got - want)) <= 1e-6 * max(1.0, np.abs(want).max())


def test_config2_attention_layer_with_rope_and_gate(cuda, golden_ckpt):
    """Layer 3 of the 4-layer checkpoint (layer-3 shapes): RMSNorm, q/k/v projections, q/k norm, partial RoPE (theta 1e7),
    cache write, attention, sigmoid gate, o_proj, MLP -- 40 consecutive positions with a bf16 cache against the oracle
    fed the same hidden states."""
    from insignia_b200.checkpoint_io import SafetensorsReader
    from insignia_b200.engine import Engine

    ref = orc.OracleModel(SafetensorsReader(golden_ckpt[0]), max_context=64, n_layers=4)
    rng = np.random.default_rng(3)
    with Engine(golden_ckpt[1], max_context=64, n_layers=4, vocab=64, kv_bf16=True, use_graph=False) as e:
        for t in range(40):
            x = bf16_round(rng.standard_normal(4096))
            e.write("hidden", x)
            e.position = t
            e.layer(3)
            ref.hidden, ref.position = x.copy(), t
            ref.layer(3)
            got, want = e.read("hidden"), ref.hidden
            cosv = float(got @ want / np.linalg.norm(got) / np.linalg.norm(want))
            rel = float(np.max(np.abs(got - want)) / np.abs(want).max())
            assert cosv >= 0.9999 and rel <= 2e-2, (t, cosv, rel)  # bf16 cache against the oracle's fp32 cache
