"""The several-token tcgen05 GEMM (eight or sixteen tokens per kind::mxf4 instruction, stream-K shares), through the C ABI, against the CPU oracle
and against the one-token kernels."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
from oracle import oracle as orc  # noqa: E402
from tests.test_kernels_gpu import bf16, dev, host, rand_matrix  # noqa: E402

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.mark.parametrize("rows,cols,M", [(256, 4096, 8), (4096, 4096, 16), (1024, 12288, 64), (2048, 1152, 5), (48, 128, 1), (128 * 150, 256, 19),
                                         (12352, 4096, 24)])
def test_gemm_umma_vs_oracle(cuda, rows, cols, M):
    from insignia_b200 import ops

    rng = np.random.default_rng(rows + cols + M)
    w, s = rand_matrix(rng, rows, cols)
    # tokens of very different magnitudes: every token has its own fixed-point scale
    x = (rng.standard_normal((M, cols)) * rng.uniform(0.01, 30, (M, 1))).astype(np.float32)
    P = ops.repack_umma(dev(w), dev(s))
    y = host(ops.gemm_umma(P, dev(x)))
    assert y.shape == (M, rows)
    for m in range(M):
        y64 = orc.gemv_mlx_f64(w, s, x[m])
        assert np.max(np.abs(y[m] - y64)) <= 4e-6 * np.abs(y64).max() + 1e-7, m
    # a token's result does not depend on which tokens travel with it
    y1 = host(ops.gemm_umma(P, dev(x[M - 1:M])))
    assert np.max(np.abs(y1[0] - y[M - 1])) <= 1e-6 * np.abs(y[M - 1]).max()


@pytest.mark.parametrize("rows,cols,M", [(128 * 37, 512, 16), (4096, 4096, 8), (640, 12288, 40)])
def test_gemm_umma_is_deterministic_across_cut_units(cuda, rows, cols, M):
    """Units cut by share boundaries are summed in share order by whichever CTA arrives last: repeated calls must agree
    bit for bit (shapes chosen so that most units are cut, some into many parts)."""
    from insignia_b200 import ops

    rng = np.random.default_rng(rows + M)
    w, s = rand_matrix(rng, rows, cols)
    x = dev((rng.standard_normal((M, cols)) * 2).astype(np.float32))
    P = ops.repack_umma(dev(w), dev(s))
    scratch = ops.umma_gemm_scratch(cols, M)
    first = host(ops.gemm_umma(P, x, scratch=scratch))
    for _ in range(5):
        assert np.array_equal(host(ops.gemm_umma(P, x, scratch=scratch)), first)
    y64 = orc.gemv_mlx_f64(w, s, host(x)[M - 1])
    assert np.max(np.abs(first[M - 1] - y64)) <= 4e-6 * np.abs(y64).max()


def test_gemm_umma_extreme_tokens(cuda):
    from insignia_b200 import ops

    rng = np.random.default_rng(7)
    rows, cols = 256, 1024
    w, s = rand_matrix(rng, rows, cols)
    P = ops.repack_umma(dev(w), dev(s))
    x = np.stack([np.zeros(cols, np.float32), np.eye(1, cols, 7, dtype=np.float32)[0] * 3e4, (rng.standard_normal(cols) * 1e-12).astype(np.float32),
                  np.where(np.arange(cols) % 97 == 0, 1000.0, 1e-3).astype(np.float32), rng.standard_normal(cols).astype(np.float32)])
    y = host(ops.gemm_umma(P, dev(x)))
    assert np.all(np.isfinite(y))
    for m in range(x.shape[0]):
        y64 = orc.gemv_mlx_f64(w, s, x[m])
        assert np.max(np.abs(y[m] - y64)) <= 4e-6 * max(np.abs(y64).max(), 1e-30), m


def test_gemm_umma_fused_inproj_over_sixteen_tokens(cuda):
    """in_proj(qkv|z|a|b) for sixteen consecutive tokens in one call: RMSNorm prologue per token, conv + SiLU with the
    history carried through the tokens in order, store, decay, beta (src/decode.cu:14-16 applied token by token)."""
    from insignia_b200 import mxfp4, ops

    rng = np.random.default_rng(31)
    nq, T = 384, 16
    wq, sq = rand_matrix(rng, nq, 4096)
    wz, sz = rand_matrix(rng, 256, 4096)
    wa, sa = rand_matrix(rng, 32, 4096, std=0.05)
    wb, sb = rand_matrix(rng, 32, 4096, std=0.05)
    conv_w = mxfp4.f32_to_bf16_bits((0.5 * rng.standard_normal((nq, 4))).astype(np.float32))
    A_log = rng.uniform(-1, 1, 32).astype(np.float32)
    dt = mxfp4.f32_to_bf16_bits((0.5 * rng.standard_normal(32)).astype(np.float32))
    nw = bf16(rng, 4096)
    P = [ops.repack_umma(dev(w), dev(s)) for w, s in ((wq, sq), (wz, sz), (wa, sa), (wb, sb))]
    state0 = (rng.standard_normal(nq * 3) * 0.3).astype(np.float32)
    conv_state = dev(state0.copy())
    o_q, o_z = torch.zeros(T * nq, device="cuda"), torch.zeros(T * 256, device="cuda")
    o_a, o_b = torch.zeros(T * 32, device="cuda"), torch.zeros(T * 32, device="cuda")
    hidden = (rng.standard_normal((T, 4096)) * 3).astype(np.float32)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    scratch = ops.umma_gemm_scratch(4096, T)
    ops.gemv_fused(dev(hidden), [
        dict(packed=P[0], out=o_q, rows=nq, epilogue="conv_silu", conv_state=conv_state, conv_w=dev(conv_w)),
        dict(packed=P[1], out=o_z, rows=256, epilogue="store"),
        dict(packed=P[2], out=o_a, rows=32, epilogue="decay", A_log=dev(A_log), dt_bias=dev(dt)),
        dict(packed=P[3], out=o_b, rows=32, epilogue="beta")], prologue="rmsnorm", norm_w=dev(nw), layout=1, error_flag=err, tokens=T,
        cols=4096, umma_scratch=scratch)
    ref_state = state0.copy()
    gq, gz, ga, gb = host(o_q).reshape(T, nq), host(o_z).reshape(T, 256), host(o_a).reshape(T, 32), host(o_b).reshape(T, 32)
    for m in range(T):
        n = orc.rmsnorm_bf16(hidden[m], nw)
        q = orc.gemv_mlx(wq, sq, n)
        orc.causal_conv4_silu(q, ref_state, conv_w)
        a, b = orc.gemv_mlx(wa, sa, n), orc.gemv_mlx(wb, sb, n)
        orc.deltanet_parameters(a, b, A_log, dt)
        assert np.max(np.abs(gq[m] - q)) <= 2e-5 * max(1.0, np.abs(q).max()), m
        assert np.max(np.abs(gz[m] - orc.gemv_mlx(wz, sz, n))) <= 2e-5, m
        assert np.max(np.abs(ga[m] - a)) <= 2e-5 * max(1.0, np.abs(a).max()), m
        assert np.max(np.abs(gb[m] - b)) <= 2e-6, m
    assert np.max(np.abs(host(conv_state) - ref_state)) <= 2e-5 * np.abs(ref_state).max()
    assert int(err.item()) == 0


def test_gemm_umma_fused_swiglu_and_residual_over_tokens(cuda):
    from insignia_b200 import ops

    rng = np.random.default_rng(32)
    T = 11
    wg, sg = rand_matrix(rng, 768, 4096)
    wu, su = rand_matrix(rng, 768, 4096)
    wd, sd = rand_matrix(rng, 256, 768)
    hidden = (rng.standard_normal((T, 4096)) * 3).astype(np.float32)
    nw = bf16(rng, 4096)
    act = torch.zeros(T * 768, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.gemv_fused(dev(hidden), [dict(packed=ops.repack_umma(dev(wg), dev(sg)), packed2=ops.repack_umma(dev(wu), dev(su)), out=act, rows=768,
                                      epilogue="swiglu")], prologue="rmsnorm", norm_w=dev(nw), layout=1, error_flag=err, tokens=T, cols=4096,
                   umma_scratch=ops.umma_gemm_scratch(4096, T))
    res0 = rng.standard_normal((T, 256)).astype(np.float32)
    out = dev(res0.copy())
    ops.gemv_fused(act, [dict(packed=ops.repack_umma(dev(wd), dev(sd)), out=out, rows=256, epilogue="residual")], layout=1, error_flag=err,
                   tokens=T, cols=768, umma_scratch=ops.umma_gemm_scratch(768, T))
    got_act, got_out = host(act).reshape(T, 768), host(out).reshape(T, 256)
    for m in range(T):
        n = orc.rmsnorm_bf16(hidden[m], nw)
        g, u = orc.gemv_mlx(wg, sg, n), orc.gemv_mlx(wu, su, n)
        want = (g / (1 + np.exp(-g)) * u).astype(np.float32)
        assert np.max(np.abs(got_act[m] - want)) <= 2e-5 * np.abs(want).max(), m
        y = orc.gemv_mlx_f64(wd, sd, got_act[m])
        assert np.max(np.abs(got_out[m] - (res0[m] + y))) <= 6e-6 * max(np.abs(y).max(), 1.0), m
    assert int(err.item()) == 0
    # argument checks
    with pytest.raises(Exception, match="scratch"):
        ops.gemv_fused(act, [dict(packed=ops.repack_umma(dev(wd), dev(sd)), out=out, rows=256, epilogue="residual")], layout=1, tokens=T, cols=768)
