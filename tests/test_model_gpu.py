"""The decode engine (C++ host classes through the C ABI) on a 4-layer synthetic checkpoint:
against golden vectors from the reference's NumPy tools, the CPU oracle, and the compiled reference engine."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
from oracle import oracle as orc  # noqa: E402
from oracle import ref_engine as refengine  # noqa: E402

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def cos(a, b):
    return float(a @ b / np.linalg.norm(a) / np.linalg.norm(b))


def close(a, b, rel=2e-2):
    """north-star layer bar: cosine >= 0.9999 and max-abs-rel <= 2e-2 (relative to the largest reference element)."""
    return cos(a, b) >= 0.9999 and np.max(np.abs(a - b)) <= rel * np.abs(b).max()


def small_engine(idx, **kw):
    from insignia_b200.engine import Engine

    kw.setdefault("n_layers", 4)
    kw.setdefault("vocab", 64)
    kw.setdefault("max_context", 64)
    return Engine(idx, **kw)


def test_layers_match_numpy_tool_golden(cuda, golden_ckpt):
    gold = np.load(os.path.join(GOLD, "layers_tok42.npy"))
    with small_engine(golden_ckpt[1], gate_elementwise=True, use_graph=False) as e:
        e.embed(42)
        for l in range(4):
            e.layer(l)
            h = e.read("hidden")
            assert close(h, gold[l]), l
            assert np.max(np.abs(h - gold[l])) <= 1e-4 * np.abs(gold[l]).max(), l


# (persistent token kernel?, graph, dependent launch): the three launch-per-operation forms, then the persistent kernel
MODES = [(False, False, False), (False, False, True), (False, True, True), (True, False, False)]


@pytest.mark.parametrize("persistent,graph,pdl", MODES)
def test_multi_token_decode_vs_oracle(cuda, golden_ckpt, persistent, graph, pdl):
    from insignia_b200.checkpoint_io import SafetensorsReader

    m = orc.OracleModel(SafetensorsReader(golden_ckpt[0]), max_context=64, gate="broadcast", n_layers=4)
    tokens = [42, 7, 63, 0, 21, 5, 33, 60, 1, 2]
    with small_engine(golden_ckpt[1], persistent=persistent, use_graph=graph, use_pdl=pdl) as e:
        for i, t in enumerate(tokens):
            got = e.decode_token(t)
            want = m.decode_token(t)
            h, lg = e.read("hidden"), e.read("logits")
            assert close(h, m.hidden, 1e-3), i
            assert np.max(np.abs(lg - m.logits[:64])) <= 1e-3 * np.abs(m.logits).max(), i
            assert got == want == int(np.argmax(lg)), i
            assert e.position == m.position == i + 1
        ds = e.read("delta_state", 3 * 32 * 128 * 128)
        assert np.max(np.abs(ds - m.delta_state[:3].reshape(-1))) <= 1e-3 * np.abs(m.delta_state[:3]).max()
        cs = e.read("conv_state", 3 * 8192 * 3)
        assert np.max(np.abs(cs - m.conv_state[:3].reshape(-1))) <= 1e-3 * np.abs(m.conv_state[:3]).max()
        assert e.launch_count > 0


def _run_tokens(idx, graph, pdl, use_generate, persistent=False):
    with small_engine(idx, persistent=persistent, use_graph=graph, use_pdl=pdl) as e:
        for t in (3, 9):
            e.forward_token(t)
        first = e.logits_argmax()
        if use_generate:
            toks = e.generate(first, 20)
        else:
            toks, t = [], first
            for _ in range(20):
                t = e.decode_token(t)
                toks.append(t)
        assert e.position == 22
        return toks, e.read("hidden"), e.read("delta_state", 3 * 32 * 128 * 128)


def test_generate_equals_decode_token_loop_bitwise(cuda, golden_ckpt):
    """Graph replay, programmatic dependent launch and device-side token feedback must not change a single bit:
    the kernels and their order are the same in every mode."""
    base = _run_tokens(golden_ckpt[1], False, False, False)
    for graph, pdl, gen in [(False, False, False), (False, True, False), (True, False, False), (True, True, False),
                            (True, True, True), (False, True, True), (True, True, True)]:
        toks, hidden, state = _run_tokens(golden_ckpt[1], graph, pdl, gen)
        assert toks == base[0], (graph, pdl, gen)
        assert np.array_equal(hidden, base[1]), (graph, pdl, gen, float(np.abs(hidden - base[1]).max()))
        assert np.array_equal(state, base[2]), (graph, pdl, gen)
    # The persistent token kernel: one launch per token (decode_token loop) and one launch for all twenty tokens
    # (generate) are bit-identical to each other.  Against the launch-per-operation path the GEMVs are bit-identical
    # too, while the DeltaNet and attention phases reduce over 16 warps instead of 8: same tokens, state within rounding.
    pa = _run_tokens(golden_ckpt[1], False, False, False, persistent=True)
    pb = _run_tokens(golden_ckpt[1], False, False, True, persistent=True)
    assert pa[0] == pb[0] == base[0]
    assert np.array_equal(pa[1], pb[1]) and np.array_equal(pa[2], pb[2])
    assert np.max(np.abs(pa[1] - base[1])) <= 2e-5 * np.abs(base[1]).max()
    assert np.max(np.abs(pa[2] - base[2])) <= 2e-5 * np.abs(base[2]).max()


def test_tcgen05_and_mma_sync_gemv_paths_agree(cuda, golden_ckpt):
    """The two GEMV kernels (tcgen05 kind::mxf4 with a fixed-point activation, mma.sync with an fp16-pair activation)
    decode the same tokens and stay within rounding of each other."""
    from insignia_b200.checkpoint_io import SafetensorsReader

    m = orc.OracleModel(SafetensorsReader(golden_ckpt[0]), max_context=64, gate="broadcast", n_layers=4)
    with small_engine(golden_ckpt[1], gemv_tcgen05=True) as a, small_engine(golden_ckpt[1], gemv_tcgen05=False) as b:
        for i, t in enumerate([42, 7, 63, 0, 21, 5, 33, 60]):
            ta, tb, tm = a.decode_token(t), b.decode_token(t), m.decode_token(t)
            assert ta == tb == tm, i
            ha, hb = a.read("hidden"), b.read("hidden")
            assert np.max(np.abs(ha - hb)) <= 2e-4 * np.abs(hb).max(), i
            assert close(ha, m.hidden, 1e-3) and close(hb, m.hidden, 1e-3), i


def test_prepared_inputs_on_and_off_agree(cuda, golden_ckpt):
    """With prepared inputs each residual / SwiGLU launch hands the next GEMV its input as fp16 pieces plus sums of
    squares; without, every GEMV normalises and converts for itself.  Same tokens, hidden states within rounding, and
    both within the oracle's tolerance."""
    from insignia_b200.checkpoint_io import SafetensorsReader

    m = orc.OracleModel(SafetensorsReader(golden_ckpt[0]), max_context=64, gate="broadcast", n_layers=4)
    with small_engine(golden_ckpt[1], prepared_inputs=True) as a, small_engine(golden_ckpt[1], prepared_inputs=False) as b:
        for i, t in enumerate([42, 7, 63, 0, 21, 5, 33, 60, 11, 12]):
            ta, tb, tm = a.decode_token(t), b.decode_token(t), m.decode_token(t)
            assert ta == tb == tm, i
            ha, hb = a.read("hidden"), b.read("hidden")
            assert np.max(np.abs(ha - hb)) <= 1e-4 * np.abs(hb).max(), i
            assert close(ha, m.hidden, 1e-3) and close(hb, m.hidden, 1e-3), i
        # the per-layer entry points take hidden from the caller: they must not read a stale prepared image
        a.write("hidden", b.read("hidden") * 0.5)
        b.write("hidden", b.read("hidden") * 0.5)
        for l in range(4):
            a.layer(l), b.layer(l)
        assert np.max(np.abs(a.read("hidden") - b.read("hidden"))) <= 1e-4 * np.abs(b.read("hidden")).max()


@pytest.mark.parametrize("count", [1, 2, 7, 13])
def test_forward_tokens_equals_token_loop(cuda, golden_ckpt, count):
    """Prompt processing four tokens per pass over the weights: the same state as forward_token in a loop (bit for bit
    without prepared inputs, which only the one-token path uses; within rounding of the default path), the same
    arg-max, and decoding continues identically afterwards."""
    prompt = [42, 7, 63, 0, 21, 5, 33, 60, 11, 12, 1, 2, 3][:count]
    with small_engine(golden_ckpt[1], prepared_inputs=False) as a, small_engine(golden_ckpt[1], prepared_inputs=False) as b, \
            small_engine(golden_ckpt[1]) as c:
        a.forward_tokens(prompt)
        for t in prompt:
            b.forward_token(t)
            c.forward_token(t)
        assert a.position == b.position == count
        for field, n in (("hidden", 4096), ("delta_state", 3 * 32 * 128 * 128), ("conv_state", 3 * 8192 * 3), ("kv_keys", count * 1024),
                         ("kv_values", count * 1024)):
            assert np.array_equal(a.read(field, n), b.read(field, n)), field
        assert np.max(np.abs(a.read("hidden") - c.read("hidden"))) <= 1e-4 * np.abs(c.read("hidden")).max()
        ta, tb = a.logits_argmax(), b.logits_argmax()
        assert ta == tb == c.logits_argmax()
        assert np.array_equal(a.read("logits", 64), b.read("logits", 64))
        for _ in range(5):  # decoding goes on from the prompt's state
            ta, tb = a.decode_token(ta), b.decode_token(tb)
            assert ta == tb
        assert np.array_equal(a.read("hidden"), b.read("hidden"))
    with small_engine(golden_ckpt[1], max_context=8) as e:
        with pytest.raises(Exception, match="KV cache full"):
            e.forward_tokens(list(range(9)))
        with pytest.raises(Exception, match="token out of range"):
            e.forward_tokens([1, 248320])


@pytest.mark.parametrize("count", [16, 37, 50, 300])
def test_forward_tokens_through_tcgen05_passes(cuda, golden_ckpt, count):
    """Prompts of 16 tokens or more go through the tcgen05 kernel in passes of up to 256 tokens (the rest in passes of
    four; 300 tokens = a full pass, a second one of 44): the same state as the token loop to rounding, the same arg-max,
    and decoding continues with the same tokens."""
    rng = np.random.default_rng(count)
    prompt = [int(t) for t in rng.integers(0, 64, count)]
    ctx = max(64, count + 8)
    with small_engine(golden_ckpt[1], max_context=ctx) as a, small_engine(golden_ckpt[1], max_context=ctx, prefill_tcgen05=False) as b, \
            small_engine(golden_ckpt[1], max_context=ctx) as c:
        a.forward_tokens(prompt)
        b.forward_tokens(prompt)
        for t in prompt:
            c.forward_token(t)
        assert a.position == b.position == c.position == count
        for field, n in (("hidden", 4096), ("delta_state", 3 * 32 * 128 * 128), ("conv_state", 3 * 8192 * 3), ("kv_keys", count * 1024),
                         ("kv_values", count * 1024)):
            ra, rc = a.read(field, n), c.read(field, n)
            assert np.max(np.abs(ra - rc)) <= 2e-4 * max(np.abs(rc).max(), 1e-6), field
            assert np.max(np.abs(b.read(field, n) - rc)) <= 2e-4 * max(np.abs(rc).max(), 1e-6), field
        ta = a.logits_argmax()
        assert ta == b.logits_argmax() == c.logits_argmax()
        tc = ta
        for _ in range(6):
            ta, tc = a.decode_token(ta), c.decode_token(tc)
            assert ta == tc


def test_kv_bf16_and_accurate_trig_modes(cuda, golden_ckpt):
    from insignia_b200.checkpoint_io import SafetensorsReader

    m = orc.OracleModel(SafetensorsReader(golden_ckpt[0]), max_context=64, gate="elementwise", n_layers=4)
    with small_engine(golden_ckpt[1], gate_elementwise=True, accurate_trig=True) as e32, \
            small_engine(golden_ckpt[1], gate_elementwise=True, accurate_trig=True, kv_bf16=True) as e16:
        for i, t in enumerate([42, 7, 63, 0, 21, 5]):
            m.forward_token(t)
            e32.forward_token(t), e16.forward_token(t)
            assert close(e32.read("hidden"), m.hidden, 1e-4), i
            assert close(e16.read("hidden"), m.hidden, 2e-2), i


def test_engine_errors_follow_reference(cuda, golden_ckpt):
    from insignia_b200.engine import InsigniaError

    with small_engine(golden_ckpt[1], max_context=2) as e:
        with pytest.raises(InsigniaError, match="not a DeltaNet layer"):
            e.layer(32)
        with pytest.raises(InsigniaError, match="token out of range"):
            e.forward_token(248320)
        with pytest.raises(InsigniaError, match="token out of range"):
            e.embed(-1)
        e.forward_token(1), e.forward_token(2)
        with pytest.raises(InsigniaError, match="KV cache full"):
            e.forward_token(3)
        e.reset()
        assert e.position == 0
        e.forward_token(1)
    with pytest.raises(InsigniaError, match="cannot open Insignia index"):
        small_engine("/nonexistent.idx")


def test_storage_budget_eviction_error(cuda, golden_ckpt):
    """A budget below one tensor throws like the reference (src/storage.cu:8)."""
    from insignia_b200.engine import InsigniaError

    with small_engine(golden_ckpt[1], budget_bytes=1 << 20, use_graph=False) as e:
        with pytest.raises(InsigniaError, match="tensor exceeds device budget"):
            e.embed(1)
            e.layer(0)


@pytest.mark.skipif(not refengine.available(), reason="compiled reference (oracle/_ref) not built")
def test_layers_vs_compiled_reference_engine(cuda, golden_ckpt):
    """The reference's own engine (unmodified sources) driven like src/dump_layers.cu:5 / src/test_full_model.cu:6:
    embed, layers 0..3, position++, for several tokens; same calls on this engine."""
    ref = refengine.RefEngine(golden_ckpt[1], max_context=64)
    try:
        with small_engine(golden_ckpt[1], use_graph=False) as e:
            for i, t in enumerate([42, 7, 63, 0, 21, 5, 33, 11]):
                ref.embed(t), e.embed(t)
                for l in range(4):
                    ref.layer(l), e.layer(l)
                    a, b = e.read("hidden"), ref.read("hidden", 4096)
                    assert close(a, b, 1e-3), (i, l)
                    assert np.max(np.abs(a - b)) <= 2e-4 * np.abs(b).max(), (i, l)
                ref.position = ref.position + 1
                e.position = e.position + 1
            ds, dr = e.read("delta_state", 3 * 32 * 128 * 128), ref.read("delta_state", 3 * 32 * 128 * 128)
            assert np.max(np.abs(ds - dr)) <= 2e-4 * np.abs(dr).max()
    finally:
        ref.close()
