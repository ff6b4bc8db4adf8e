"""Decode batches: several sequences in lock step on one weight copy give, sequence by sequence, what the single-sequence
engine gives."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))

pytestmark = pytest.mark.gpu


def small_engine(idx, **kw):
    from insignia_b200.engine import Engine

    kw.setdefault("n_layers", 4)
    kw.setdefault("vocab", 64)
    kw.setdefault("max_context", 64)
    return Engine(idx, **kw)


@pytest.mark.parametrize("sequences", [1, 2, 3, 4, 5, 8])
def test_batch_equals_independent_engines(cuda, golden_ckpt, sequences):
    """Every sequence of a batch decodes the tokens the single-sequence engine decodes from the same prompt; states agree
    to rounding (1..4 sequences ride the mma.sync kernel, 5..8 the tcgen05 kernel)."""
    from insignia_b200.engine import Batch

    rng = np.random.default_rng(sequences)
    prompts = rng.integers(0, 64, (sequences, 9))
    with small_engine(golden_ckpt[1], prepared_inputs=False) as e:
        want, hidden, state = [], [], []
        for s in range(sequences):
            e.reset()
            for t in prompts[s]:
                e.forward_token(int(t))
            t = e.logits_argmax()
            toks = [t]
            for _ in range(12):
                t = e.decode_token(t)
                toks.append(t)
            want.append(toks)
            hidden.append(e.read("hidden"))
            state.append(e.read("delta_state", 3 * 32 * 128 * 128))
        with Batch(e, sequences) as b:
            for i in range(8):
                b.forward_tokens(prompts[:, i])
            first = b.decode_tokens(prompts[:, 8])
            assert first == [w[0] for w in want]
            got = b.generate(first, 12)
            assert b.position == 9 + 12
            for s in range(sequences):
                assert list(got[:, s]) == want[s][1:], s
                h = b.read("hidden", s)
                assert np.max(np.abs(h - hidden[s])) <= 2e-4 * np.abs(hidden[s]).max(), s
                st = b.read("delta_state", s, 3 * 32 * 128 * 128)
                assert np.max(np.abs(st - state[s])) <= 2e-4 * np.abs(state[s]).max(), s
            # a second run after reset gives the same tokens (graph replay, scratch and tickets left clean)
            b.reset()
            for i in range(8):
                b.forward_tokens(prompts[:, i])
            assert b.decode_tokens(prompts[:, 8]) == first
            with pytest.raises(Exception, match="token out of range"):
                b.forward_tokens([248320] * sequences)


def test_batch_errors(cuda, golden_ckpt):
    from insignia_b200.engine import Batch

    with small_engine(golden_ckpt[1], max_context=3) as e:
        with pytest.raises(Exception, match="1..8 sequences"):
            Batch(e, 9)
        with Batch(e, 2) as b:
            for _ in range(3):
                b.forward_tokens([1, 2])
            with pytest.raises(Exception, match="KV cache full"):
                b.forward_tokens([1, 2])
