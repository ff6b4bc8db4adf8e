"""Python mirror of the reference's decode classes over the C ABI's engine handle.

``Engine`` bundles what the reference's drivers build by hand (src/test_generate.cu:3):
``ModelFile`` -> ``Qwen35Weights`` -> ``DecodeWorkspace`` -> ``Qwen35Decode``, with the
same method names (``embed``, ``layer``, ``forward_token``, ``logits_argmax``,
``decode_token``, ``mtp_draft``) and the same errors, surfaced as ``InsigniaError``.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import EngineOptions, InsigniaError, check

FIELD_SIZES = {"hidden": 4096, "norm": 4096, "qkv": 8192, "core": 4096, "z": 4096, "a": 32, "b": 32, "gate": 12288,
               "key": 1024, "value": 1024, "down": 4096, "logits": 248320, "delta_state": 24 * 32 * 128 * 128,
               "conv_state": 24 * 8192 * 3}


class Engine:
    def __init__(self, index_path: str, max_context: int = 4096, budget_bytes: int = 16 << 30, kv_bf16: bool = False,
                 gate_elementwise: bool = False, accurate_trig: bool = False, use_graph: bool = True,
                 use_pdl: bool = True, n_layers: int = 32, vocab: int = 248320, device: int = 0,
                 gemv_tcgen05: bool = False, prepared_inputs: bool = True, persistent: bool = False, prefill_tcgen05: bool = True):
        """``persistent=False`` (default): one launch per fused operation, replayed from a CUDA graph when ``use_graph``;
        ``True``: a token step is one persistent cooperative launch (``insg_program_*``)."""
        o = EngineOptions(budget_bytes, max_context, int(kv_bf16), int(gate_elementwise), int(accurate_trig),
                          int(use_graph), int(use_pdl), int(gemv_tcgen05), n_layers, vocab, device, int(persistent), int(not prefill_tcgen05),
                          int(not prepared_inputs))
        self.vocab = vocab
        self._destroy = _lib.lib().insg_engine_destroy  # held here: module globals may be gone when __del__ runs at exit
        self._h = _lib.lib().insg_engine_create(index_path.encode(), C.byref(o))
        if not self._h:
            raise InsigniaError(_lib.lib().insg_last_error().decode())

    def close(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._destroy(h)

    def __del__(self):
        self.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def embed(self, token: int):
        check(_lib.lib().insg_engine_embed(self._h, token))

    def layer(self, layer: int):
        check(_lib.lib().insg_engine_layer(self._h, layer))

    def forward_token(self, token: int):
        check(_lib.lib().insg_engine_forward_token(self._h, token))

    def forward_tokens(self, tokens):
        """``forward_token`` over a list of consecutive tokens, four per pass over the weights (prompt processing)."""
        arr = (C.c_int * len(tokens))(*[int(t) for t in tokens])
        check(_lib.lib().insg_engine_forward_tokens(self._h, arr, len(tokens)))

    def logits_argmax(self) -> int:
        return check(_lib.lib().insg_engine_logits_argmax(self._h))

    def decode_token(self, token: int) -> int:
        return check(_lib.lib().insg_engine_decode_token(self._h, token))

    def mtp_draft(self, token: int) -> int:
        return check(_lib.lib().insg_engine_mtp_draft(self._h, token))

    def generate(self, first_token: int, count: int) -> list[int]:
        buf = (C.c_int * count)()
        check(_lib.lib().insg_engine_generate(self._h, first_token, count, buf))
        return list(buf)

    def prime_speculative(self, prompt) -> int:
        """The prompt token by token, every position's row left in the MTP cache; returns the greedy next token."""
        arr = (C.c_int * len(prompt))(*[int(t) for t in prompt])
        return check(_lib.lib().insg_engine_prime_speculative(self._h, arr, len(prompt)))

    def generate_speculative(self, first_token: int, count: int, forced_drafts=None):
        """``count`` greedy tokens by draft-1 / verify; returns (tokens, number of accepted drafts)."""
        buf, acc = (C.c_int * count)(), C.c_int()
        forced = None
        if forced_drafts is not None:  # entry i is the draft offered when i tokens have been produced
            if len(forced_drafts) < count:
                raise ValueError("forced_drafts needs one entry per generated token")
            forced = (C.c_int * len(forced_drafts))(*[int(t) for t in forced_drafts])
        check(_lib.lib().insg_engine_generate_speculative(self._h, first_token, count, buf, C.byref(acc), forced))
        return list(buf), acc.value

    def profile_gemv_chain(self, replays: int = 8) -> dict:
        """The token step's fused-GEMV operations alone, timed between two CUDA events; the sequence state is garbage afterwards (reset())."""
        ms, by, ln = C.c_float(), C.c_uint64(), C.c_int()
        check(_lib.lib().insg_engine_profile_gemv_chain(self._h, replays, C.byref(ms), C.byref(by), C.byref(ln)))
        return {"ms_per_token": ms.value, "bytes": by.value, "launches": ln.value}

    def set_program_option(self, key: str, value: int):
        """Option of the persistent token program, e.g. ``prefetch_records`` (weight records per warp kept requested into
        L2 ahead of consumption; 0 = off)."""
        check(_lib.lib().insg_engine_set_program_option(self._h, key.encode(), value))

    def selftest_barrier_timeout(self) -> bool:
        """Runs the persistent kernel once with a grid barrier that cannot be met and a 2 ms wait limit; True when the
        kernel gave up and raised its error status.  Call reset() afterwards."""
        return check(_lib.lib().insg_engine_selftest_barrier_timeout(self._h)) == 1

    @property
    def position(self) -> int:
        return _lib.lib().insg_engine_position(self._h)

    @position.setter
    def position(self, p: int):
        check(_lib.lib().insg_engine_set_position(self._h, p))

    def reset(self):
        check(_lib.lib().insg_engine_reset(self._h))

    def read(self, field: str, count: int | None = None) -> np.ndarray:
        n = count if count is not None else (self.vocab if field == "logits" else FIELD_SIZES[field])
        out = np.empty(n, np.float32)
        check(_lib.lib().insg_engine_read(self._h, field.encode(), out.ctypes.data, n))
        return out

    def write(self, field: str, values: np.ndarray):
        v = np.ascontiguousarray(values, np.float32)
        check(_lib.lib().insg_engine_write(self._h, field.encode(), v.ctypes.data, v.size))

    def buffer(self, field: str) -> int:
        return _lib.lib().insg_engine_buffer(self._h, field.encode())

    @property
    def stream(self) -> int:
        return _lib.lib().insg_engine_stream(self._h) or 0

    @property
    def launch_count(self) -> int:
        return _lib.lib().insg_engine_launch_count(self._h)

    @property
    def device_bytes(self) -> int:
        return _lib.lib().insg_engine_device_bytes(self._h)


class Batch:
    """1..8 independent sequences decoded in lock step on the weights of an :class:`Engine` (one weight copy, every
    matrix streamed once per step for all sequences): ``insg_batch_*``.  Close it before its engine."""

    def __init__(self, engine: Engine, sequences: int, max_context: int = 0):
        self.n = sequences
        self._engine = engine
        self._destroy = _lib.lib().insg_batch_destroy
        self._h = _lib.lib().insg_batch_create(engine._h, sequences, max_context)
        if not self._h:
            raise InsigniaError(_lib.lib().insg_last_error().decode())

    def close(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._destroy(h)

    def __del__(self):
        self.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def _arr(self, tokens):
        assert len(tokens) == self.n
        return (C.c_int * self.n)(*[int(t) for t in tokens])

    def forward_tokens(self, tokens):
        check(_lib.lib().insg_batch_forward_tokens(self._h, self._arr(tokens)))

    def decode_tokens(self, tokens) -> list[int]:
        out = (C.c_int * self.n)()
        check(_lib.lib().insg_batch_decode_tokens(self._h, self._arr(tokens), out))
        return list(out)

    def generate(self, first_tokens, count: int) -> np.ndarray:
        out = (C.c_int * (self.n * count))()
        check(_lib.lib().insg_batch_generate(self._h, self._arr(first_tokens), count, out))
        return np.array(out, dtype=np.int64).reshape(count, self.n)

    def reset(self):
        check(_lib.lib().insg_batch_reset(self._h))

    @property
    def position(self) -> int:
        return _lib.lib().insg_batch_position(self._h)

    def read(self, field: str, sequence: int, count: int = 4096) -> np.ndarray:
        out = np.empty(count, np.float32)
        check(_lib.lib().insg_batch_read(self._h, field.encode(), sequence, out.ctypes.data, count))
        return out

    @property
    def stream(self) -> int:
        return _lib.lib().insg_batch_stream(self._h) or 0

    @property
    def launch_count(self) -> int:
        return _lib.lib().insg_batch_launch_count(self._h)
