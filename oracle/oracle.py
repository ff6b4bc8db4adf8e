"""Python face of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Loads ``oracle/_build/liboracle.so`` (built from ``insg_oracle.c`` by ``oracle/Makefile``)
and offers numpy wrappers for every restated kernel plus :class:`OracleModel`, a
multi-token restatement of the reference's decode loop (src/decode.cu:13-69).
Only ``tests/``, the smoke check and the benchmark's CPU-baseline leg import this
module; the shipped library never does.

The reference has two behaviours for the attention output gate: its CUDA engine
broadcasts element 0 of each head's gate (src/qwen_kernels.cu:36) while its
NumPy tools gate element by element (tools/reference_all_layers.py:13).
``OracleModel(gate="broadcast"|"elementwise")`` selects which one is restated.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")
_lib = None

f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")
u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")


def build(force: bool = False) -> str:
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(
            os.path.join(_HERE, "insg_oracle.c")):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B", "_build/liboracle.so"])
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        L = _lib
        L.orc_fp4_e2m1.restype = C.c_float
        L.orc_fp4_e2m1.argtypes = [C.c_uint8]
        L.orc_e8m0.restype = C.c_float
        L.orc_e8m0.argtypes = [C.c_uint8]
        L.orc_e8m0_mlx.restype = C.c_float
        L.orc_e8m0_mlx.argtypes = [C.c_uint8]
        L.orc_mxfp4_dequant_mlx.argtypes = [u32p, u8p, f32p, C.c_int, C.c_int]
        L.orc_mxfp4_get_row_mlx.argtypes = [u32p, u8p, f32p, C.c_int, C.c_int]
        L.orc_mxfp4_gemv_mlx.argtypes = [u32p, u8p, f32p, f32p, C.c_int, C.c_int, C.c_int]
        L.orc_mxfp4_gemv_mlx_fast.argtypes = [u32p, u8p, f32p, f32p, C.c_int, C.c_int]
        L.orc_mxfp4_gemv_mlx_f64.argtypes = [u32p, u8p, f32p, f64p, C.c_int, C.c_int]
        L.orc_mxfp4_gemv_block17.argtypes = [u8p, f32p, f32p, C.c_int, C.c_int]
        L.orc_rmsnorm_bf16.argtypes = [f32p, u16p, C.c_void_p, f32p, C.c_int, C.c_int, C.c_int]
        L.orc_rmsnorm_zero_centered.argtypes = [f32p, f32p, f32p, C.c_int, C.c_int, C.c_float]
        L.orc_causal_conv4_silu.argtypes = [f32p, f32p, u16p, C.c_int]
        L.orc_deltanet_parameters.argtypes = [f32p, f32p, f32p, u16p, C.c_int]
        L.orc_deltanet_decode.argtypes = [f32p] * 7
        L.orc_qk_norm_rope.argtypes = [f32p, f32p, u16p, u16p, C.c_int]
        L.orc_split_q_gate.argtypes = [f32p, f32p, f32p]
        L.orc_store_kv.argtypes = [f32p, f32p, f32p, f32p, C.c_int]
        L.orc_gqa_decode.argtypes = [f32p, f32p, f32p, f32p, C.c_int]
        L.orc_expand_gate_heads.argtypes = [f32p, f32p]
        L.orc_sigmoid_mul.argtypes = [f32p, f32p, C.c_int]
        L.orc_silu_mul.argtypes = [f32p, f32p, f32p, C.c_int]
        L.orc_residual_add.argtypes = [f32p, f32p, C.c_int]
        L.orc_bf16_gemv.argtypes = [u16p, f32p, f32p, C.c_int, C.c_int]
        L.orc_concat.argtypes = [f32p, f32p, f32p, C.c_int]
        L.orc_argmax.restype = C.c_int
        L.orc_argmax.argtypes = [f32p, C.c_int]
        L.orc_num_threads.restype = C.c_int
    return _lib


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


# ---------------------------------------------------------------- kernel wrappers
def fp4_e2m1(code: int) -> float:
    return lib().orc_fp4_e2m1(code)


def e8m0(byte: int) -> float:
    return lib().orc_e8m0(byte)


def e8m0_mlx(byte: int) -> float:
    return lib().orc_e8m0_mlx(byte)


def dequant_mlx(w, s):
    w, s = _c(w, np.uint32), _c(s, np.uint8)
    rows, cols = w.shape[0], w.shape[1] * 8
    out = np.empty((rows, cols), np.float32)
    lib().orc_mxfp4_dequant_mlx(w, s, out, rows, cols)
    return out


def get_row_mlx(w, s, row):
    w, s = _c(w, np.uint32), _c(s, np.uint8)
    cols = w.shape[1] * 8
    out = np.empty(cols, np.float32)
    lib().orc_mxfp4_get_row_mlx(w, s, out, row, cols)
    return out


def gemv_mlx(w, s, x, warps=2, fast=False):
    """y = W x.  ``warps=2`` is what the decode loop passes (src/decode.cu:13)."""
    w, s, x = _c(w, np.uint32), _c(s, np.uint8), _c(x, np.float32)
    rows, cols = w.shape[0], w.shape[1] * 8
    y = np.zeros(rows, np.float32)
    if fast:
        lib().orc_mxfp4_gemv_mlx_fast(w, s, x, y, rows, cols)
    else:
        lib().orc_mxfp4_gemv_mlx(w, s, x, y, rows, cols, warps)
    return y


def gemv_mlx_f64(w, s, x):
    w, s, x = _c(w, np.uint32), _c(s, np.uint8), _c(x, np.float32)
    rows, cols = w.shape[0], w.shape[1] * 8
    y = np.zeros(rows, np.float64)
    lib().orc_mxfp4_gemv_mlx_f64(w, s, x, y, rows, cols)
    return y


def gemv_block17(blocks, x, rows, cols):
    y = np.zeros(rows, np.float32)
    lib().orc_mxfp4_gemv_block17(_c(blocks, np.uint8), _c(x, np.float32), y, rows, cols)
    return y


def rmsnorm_bf16(x, w, zero_centered=False, gate=None):
    x = _c(x, np.float32)
    x2 = x.reshape(-1, x.shape[-1])
    y = np.empty_like(x2)
    g = None if gate is None else _c(gate, np.float32)
    lib().orc_rmsnorm_bf16(x2, _c(w, np.uint16), None if g is None else g.ctypes.data, y, x2.shape[0], x2.shape[1],
                           int(zero_centered))
    return y.reshape(x.shape)


def rmsnorm_zero_centered(x, w, eps=1e-6):
    x = _c(x, np.float32)
    y = np.empty_like(x)
    lib().orc_rmsnorm_zero_centered(x, _c(w, np.float32), y, x.shape[0], x.shape[1], eps)
    return y


def causal_conv4_silu(x, state, w):
    """In place on ``x`` [n] and ``state`` [n,3]; ``w`` bf16 bits [n,4]."""
    lib().orc_causal_conv4_silu(x, state, _c(w, np.uint16).reshape(-1), x.size)


def deltanet_parameters(a, b, A_log, dt_bias):
    lib().orc_deltanet_parameters(a, b, _c(A_log, np.float32), _c(dt_bias, np.uint16), a.size)


def deltanet_decode(state, q, k, v, g, beta):
    out = np.empty(32 * 128, np.float32)
    lib().orc_deltanet_decode(state, _c(q, np.float32), _c(k, np.float32), _c(v, np.float32), _c(g, np.float32),
                              _c(beta, np.float32), out)
    return out


def qk_norm_rope(q, k, qw, kw, pos):
    lib().orc_qk_norm_rope(q, k, _c(qw, np.uint16), _c(kw, np.uint16), pos)


def gqa_decode(q, kc, vc, tokens):
    out = np.empty(16 * 256, np.float32)
    lib().orc_gqa_decode(_c(q, np.float32), kc, vc, out, tokens)
    return out


def argmax(x):
    x = _c(x, np.float32)
    return lib().orc_argmax(x, x.size)


def bf16_gemv(w, x):
    w = _c(w, np.uint16)
    y = np.empty(w.shape[0], np.float32)
    lib().orc_bf16_gemv(w, _c(x, np.float32), y, w.shape[0], w.shape[1])
    return y


def num_threads():
    return lib().orc_num_threads()


# ------------------------------------------------------------------- model level
class OracleModel:
    """CPU restatement of Qwen35Decode + DecodeWorkspace (src/decode.cu:10-69).

    ``tensors`` is any object with ``get(name) -> ndarray`` (bf16 tensors as uint16
    bits), e.g. ``insignia_b200.checkpoint_io.SafetensorsReader``.
    """

    LM = "language_model"

    def __init__(self, tensors, max_context=4096, gate="broadcast", fast_gemv=False, n_layers=32):
        self.t = tensors
        self.ctx = max_context
        self.gate_mode = gate
        self.fast = fast_gemv
        self.n_layers = n_layers
        self.position = 0
        self.hidden = np.zeros(4096, np.float32)
        self.logits = None
        # src/decode.cu:10 : zeroed recurrent state, [24][32][128][128] and [24][8192][3]
        self.delta_state = np.zeros((24, 32 * 128 * 128), np.float32)
        self.conv_state = np.zeros((24, 8192 * 3), np.float32)
        self.kv_keys = np.zeros((8, max_context * 1024), np.float32)
        self.kv_values = np.zeros((8, max_context * 1024), np.float32)
        self.mtp_keys = np.zeros(max_context * 1024, np.float32)
        self.mtp_values = np.zeros(max_context * 1024, np.float32)

    # src/decode.cu:13
    def linear(self, base, x):
        return gemv_mlx(self.t.get(base + ".weight"), self.t.get(base + ".scales"), x, warps=2, fast=self.fast)

    def norm(self, x, name):
        return rmsnorm_bf16(x, self.t.get(name), zero_centered=False)

    # src/qwen35.cu:9
    def embed(self, token):
        if token < 0 or token >= 248320:
            raise RuntimeError("token out of range")
        b = self.LM + ".model.embed_tokens"
        return get_row_mlx(self.t.get(b + ".weight"), self.t.get(b + ".scales"), token)

    # src/decode.cu:17
    def mlp(self, p):
        n = self.norm(self.hidden, p + ".post_attention_layernorm.weight")
        gate, up = self.linear(p + ".mlp.gate_proj", n), self.linear(p + ".mlp.up_proj", n)
        act = np.empty_like(gate)
        lib().orc_silu_mul(gate, up, act, act.size)
        self.hidden = self.hidden + self.linear(p + ".mlp.down_proj", act)

    # src/decode.cu:14-17
    def delta_layer(self, l):
        if l < 0 or l >= 32 or (l & 3) == 3:
            raise RuntimeError("not a DeltaNet layer")
        p = f"{self.LM}.model.layers.{l}"
        a = p + ".linear_attn"
        n = self.norm(self.hidden, p + ".input_layernorm.weight")
        qkv, z = self.linear(a + ".in_proj_qkv", n), self.linear(a + ".in_proj_z", n)
        aa, bb = self.linear(a + ".in_proj_a", n), self.linear(a + ".in_proj_b", n)
        di = l - l // 4
        causal_conv4_silu(qkv, self.conv_state[di], self.t.get(a + ".conv1d.weight"))
        deltanet_parameters(aa, bb, self.t.get(a + ".A_log"), self.t.get(a + ".dt_bias"))
        core = deltanet_decode(self.delta_state[di], qkv[:2048], qkv[2048:4096], qkv[4096:], aa, bb)
        core = rmsnorm_bf16(core.reshape(32, 128), self.t.get(a + ".norm.weight"), gate=z.reshape(32, 128)).reshape(-1)
        self.seam = {"qkv": qkv, "z": z, "g": aa, "beta": bb, "core": core}
        self.hidden = self.hidden + self.linear(a + ".out_proj", core)
        self.mlp(p)

    def _attention_block(self, p, keys, values, rope_pos, tokens):
        a = p + ".self_attn"
        n = self.norm(self.hidden, p + ".input_layernorm.weight")
        raw = self.linear(a + ".q_proj", n)
        q, gate = np.empty(4096, np.float32), np.empty(4096, np.float32)
        lib().orc_split_q_gate(raw, q, gate)
        k, v = self.linear(a + ".k_proj", n), self.linear(a + ".v_proj", n)
        qk_norm_rope(q, k, self.t.get(a + ".q_norm.weight"), self.t.get(a + ".k_norm.weight"), rope_pos)
        lib().orc_store_kv(k, v, keys, values, rope_pos)
        core = gqa_decode(q, keys, values, tokens)
        if self.gate_mode == "broadcast":
            g = np.empty(4096, np.float32)
            lib().orc_expand_gate_heads(gate, g)
        else:
            g = gate
        lib().orc_sigmoid_mul(core, g, 4096)
        self.seam = {"q": q, "k": k, "v": v, "gate": gate, "core": core}
        self.hidden = self.hidden + self.linear(a + ".o_proj", core)
        self.mlp(p)

    # src/decode.cu:19
    def attention_layer(self, l):
        if l < 0 or l >= 32 or (l & 3) != 3:
            raise RuntimeError("not a full attention layer")
        if self.position >= self.ctx:
            raise RuntimeError("KV cache full")
        ai = l // 4
        self._attention_block(f"{self.LM}.model.layers.{l}", self.kv_keys[ai], self.kv_values[ai], self.position,
                              self.position + 1)

    def layer(self, l):
        self.attention_layer(l) if (l & 3) == 3 else self.delta_layer(l)

    # src/decode.cu:21
    def forward_token(self, token, want_logits=True):
        self.hidden = self.embed(token)
        for l in range(self.n_layers):
            self.layer(l)
        if want_logits:
            n = self.norm(self.hidden, self.LM + ".model.norm.weight")
            self.logits = self.linear(self.LM + ".lm_head", n)
        self.position += 1

    # src/decode.cu:22-23
    def logits_argmax(self):
        return argmax(self.logits)

    def decode_token(self, token):
        self.forward_token(token)
        return self.logits_argmax()

    # src/decode.cu:24-69 (note: overwrites self.hidden exactly as the reference overwrites x.hidden)
    def mtp_draft(self, token):
        m = self.LM + ".mtp"
        e = self.norm(self.embed(token), m + ".pre_fc_norm_embedding.weight")
        h = self.norm(self.hidden, m + ".pre_fc_norm_hidden.weight")
        self.hidden = bf16_gemv(self.t.get(m + ".fc.weight"), np.concatenate([e, h]))
        self._attention_block(m + ".layers.0", self.mtp_keys, self.mtp_values, self.position - 1, self.position)
        n = self.norm(self.hidden, m + ".norm.weight")
        self.logits = self.linear(self.LM + ".lm_head", n)
        return self.logits_argmax()
