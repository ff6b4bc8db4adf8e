"""Thin Python callers of the C ABI on torch CUDA tensors (torch only supplies device memory and streams).

Every function forwards to one ``insg_*`` entry point of include/insignia_b200.h on the
current torch stream.  Inputs must be contiguous CUDA tensors of the stated dtype;
nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import AttnOp, GemvOp, check

PRO = {"plain": 0, "rmsnorm": 1, "gated_rmsnorm": 2, "sigmoid_gate": 3, "sigmoid_gate_head0": 4, "sigmoid_gate_qproj": 5, "prepared": 6}
EPI = {"store": 0, "residual": 1, "conv_silu": 2, "beta": 3, "decay": 4, "swiglu": 5, "logits": 6}
KV_F32, KV_BF16 = 0, 1


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    if t is None:
        return None
    if not t.is_cuda or not t.is_contiguous():
        raise ValueError("expected a contiguous CUDA tensor")
    return t.data_ptr()


def tune(key: str, value: int) -> None:
    check(_lib.lib().insg_tune_set(key.encode(), value))


def gemv_mlx(weight, scales, x):
    rows, cols = weight.shape[0], weight.shape[1] * 8
    y = torch.empty(rows, dtype=torch.float32, device=x.device)
    check(_lib.lib().insg_mxfp4_gemv_mlx(_p(weight), _p(scales), _p(x), _p(y), rows, cols, _stream()))
    return y


def get_row_mlx(weight, scales, row):
    cols = weight.shape[1] * 8
    out = torch.empty(cols, dtype=torch.float32, device=weight.device)
    check(_lib.lib().insg_mxfp4_get_row_mlx(_p(weight), _p(scales), _p(out), row, cols, _stream()))
    return out


def dequant_mlx(weight, scales):
    rows, cols = weight.shape[0], weight.shape[1] * 8
    out = torch.empty((rows, cols), dtype=torch.float32, device=weight.device)
    check(_lib.lib().insg_mxfp4_dequant_mlx(_p(weight), _p(scales), _p(out), rows, cols, _stream()))
    return out


def repack(weight, scales):
    rows, cols = weight.shape[0], weight.shape[1] * 8
    n = _lib.lib().insg_mxfp4_packed_bytes(rows, cols)
    if n == 0:
        raise ValueError("rows % 16 and cols % 128 must be 0")
    packed = torch.empty(n, dtype=torch.uint8, device=weight.device)
    check(_lib.lib().insg_mxfp4_repack(_p(weight), _p(scales), _p(packed), rows, cols, _stream()))
    packed.rows, packed.cols = rows, cols
    return packed


def repack_umma(weight, scales):
    """Weights in the layout of the tcgen05 kernel (pass ``layout=1`` to :func:`gemv_fused`)."""
    rows, cols = weight.shape[0], weight.shape[1] * 8
    n = _lib.lib().insg_mxfp4_packed_umma_bytes(rows, cols)
    if n == 0:
        raise ValueError("cols % 128 must be 0")
    packed = torch.empty(n, dtype=torch.uint8, device=weight.device)
    check(_lib.lib().insg_mxfp4_repack_umma(_p(weight), _p(scales), _p(packed), rows, cols, _stream()))
    packed.rows, packed.cols = rows, cols
    return packed


def gemv_packed(packed, x, rows=None, cols=None):
    rows = rows or packed.rows
    cols = cols or packed.cols
    x2 = x.reshape(-1, cols)
    y = torch.empty((x2.shape[0], rows), dtype=torch.float32, device=x.device)
    check(_lib.lib().insg_mxfp4_gemv_packed(_p(packed), _p(x2), _p(y), rows, cols, x2.shape[0], _stream()))
    return y.reshape(*x.shape[:-1], rows)


def _gemv_op(inp, segments, prologue="plain", aux=None, norm_w=None, x_out=None, argmax=None, pdl=False, layout=0, error_flag=None,
             prep_partials=None, prep_rms=False, cols=None, tokens=1, umma_scratch=None):
    op = GemvOp()
    if umma_scratch is not None:
        op.umma_scratch, op.umma_scratch_bytes = _p(umma_scratch), umma_scratch.numel()
    op.in_, op.aux, op.norm_w, op.x_out = _p(inp), _p(aux), _p(norm_w), _p(x_out)
    op.cols, op.prologue, op.n_segments = cols or inp.shape[-1], PRO[prologue], len(segments)
    op.prep_partials, op.prep_rms, op.tokens = _p(prep_partials), int(prep_rms), tokens
    for i, s in enumerate(segments):
        g = op.seg[i]
        g.packed, g.packed2, g.out = _p(s["packed"]), _p(s.get("packed2")), _p(s["out"])
        g.rows, g.epilogue = s["rows"], EPI[s["epilogue"]]
        g.conv_state, g.conv_w = _p(s.get("conv_state")), _p(s.get("conv_w"))
        g.A_log, g.dt_bias = _p(s.get("A_log")), _p(s.get("dt_bias"))
        g.prep, g.prep_w, g.prep_partials = _p(s.get("prep")), _p(s.get("prep_w")), _p(s.get("prep_partials"))
        g.conv_token_stride = s.get("conv_token_stride", 0)
    if argmax:
        op.argmax_scratch, op.token_out = _p(argmax["scratch"]), _p(argmax["token_out"])
        op.token_feedback, op.token_log = _p(argmax.get("token_feedback")), _p(argmax.get("token_log"))
        op.token_log_capacity = argmax["token_log"].numel() if argmax.get("token_log") is not None else 0
        op.position_inout = _p(argmax.get("position"))
    op.layout = layout
    op.error_flag = _p(error_flag)
    op.pdl = int(pdl)
    return op


def umma_gemm_scratch(cols, tokens, device="cuda"):
    return torch.empty(_lib.lib().insg_umma_gemm_scratch_bytes(cols, tokens), dtype=torch.uint8, device=device)


def gemm_umma(packed_umma, x, rows=None, cols=None, scratch=None):
    """``y[m] = W x[m]`` for all rows of ``x`` on the tcgen05 tensor cores (weights from :func:`repack_umma`)."""
    rows = rows or packed_umma.rows
    cols = cols or packed_umma.cols
    x2 = x.reshape(-1, cols)
    M = x2.shape[0]
    scratch = scratch if scratch is not None else umma_gemm_scratch(cols, M, x.device)
    y = torch.empty((M, rows), dtype=torch.float32, device=x.device)
    check(_lib.lib().insg_mxfp4_gemm_umma(_p(packed_umma), _p(x2), _p(y), rows, cols, M, _p(scratch), scratch.numel(), _stream()))
    return y.reshape(*x.shape[:-1], rows)


def gemv_fused(inp, segments, **kw):
    """``segments``: list of dicts with packed, out, rows, epilogue (+ packed2 / conv_state, conv_w / A_log, dt_bias /
    prep, prep_w, prep_partials).  Keywords: prologue, aux, norm_w, x_out, pdl, layout, error_flag, prep_partials,
    prep_rms, cols, tokens, and ``argmax``: dict(scratch, token_out[, token_feedback, token_log, position]) for the
    logits epilogue.  With ``prologue="prepared"`` ``inp`` is the fp16 image [2][cols] a producer left through ``prep``."""
    op = _gemv_op(inp, segments, **kw)
    check(_lib.lib().insg_gemv_fused(C.byref(op), _stream()))


class Program:
    """A recorded sequence of fused operations run by ONE persistent cooperative launch (``insg_program_*``): the
    ``add_*`` methods take what :func:`gemv_fused`, :func:`deltanet_decode`, :func:`attention_step` and the embedding
    lookup take.  Tensors handed to ``add_*`` must stay alive while the program exists."""

    def __init__(self):
        self._destroy = _lib.lib().insg_program_destroy
        self._h = _lib.lib().insg_program_create()
        if not self._h:
            raise RuntimeError("insg_program_create failed")
        self._keep = []

    def close(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._destroy(h)

    def __del__(self):
        self.close()

    def add_gemv(self, inp, segments, **kw):
        op = _gemv_op(inp, segments, **kw)
        self._keep.append((inp, segments, kw))
        check(_lib.lib().insg_program_add_gemv(self._h, C.byref(op)))

    def add_deltanet(self, state, q16, k16, v32, g32, beta32, out):
        self._keep.append((state, q16, k16, v32, g32, beta32, out))
        check(_lib.lib().insg_program_add_deltanet(self._h, _p(state), _p(q16), _p(k16), _p(v32), _p(g32), _p(beta32), _p(out)))

    def add_attention(self, qraw, k_raw, v, q_w, k_w, k_cache, v_cache, out, position, max_context, scratch, position_offset=0,
                      fast_trig=True):
        op = AttnOp()
        op.qraw, op.k_raw, op.v, op.q_norm_w, op.k_norm_w = _p(qraw), _p(k_raw), _p(v), _p(q_w), _p(k_w)
        op.k_cache, op.v_cache = _p(k_cache), _p(v_cache)
        op.out, op.position, op.position_offset, op.max_context = _p(out), _p(position), position_offset, max_context
        op.kv_dtype = KV_BF16 if k_cache.dtype == torch.bfloat16 else KV_F32
        op.fast_trig, op.scratch, op.scratch_bytes = int(fast_trig), _p(scratch), scratch.numel()
        self._keep.append((qraw, k_raw, v, q_w, k_w, k_cache, v_cache, out, position, scratch))
        check(_lib.lib().insg_program_add_attention(self._h, C.byref(op)))

    def add_embed(self, weight, scales, out, device_row):
        self._keep.append((weight, scales, out, device_row))
        check(_lib.lib().insg_program_add_embed(self._h, _p(weight), _p(scales), _p(out), _p(device_row), weight.shape[0],
                                                weight.shape[1] * 8))

    def finalize(self):
        check(_lib.lib().insg_program_finalize(self._h))

    def set_option(self, key: str, value: int):
        check(_lib.lib().insg_program_set_option(self._h, key.encode(), value))

    def run(self, n_tokens=1, token=-1, position=-1, device_token=None, device_position=None, error_flag=None):
        check(_lib.lib().insg_program_run(self._h, n_tokens, token, position, _p(device_token), _p(device_position), _p(error_flag),
                                          _stream()))

    def recover(self):
        check(_lib.lib().insg_program_recover(self._h, _stream()))

    def selftest_barrier_timeout(self, timeout_ns, error_flag):
        check(_lib.lib().insg_program_selftest_barrier_timeout(self._h, timeout_ns, _p(error_flag), _stream()))

    @property
    def phase_count(self) -> int:
        return _lib.lib().insg_program_phase_count(self._h)

    @property
    def weight_bytes(self) -> int:
        return _lib.lib().insg_program_weight_bytes(self._h)


class Comm:
    """One rank's end of the one-shot all-reduce (``insg_comm_*``).  ``Comm.local(world, n)`` builds all ranks on the
    current GPU (they then run as one cooperative launch); across processes: create, all-gather ``handle()``, ``connect``."""

    def __init__(self, rank: int, world: int, max_floats: int):
        self._h = _lib.lib().insg_comm_create(rank, world, max_floats)
        if not self._h:
            raise RuntimeError(_lib.lib().insg_last_error().decode())
        self.rank, self.world, self.max_floats = rank, world, max_floats

    def close(self):
        if getattr(self, "_h", None):
            _lib.lib().insg_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def handle(self) -> bytes:
        buf = C.create_string_buffer(64)
        check(_lib.lib().insg_comm_handle(self._h, buf))
        return buf.raw

    def connect(self, handles):
        blob = b"".join(handles)
        assert len(blob) == 64 * self.world
        check(_lib.lib().insg_comm_connect(self._h, blob))

    def set_timeout(self, ns: int):
        check(_lib.lib().insg_comm_set_timeout(self._h, ns))

    def error(self) -> int:
        out = C.c_int()
        check(_lib.lib().insg_comm_error(self._h, C.byref(out), _stream()))
        return out.value

    def reset(self):
        check(_lib.lib().insg_comm_reset(self._h, _stream()))

    def allreduce(self, data, count=None):
        check(_lib.lib().insg_allreduce_oneshot(self._h, _p(data), count or data.numel(), _stream()))
        return data

    @staticmethod
    def local(world: int, max_floats: int):
        comms = [Comm(r, world, max_floats) for r in range(world)]
        arr = (C.c_void_p * world)(*[c._h for c in comms])
        check(_lib.lib().insg_comm_connect_local(arr, world))
        return comms

    @staticmethod
    def allreduce_local(comms, tensors, count=None, skip_rank=-1):
        world = len(comms)
        hs = (C.c_void_p * world)(*[c._h for c in comms])
        ds = (C.c_void_p * world)(*[_p(t) for t in tensors])
        check(_lib.lib().insg_allreduce_oneshot_local(hs, ds, world, count or tensors[0].numel(), skip_rank, _stream()))


def argmax_scratch(device):
    return torch.zeros(_lib.lib().insg_gemv_argmax_scratch_bytes(), dtype=torch.uint8, device=device)


def deltanet_decode(state, q16, k16, v32, g32, beta32, pdl=False):
    out = torch.empty(32 * 128, dtype=torch.float32, device=state.device)
    check(_lib.lib().insg_deltanet_decode(_p(state), _p(q16), _p(k16), _p(v32), _p(g32), _p(beta32), _p(out), int(pdl),
                                          _stream()))
    return out


def deltanet_decode_tokens(state, q16, k16, v32, g32, beta32, tokens, qkv_stride, pdl=False):
    """``tokens`` consecutive DeltaNet steps in one launch; inputs of step m at + m * qkv_stride (q, k, v) and + m * 32 (g, beta)."""
    out = torch.empty(tokens * 32 * 128, dtype=torch.float32, device=state.device)
    check(_lib.lib().insg_deltanet_decode_tokens(_p(state), _p(q16), _p(k16), _p(v32), _p(g32), _p(beta32), _p(out), tokens,
                                                 qkv_stride, int(pdl), _stream()))
    return out.reshape(tokens, 32 * 128)


def deltanet_decode_batch(state, q16, k16, v32, g32, beta32, sequences, qkv_stride, pdl=False):
    """One DeltaNet step for ``sequences`` independent sequences; state [sequences][32][128][128], inputs strided like
    :func:`deltanet_decode_tokens`."""
    out = torch.empty(sequences * 32 * 128, dtype=torch.float32, device=state.device)
    check(_lib.lib().insg_deltanet_decode_batch(_p(state), 32 * 128 * 128, _p(q16), _p(k16), _p(v32), _p(g32), _p(beta32), _p(out), sequences,
                                                qkv_stride, int(pdl), _stream()))
    return out.reshape(sequences, 32 * 128)


def gqa_scratch(device, tokens=0):
    return torch.zeros(_lib.lib().insg_gqa_scratch_bytes(tokens), dtype=torch.uint8, device=device)


def gqa_decode(q, k_cache, v_cache, tokens, scratch=None):
    kv = KV_BF16 if k_cache.dtype == torch.bfloat16 else KV_F32
    scratch = scratch if scratch is not None else gqa_scratch(q.device, tokens)
    out = torch.empty(16 * 256, dtype=torch.float32, device=q.device)
    check(_lib.lib().insg_gqa_decode(_p(q), _p(k_cache), _p(v_cache), _p(out), tokens, kv, _p(scratch), scratch.numel(),
                                     _stream()))
    return out


def gqa_decode_noalloc(q, k_cache, v_cache, tokens):
    """Same result as :func:`gqa_decode` without a scratch buffer: the partials live in a fixed array inside the
    library (one per GPU), so nothing is allocated; calls that overlap on the GPU must be serialised by the caller."""
    kv = KV_BF16 if k_cache.dtype == torch.bfloat16 else KV_F32
    out = torch.empty(16 * 256, dtype=torch.float32, device=q.device)
    check(_lib.lib().insg_gqa_decode_noalloc(_p(q), _p(k_cache), _p(v_cache), _p(out), tokens, kv, _stream()))
    return out


def attention_step(qraw, k_raw, v, q_w, k_w, k_cache, v_cache, position, max_context, scratch, position_offset=0,
                   fast_trig=True, pdl=False):
    op = AttnOp()
    op.qraw, op.k_raw, op.v, op.q_norm_w, op.k_norm_w = _p(qraw), _p(k_raw), _p(v), _p(q_w), _p(k_w)
    op.k_cache, op.v_cache = _p(k_cache), _p(v_cache)
    out = torch.empty(16 * 256, dtype=torch.float32, device=qraw.device)
    op.out, op.position, op.position_offset, op.max_context = _p(out), _p(position), position_offset, max_context
    op.kv_dtype = KV_BF16 if k_cache.dtype == torch.bfloat16 else KV_F32
    op.fast_trig, op.scratch, op.scratch_bytes, op.pdl = int(fast_trig), _p(scratch), scratch.numel(), int(pdl)
    check(_lib.lib().insg_attention_step(C.byref(op), _stream()))
    return out


def attention_batch(qraw, k_raw, v, q_w, k_w, k_cache, v_cache, position, max_context, scratch, sequences, fast_trig=True, pdl=False):
    """One step for ``sequences`` independent sequences at the same position in one launch; qraw [sequences][8192], k_raw
    and v [sequences][1024], k_cache / v_cache [sequences][max_context * 1024]; scratch: ``sequences`` zero-headed regions."""
    op = AttnOp()
    op.qraw, op.k_raw, op.v, op.q_norm_w, op.k_norm_w = _p(qraw), _p(k_raw), _p(v), _p(q_w), _p(k_w)
    op.k_cache, op.v_cache = _p(k_cache), _p(v_cache)
    out = torch.empty(sequences * 16 * 256, dtype=torch.float32, device=qraw.device)
    op.out, op.position, op.position_offset, op.max_context = _p(out), _p(position), 0, max_context
    op.kv_dtype = KV_BF16 if k_cache.dtype == torch.bfloat16 else KV_F32
    op.fast_trig, op.scratch, op.scratch_bytes, op.pdl = int(fast_trig), _p(scratch), scratch.numel(), int(pdl)
    stride = k_cache.numel() // sequences * k_cache.element_size()
    check(_lib.lib().insg_attention_batch(C.byref(op), sequences, stride, _stream()))
    return out.reshape(sequences, 4096)


def attention_chunk(qraw, k_raw, v, q_w, k_w, k_cache, v_cache, position, max_context, scratch, tokens, fast_trig=True, rows_hint=0):
    """``tokens`` consecutive tokens of one sequence (rows position .. position + tokens - 1) in two launches; qraw
    [tokens][8192], k_raw and v [tokens][1024]; scratch holds ``tokens`` zero-headed regions of :func:`gqa_scratch` size."""
    op = AttnOp()
    op.qraw, op.k_raw, op.v, op.q_norm_w, op.k_norm_w = _p(qraw), _p(k_raw), _p(v), _p(q_w), _p(k_w)
    op.k_cache, op.v_cache = _p(k_cache), _p(v_cache)
    out = torch.empty(tokens * 16 * 256, dtype=torch.float32, device=qraw.device)
    op.out, op.position, op.position_offset, op.max_context = _p(out), _p(position), 0, max_context
    op.kv_dtype = KV_BF16 if k_cache.dtype == torch.bfloat16 else KV_F32
    op.fast_trig, op.scratch, op.scratch_bytes, op.pdl = int(fast_trig), _p(scratch), scratch.numel(), 0
    qn = torch.empty(tokens * 4096, dtype=torch.float32, device=qraw.device)
    check(_lib.lib().insg_attention_chunk(C.byref(op), tokens, _p(qn), rows_hint, _stream()))
    return out.reshape(tokens, 4096)


def rmsnorm_bf16(x, w, zero_centered=False, gate=None):
    x2 = x.reshape(-1, x.shape[-1])
    y = torch.empty_like(x2)
    check(_lib.lib().insg_rmsnorm_bf16(_p(x2), _p(w), _p(gate), _p(y), x2.shape[0], x2.shape[1], int(zero_centered),
                                       _stream()))
    return y.reshape(x.shape)


def rmsnorm_zero_centered(x, w, eps=1e-6):
    y = torch.empty_like(x)
    check(_lib.lib().insg_rmsnorm_zero_centered(_p(x), _p(w), _p(y), x.shape[0], x.shape[1], eps, _stream()))
    return y


def causal_conv4_silu(x, state, w):
    check(_lib.lib().insg_causal_conv4_silu(_p(x), _p(state), _p(w), x.numel(), _stream()))


def deltanet_parameters(a, b, A_log, dt_bias):
    check(_lib.lib().insg_deltanet_parameters(_p(a), _p(b), _p(A_log), _p(dt_bias), a.numel(), _stream()))


def qk_norm_rope(q, k, q_w, k_w, position, fast_trig=True):
    check(_lib.lib().insg_qk_norm_rope(_p(q), _p(k), _p(q_w), _p(k_w), position, int(fast_trig), _stream()))


def silu_mul(gate, up):
    y = torch.empty_like(gate)
    check(_lib.lib().insg_silu_mul(_p(gate), _p(up), _p(y), gate.numel(), _stream()))
    return y


def residual_add(x, delta):
    check(_lib.lib().insg_residual_add(_p(x), _p(delta), x.numel(), _stream()))


def sigmoid_mul(x, gate):
    check(_lib.lib().insg_sigmoid_mul(_p(x), _p(gate), x.numel(), _stream()))


def store_kv(k, v, k_cache, v_cache, position):
    kv = KV_BF16 if k_cache.dtype == torch.bfloat16 else KV_F32
    check(_lib.lib().insg_store_kv(_p(k), _p(v), _p(k_cache), _p(v_cache), position, kv, _stream()))


def split_q_gate(interleaved):
    q = torch.empty(4096, dtype=torch.float32, device=interleaved.device)
    g = torch.empty_like(q)
    check(_lib.lib().insg_split_q_gate(_p(interleaved), _p(q), _p(g), _stream()))
    return q, g


def expand_gate_heads(gate):
    out = torch.empty_like(gate)
    check(_lib.lib().insg_expand_gate_heads(_p(gate), _p(out), _stream()))
    return out


def concat(a, b):
    out = torch.empty(a.numel() * 2, dtype=torch.float32, device=a.device)
    check(_lib.lib().insg_concat(_p(a), _p(b), _p(out), a.numel(), _stream()))
    return out


def argmax_logits(logits):
    out = torch.zeros(1, dtype=torch.int32, device=logits.device)
    check(_lib.lib().insg_argmax_logits(_p(logits), logits.numel(), _p(out), _stream()))
    return out


def bf16_gemv(w, x, pdl=False):
    y = torch.empty(w.shape[0], dtype=torch.float32, device=x.device)
    check(_lib.lib().insg_bf16_gemv(_p(w), _p(x), _p(y), w.shape[0], w.shape[1], int(pdl), _stream()))
    return y
