"""ctypes loader for ``libinsignia_b200.so`` (the C ABI in include/insignia_b200.h).

There is no CPU fallback: if the library is missing or fails to load, importing
this module's :func:`lib` raises, and every op built on it fails loudly.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# INSIGNIA_B200_LIB points at another build of the same library (e.g. one compiled with a development macro)
LIB_PATH = os.environ.get("INSIGNIA_B200_LIB") or os.path.join(_HERE, "lib", "libinsignia_b200.so")
_lib = None

vp, i32, u64, sz = C.c_void_p, C.c_int, C.c_uint64, C.c_size_t


class GemvSegment(C.Structure):
    _fields_ = [("packed", vp), ("packed2", vp), ("out", vp), ("rows", i32), ("epilogue", i32), ("conv_state", vp),
                ("conv_w", vp), ("A_log", vp), ("dt_bias", vp), ("prep", vp), ("prep_w", vp), ("prep_partials", vp), ("conv_token_stride", C.c_longlong)]


class GemvOp(C.Structure):
    _fields_ = [("in_", vp), ("aux", vp), ("norm_w", vp), ("x_out", vp), ("cols", i32), ("prologue", i32),
                ("n_segments", i32), ("seg", GemvSegment * 4), ("argmax_scratch", vp), ("token_out", vp),
                ("token_feedback", vp), ("token_log", vp), ("token_log_capacity", i32), ("position_inout", vp), ("layout", i32), ("error_flag", vp), ("pdl", i32),
                ("prep_partials", vp), ("prep_rms", i32), ("tokens", i32), ("umma_scratch", vp), ("umma_scratch_bytes", sz)]


class AttnOp(C.Structure):
    _fields_ = [("qraw", vp), ("k_raw", vp), ("v", vp), ("q_norm_w", vp), ("k_norm_w", vp), ("k_cache", vp),
                ("v_cache", vp), ("out", vp), ("position", vp), ("position_offset", i32), ("max_context", i32),
                ("kv_dtype", i32), ("fast_trig", i32), ("scratch", vp), ("scratch_bytes", sz), ("pdl", i32), ("error_flag", vp)]


class EngineOptions(C.Structure):
    _fields_ = [("device_budget_bytes", u64), ("max_context", i32), ("kv_dtype", i32), ("gate_elementwise", i32),
                ("accurate_trig", i32), ("use_graph", i32), ("use_pdl", i32), ("gemv_tcgen05", i32), ("n_layers", i32), ("vocab", i32),
                ("device", i32), ("persistent", i32), ("prefill_mma_sync", i32), ("gemv_unprepared", i32)]


# name -> (restype, argtypes); every symbol include/insignia_b200.h declares
SIGNATURES = {
    "insg_last_error": (C.c_char_p, []),
    "insg_version": (i32, []),
    "insg_tune_set": (i32, [C.c_char_p, i32]),
    "insg_mxfp4_gemv_mlx": (i32, [vp, vp, vp, vp, i32, i32, vp]),
    "insg_mxfp4_get_row_mlx": (i32, [vp, vp, vp, i32, i32, vp]),
    "insg_mxfp4_gemv_blocks": (i32, [vp, vp, vp, i32, i32, vp]),
    "insg_quantize_q8_groups": (i32, [vp, vp, vp, i32, vp]),
    "insg_mxfp4_gemv_dp4a": (i32, [vp, vp, vp, vp, vp, i32, i32, vp]),
    "insg_mxfp4_embed": (i32, [vp, vp, vp, vp, i32, i32, i32, vp]),
    "insg_mxfp4_embed_tokens": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, vp]),
    "insg_set_scalars": (i32, [vp, i32, vp, i32, vp]),
    "insg_mxfp4_dequant_mlx": (i32, [vp, vp, vp, i32, i32, vp]),
    "insg_mxfp4_packed_bytes": (sz, [i32, i32]),
    "insg_mxfp4_repack": (i32, [vp, vp, vp, i32, i32, vp]),
    "insg_mxfp4_packed_umma_bytes": (sz, [i32, i32]),
    "insg_mxfp4_repack_umma": (i32, [vp, vp, vp, i32, i32, vp]),
    "insg_mxfp4_gemv_packed": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "insg_umma_gemm_scratch_bytes": (sz, [i32, i32]),
    "insg_mxfp4_gemm_umma": (i32, [vp, vp, vp, i32, i32, i32, vp, sz, vp]),
    "insg_gemv_argmax_scratch_bytes": (sz, []),
    "insg_gemv_fused": (i32, [C.POINTER(GemvOp), vp]),
    "insg_program_create": (vp, []),
    "insg_program_destroy": (None, [vp]),
    "insg_program_add_gemv": (i32, [vp, C.POINTER(GemvOp)]),
    "insg_program_add_deltanet": (i32, [vp] * 8),
    "insg_program_add_attention": (i32, [vp, C.POINTER(AttnOp)]),
    "insg_program_add_embed": (i32, [vp, vp, vp, vp, vp, i32, i32]),
    "insg_program_finalize": (i32, [vp]),
    "insg_program_set_option": (i32, [vp, C.c_char_p, C.c_longlong]),
    "insg_program_run": (i32, [vp, i32, i32, i32, vp, vp, vp, vp]),
    "insg_program_recover": (i32, [vp, vp]),
    "insg_program_selftest_barrier_timeout": (i32, [vp, C.c_ulonglong, vp, vp]),
    "insg_program_phase_count": (i32, [vp]),
    "insg_program_weight_bytes": (u64, [vp]),
    "insg_deltanet_decode": (i32, [vp] * 7 + [i32, vp]),
    "insg_deltanet_decode_tokens": (i32, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp]),
    "insg_deltanet_decode_batch": (i32, [vp, C.c_longlong, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp]),
    "insg_deltanet_decode_verify": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, vp]),
    "insg_conv_rollback": (i32, [vp, vp, C.c_longlong, vp]),
    "insg_gqa_scratch_bytes": (sz, [i32]),
    "insg_gqa_decode": (i32, [vp, vp, vp, vp, i32, i32, vp, sz, vp]),
    "insg_gqa_decode_noalloc": (i32, [vp, vp, vp, vp, i32, i32, vp]),
    "insg_comm_create": (vp, [i32, i32, i32]),
    "insg_comm_destroy": (None, [vp]),
    "insg_comm_handle": (i32, [vp, vp]),
    "insg_comm_connect": (i32, [vp, vp]),
    "insg_comm_set_timeout": (i32, [vp, C.c_ulonglong]),
    "insg_comm_error": (i32, [vp, vp, vp]),
    "insg_comm_reset": (i32, [vp, vp]),
    "insg_allreduce_oneshot": (i32, [vp, vp, i32, vp]),
    "insg_comm_connect_local": (i32, [vp, i32]),
    "insg_allreduce_oneshot_local": (i32, [vp, vp, i32, i32, i32, vp]),
    "insg_attention_batch": (i32, [vp, i32, sz, vp]),
    "insg_attention_chunk": (i32, [vp, i32, vp, i32, vp]),
    "insg_attention_step": (i32, [C.POINTER(AttnOp), vp]),
    "insg_rmsnorm_bf16": (i32, [vp, vp, vp, vp, i32, i32, i32, vp]),
    "insg_rmsnorm_zero_centered": (i32, [vp, vp, vp, i32, i32, C.c_float, vp]),
    "insg_rmsnorm_gated_silu": (i32, [vp, vp, vp, vp, i32, i32, C.c_float, vp]),
    "insg_causal_conv4_silu": (i32, [vp, vp, vp, i32, vp]),
    "insg_deltanet_parameters": (i32, [vp, vp, vp, vp, i32, vp]),
    "insg_qk_norm_rope": (i32, [vp, vp, vp, vp, i32, i32, vp]),
    "insg_silu_mul": (i32, [vp, vp, vp, i32, vp]),
    "insg_residual_add": (i32, [vp, vp, i32, vp]),
    "insg_sigmoid_mul": (i32, [vp, vp, i32, vp]),
    "insg_store_kv": (i32, [vp, vp, vp, vp, i32, i32, vp]),
    "insg_split_q_gate": (i32, [vp, vp, vp, vp]),
    "insg_expand_gate_heads": (i32, [vp, vp, vp]),
    "insg_concat": (i32, [vp, vp, vp, i32, vp]),
    "insg_argmax_logits": (i32, [vp, i32, vp, vp]),
    "insg_argmax_rows": (i32, [vp, C.c_longlong, i32, i32, vp, vp]),
    "insg_commit_tokens": (i32, [vp, vp, vp, i32, vp, i32, vp]),
    "insg_bf16_gemv": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "insg_storage_open": (vp, [C.c_char_p, u64, i32]),
    "insg_storage_close": (None, [vp]),
    "insg_storage_acquire": (i32, [vp, C.c_char_p, C.POINTER(vp), C.POINTER(u64)]),
    "insg_storage_release": (i32, [vp, C.c_char_p]),
    "insg_storage_prefetch": (i32, [vp, C.c_char_p]),
    "insg_storage_tier": (i32, [vp, C.c_char_p]),
    "insg_storage_reserve": (i32, [vp, u64]),
    "insg_storage_unreserve": (i32, [vp, u64]),
    "insg_storage_set_host_cache": (i32, [vp, u64]),
    "insg_storage_clear": (i32, [vp]),
    "insg_storage_device_bytes": (u64, [vp]),
    "insg_storage_reserved_bytes": (u64, [vp]),
    "insg_storage_stats": (i32, [vp, C.POINTER(u64)]),
    "insg_engine_create": (vp, [C.c_char_p, C.POINTER(EngineOptions)]),
    "insg_engine_destroy": (None, [vp]),
    "insg_engine_embed": (i32, [vp, i32]),
    "insg_engine_layer": (i32, [vp, i32]),
    "insg_engine_forward_token": (i32, [vp, i32]),
    "insg_engine_forward_tokens": (i32, [vp, vp, i32]),
    "insg_engine_logits_argmax": (i32, [vp]),
    "insg_engine_decode_token": (i32, [vp, i32]),
    "insg_engine_mtp_draft": (i32, [vp, i32]),
    "insg_engine_generate": (i32, [vp, i32, i32, C.POINTER(i32)]),
    "insg_engine_prime_speculative": (i32, [vp, vp, i32]),
    "insg_engine_generate_speculative": (i32, [vp, i32, i32, vp, vp, vp]),
    "insg_engine_profile_gemv_chain": (i32, [vp, i32, vp, vp, vp]),
    "insg_engine_set_program_option": (i32, [vp, C.c_char_p, C.c_longlong]),
    "insg_engine_selftest_barrier_timeout": (i32, [vp]),
    "insg_engine_position": (i32, [vp]),
    "insg_engine_set_position": (i32, [vp, i32]),
    "insg_engine_reset": (i32, [vp]),
    "insg_engine_read": (i32, [vp, C.c_char_p, vp, u64]),
    "insg_engine_write": (i32, [vp, C.c_char_p, vp, u64]),
    "insg_engine_buffer": (vp, [vp, C.c_char_p]),
    "insg_engine_stream": (vp, [vp]),
    "insg_engine_launch_count": (u64, [vp]),
    "insg_engine_device_bytes": (u64, [vp]),
    "insg_batch_create": (vp, [vp, i32, i32]),
    "insg_batch_destroy": (None, [vp]),
    "insg_batch_forward_tokens": (i32, [vp, vp]),
    "insg_batch_decode_tokens": (i32, [vp, vp, vp]),
    "insg_batch_generate": (i32, [vp, vp, i32, vp]),
    "insg_batch_reset": (i32, [vp]),
    "insg_batch_position": (i32, [vp]),
    "insg_batch_read": (i32, [vp, C.c_char_p, i32, vp, u64]),
    "insg_batch_launch_count": (u64, [vp]),
    "insg_batch_stream": (vp, [vp]),
}


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m insignia_b200.build` (there is no CPU fallback)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


class InsigniaError(RuntimeError):
    pass


def check(rc: int) -> int:
    if rc < 0:
        raise InsigniaError(lib().insg_last_error().decode() or f"error {rc}")
    return rc
