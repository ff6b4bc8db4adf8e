// The small per-layer launchers of the Qwen3.5 hybrid (bf16 parameters).
//
// Drop-in for the reference header of the same name (include/insignia_qwen_kernels.cuh:5-15, behaviour
// src/qwen_kernels.cu:5-37).  The decode engine fuses all of these into its GEMV, DeltaNet and attention
// kernels; the stand-alone forms exist for drivers that call them one by one (src/dump_attention.cu).
#pragma once
#include "insignia_b200.h"

#include <cuda_runtime.h>

#include <cstdint>

namespace insignia {

inline void rmsnorm_bf16(const float *x, const uint16_t *w, float *y, int rows, int cols, bool zero_centered,
                         cudaStream_t stream = nullptr)
{
    (void)insg_rmsnorm_bf16(x, w, nullptr, y, rows, cols, zero_centered ? 1 : 0, stream);
}

inline void gated_rmsnorm_bf16(const float *x, const uint16_t *w, const float *gate, float *y, int rows, int cols,
                               cudaStream_t stream = nullptr)
{
    (void)insg_rmsnorm_bf16(x, w, gate, y, rows, cols, 0, stream);
}

inline void causal_conv4_silu(float *x, float *state, const uint16_t *weight, int channels, cudaStream_t stream = nullptr)
{
    (void)insg_causal_conv4_silu(x, state, weight, channels, stream);
}

inline void deltanet_parameters(float *a, float *b, const float *A_log, const uint16_t *dt_bias, int heads,
                                cudaStream_t stream = nullptr)
{
    (void)insg_deltanet_parameters(a, b, A_log, dt_bias, heads, stream);
}

inline void expand_gate_heads(const float *head_gate, float *gate256, cudaStream_t stream = nullptr)
{
    (void)insg_expand_gate_heads(head_gate, gate256, stream);
}

inline void sigmoid_mul(float *x, const float *gate, int n, cudaStream_t stream = nullptr)
{
    (void)insg_sigmoid_mul(x, gate, n, stream);
}

inline void split_q_gate(const float *interleaved, float *q, float *gate, cudaStream_t stream = nullptr)
{
    (void)insg_split_q_gate(interleaved, q, gate, stream);
}

inline void store_kv(const float *k, const float *v, float *kc, float *vc, int position, cudaStream_t stream = nullptr)
{
    (void)insg_store_kv(k, v, kc, vc, position, INSG_KV_F32, stream);
}

inline void bf16_gemv(const uint16_t *weight, const float *x, float *y, int rows, int cols, cudaStream_t stream = nullptr)
{
    (void)insg_bf16_gemv(weight, x, y, rows, cols, /*pdl*/ 0, stream);
}

inline void concat(const float *a, const float *b, float *out, int n, cudaStream_t stream = nullptr)
{
    (void)insg_concat(a, b, out, n, stream);
}

inline void argmax_logits(const float *logits, int n, int *device_token, cudaStream_t stream = nullptr)
{
    (void)insg_argmax_logits(logits, n, device_token, stream);
}

} // namespace insignia
