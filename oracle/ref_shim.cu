// extern "C" driver around the UNMODIFIED reference engine, built into
// oracle/_ref/libinsignia_ref.so together with the reference's own sources.
// TEST INFRASTRUCTURE ONLY: the test-suite loads it with ctypes to obtain the
// reference's outputs (kernel results, per-layer hidden states, greedy token ids)
// on the same inputs as the library under test.  Nothing shipped links it.
//
// Every entry point forwards to the reference function named in its comment.
#include "insignia_attention.cuh"
#include "insignia_decode.hpp"
#include "insignia_deltanet.cuh"
#include "insignia_layout.cuh"
#include "insignia_ops.cuh"
#include "insignia_qwen_kernels.cuh"

#include <cstring>
#include <memory>
#include <string>

namespace {
thread_local std::string g_err;
int fail(const char *what)
{
    g_err = what;
    return -1;
}
int sync_status()
{
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return fail(cudaGetErrorString(e));
    return 0;
}
struct Engine {
    insignia::ModelFile model;
    std::unique_ptr<insignia::Qwen35Weights> weights;
    std::unique_ptr<insignia::DecodeWorkspace> ws;
    std::unique_ptr<insignia::Qwen35Decode> dec;
};
} // namespace

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API const char *ref_last_error() { return g_err.c_str(); }

// ---- kernel-level entry points (device pointers) ---------------------------
// src/mxfp4.cu:68
REF_API int ref_mxfp4_gemv_mlx(const uint32_t *w, const uint8_t *s, const float *x, float *y, int rows, int cols, int warps)
{
    insignia::mxfp4_gemv_mlx(w, s, x, y, rows, cols, warps, nullptr);
    return sync_status();
}
// src/mxfp4.cu:32
REF_API int ref_mxfp4_gemv_block17(const void *blocks, const float *x, float *y, int rows, int cols)
{
    insignia::mxfp4_gemv(static_cast<const insignia::MxFp4Block *>(blocks), x, y, rows, cols, nullptr);
    return sync_status();
}
// src/mxfp4.cu:133
REF_API int ref_mxfp4_get_row_mlx(const uint32_t *w, const uint8_t *s, float *out, int row, int cols)
{
    insignia::mxfp4_get_row_mlx(w, s, out, row, cols, nullptr);
    return sync_status();
}
// src/deltanet.cu:14
REF_API int ref_deltanet_decode(float *state, const float *q, const float *k, const float *v, const float *g,
                                const float *beta, float *out)
{
    insignia::deltanet_decode(state, q, k, v, g, beta, out, nullptr);
    return sync_status();
}
// src/attention.cu:5
REF_API int ref_gqa_decode(const float *q, const float *kc, const float *vc, float *out, int tokens)
{
    insignia::gqa_decode(q, kc, vc, out, tokens, nullptr);
    return sync_status();
}
// src/qwen_kernels.cu:6
REF_API int ref_rmsnorm_bf16(const float *x, const uint16_t *w, float *y, int rows, int cols, int zero_centered)
{
    insignia::rmsnorm_bf16(x, w, y, rows, cols, zero_centered != 0, nullptr);
    return sync_status();
}
REF_API int ref_gated_rmsnorm_bf16(const float *x, const uint16_t *w, const float *gate, float *y, int rows, int cols)
{
    insignia::gated_rmsnorm_bf16(x, w, gate, y, rows, cols, nullptr);
    return sync_status();
}
// src/ops.cu:6
REF_API int ref_rmsnorm_zero_centered(const float *x, const float *w, float *y, int rows, int cols)
{
    insignia::rmsnorm_zero_centered(x, w, y, rows, cols, 1e-6f, nullptr);
    return sync_status();
}
// src/qwen_kernels.cu:8,10
REF_API int ref_causal_conv4_silu(float *x, float *state, const uint16_t *w, int channels)
{
    insignia::causal_conv4_silu(x, state, w, channels, nullptr);
    return sync_status();
}
REF_API int ref_deltanet_parameters(float *a, float *b, const float *A_log, const uint16_t *dt, int heads)
{
    insignia::deltanet_parameters(a, b, A_log, dt, heads, nullptr);
    return sync_status();
}
// src/ops.cu:10
REF_API int ref_qk_norm_rope(float *q, float *k, const uint16_t *qw, const uint16_t *kw, int pos)
{
    insignia::qwen35_qk_norm_rope_gate(q, k, qw, kw, nullptr, pos, nullptr);
    return sync_status();
}
// src/ops.cu:7,8
REF_API int ref_silu_mul(const float *g, const float *u, float *y, int n)
{
    insignia::silu_mul(g, u, y, n, nullptr);
    return sync_status();
}
REF_API int ref_residual_add(float *x, const float *d, int n)
{
    insignia::residual_add(x, d, n, nullptr);
    return sync_status();
}
// src/qwen_kernels.cu:11,16,21,26,27,32,37
REF_API int ref_sigmoid_mul(float *x, const float *g, int n)
{
    insignia::sigmoid_mul(x, g, n, nullptr);
    return sync_status();
}
REF_API int ref_store_kv(const float *k, const float *v, float *kc, float *vc, int pos)
{
    insignia::store_kv(k, v, kc, vc, pos, nullptr);
    return sync_status();
}
REF_API int ref_argmax_logits(const float *x, int n, int *out)
{
    insignia::argmax_logits(x, n, out, nullptr);
    return sync_status();
}
REF_API int ref_bf16_gemv(const uint16_t *w, const float *x, float *y, int rows, int cols)
{
    insignia::bf16_gemv(w, x, y, rows, cols, nullptr);
    return sync_status();
}
REF_API int ref_split_q_gate(const float *src, float *q, float *g)
{
    insignia::split_q_gate(src, q, g, nullptr);
    return sync_status();
}
REF_API int ref_expand_gate_heads(const float *g, float *out)
{
    insignia::expand_gate_heads(g, out, nullptr);
    return sync_status();
}

// ---- whole-engine entry points ---------------------------------------------
// Construction as in src/test_generate.cu:3.
REF_API void *ref_engine_create(const char *index_path, unsigned long long budget_bytes, int max_context)
{
    try {
        std::wstring wide;
        for (const char *p = index_path; *p; ++p) wide.push_back(static_cast<wchar_t>(*p));
        auto e = std::make_unique<Engine>();
        e->model = insignia::ModelFile(wide.c_str());
        e->weights = std::make_unique<insignia::Qwen35Weights>(e->model, budget_bytes);
        e->ws = std::make_unique<insignia::DecodeWorkspace>(max_context);
        e->dec = std::make_unique<insignia::Qwen35Decode>(*e->weights, *e->ws);
        return e.release();
    } catch (const std::exception &ex) {
        g_err = ex.what();
        return nullptr;
    }
}
REF_API void ref_engine_destroy(void *h) { delete static_cast<Engine *>(h); }

#define GUARD(expr)                                                                                                    \
    try {                                                                                                              \
        expr;                                                                                                          \
    } catch (const std::exception &ex) {                                                                               \
        g_err = ex.what();                                                                                             \
        return -1;                                                                                                     \
    }

// src/qwen35.cu:9 into workspace.hidden (src/test_full_model.cu:6)
REF_API int ref_engine_embed(void *h, int token)
{
    auto *e = static_cast<Engine *>(h);
    GUARD(e->weights->embed(token, e->ws->hidden));
    return sync_status();
}
// src/decode.cu:20
REF_API int ref_engine_layer(void *h, int layer)
{
    auto *e = static_cast<Engine *>(h);
    GUARD(e->dec->layer(layer));
    return sync_status();
}
// src/decode.cu:21
REF_API int ref_engine_forward_token(void *h, int token)
{
    auto *e = static_cast<Engine *>(h);
    GUARD(e->dec->forward_token(token));
    return 0;
}
// src/decode.cu:22
REF_API int ref_engine_logits_argmax(void *h)
{
    auto *e = static_cast<Engine *>(h);
    int t = -1;
    GUARD(t = e->dec->logits_argmax());
    return t;
}
// src/decode.cu:23
REF_API int ref_engine_decode_token(void *h, int token)
{
    auto *e = static_cast<Engine *>(h);
    int t = -1;
    GUARD(t = e->dec->decode_token(token));
    return t;
}
// src/decode.cu:24
REF_API int ref_engine_mtp_draft(void *h, int token)
{
    auto *e = static_cast<Engine *>(h);
    int t = -1;
    GUARD(t = e->dec->mtp_draft(token));
    return t;
}
REF_API int ref_engine_position(void *h) { return static_cast<Engine *>(h)->ws->position; }
REF_API void ref_engine_set_position(void *h, int p) { static_cast<Engine *>(h)->ws->position = p; }

// Copies a public workspace buffer (include/insignia_decode.hpp:8) to the host.
REF_API int ref_engine_read(void *h, const char *field, float *out, unsigned long long count)
{
    auto *e = static_cast<Engine *>(h);
    const float *src = nullptr;
    const std::string f = field;
    auto &x = *e->ws;
    if (f == "hidden") src = x.hidden;
    else if (f == "norm") src = x.norm;
    else if (f == "logits") src = x.logits;
    else if (f == "qkv") src = x.qkv;
    else if (f == "core") src = x.core;
    else if (f == "down") src = x.down;
    else if (f == "delta_state") src = x.delta_state;
    else if (f == "conv_state") src = x.conv_state;
    else if (f == "kv_keys") src = x.kv_keys;
    else if (f == "kv_values") src = x.kv_values;
    else return fail("unknown workspace field");
    cudaError_t err = cudaMemcpy(out, src, count * sizeof(float), cudaMemcpyDeviceToHost);
    if (err != cudaSuccess) return fail(cudaGetErrorString(err));
    return 0;
}
