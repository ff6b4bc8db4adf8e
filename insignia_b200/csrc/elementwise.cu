// Stand-alone forms of the reference's small kernels (src/qwen_kernels.cu, src/ops.cu).
// The decode engine fuses all of these into the GEMV / attention / DeltaNet
// kernels; they exist so that every reference free function has a drop-in
// counterpart and so the fused paths can be checked piece by piece.
#include "common.cuh"
#include "host_util.h"

namespace insg {

// rows x cols RMSNorm, bf16 or fp32 weight, optional 1+w, optional * silu(gate)  (src/qwen_kernels.cu:5, src/ops.cu:5)
template <bool WF32> __global__ void __launch_bounds__(256) rmsnorm_kernel(const float *__restrict__ x, const void *__restrict__ w,
                                                                           const float *__restrict__ gate, float *__restrict__ y,
                                                                           int cols, int zero_centered, float eps)
{
    __shared__ float scratch[8];
    const size_t row = blockIdx.x;
    const float *xr = x + row * cols;
    float ss = 0.f;
    for (int i = threadIdx.x; i < cols; i += 256) ss = fmaf(xr[i], xr[i], ss);
    ss = block_sum<8>(ss, scratch);
    const float inv = rsqrtf(ss / float(cols) + eps);
    for (int i = threadIdx.x; i < cols; i += 256) {
        const float wf = WF32 ? static_cast<const float *>(w)[i] : bf16_bits_to_float(static_cast<const uint16_t *>(w)[i]);
        float z = xr[i] * inv * (zero_centered ? 1.0f + wf : wf);
        if (gate) z *= fast_silu(gate[row * cols + i]);
        y[row * cols + i] = z;
    }
}

// src/qwen_kernels.cu:7
__global__ void conv4_silu_kernel(float *x, float *state, const uint16_t *w, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float s0 = state[i * 3], s1 = state[i * 3 + 1], s2 = state[i * 3 + 2], xv = x[i];
    const float z = fmaf(s0, bf16_bits_to_float(w[i * 4]),
                         fmaf(s1, bf16_bits_to_float(w[i * 4 + 1]), fmaf(s2, bf16_bits_to_float(w[i * 4 + 2]), xv * bf16_bits_to_float(w[i * 4 + 3]))));
    state[i * 3] = s1;
    state[i * 3 + 1] = s2;
    state[i * 3 + 2] = xv;
    x[i] = fast_silu(z);
}

// src/qwen_kernels.cu:9
__global__ void delta_params_kernel(float *a, float *b, const float *A_log, const uint16_t *dt, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    b[i] = fast_sigmoid(b[i]);
    const float z = a[i] + bf16_bits_to_float(dt[i]);
    const float soft = z > 20.f ? z : log1pf(__expf(z));
    a[i] = -__expf(A_log[i]) * soft;
}

// src/ops.cu:9 : 20 heads of 256 (16 q + 4 k), one warp per head
__global__ void __launch_bounds__(32) qk_norm_rope_kernel(float *q, float *k, const uint16_t *qw, const uint16_t *kw, int pos, int fast)
{
    const int head = blockIdx.x, lane = threadIdx.x;
    float *p = head < 16 ? q + head * 256 : k + (head - 16) * 256;
    const uint16_t *w = head < 16 ? qw : kw;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] = p[lane * 8 + j];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) ss = fmaf(v[j], v[j], ss);
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / 256.f + 1e-6f);
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] *= inv * bf16_bits_to_float(w[lane * 8 + j]);
    if (pos != 0) {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float other = __shfl_xor_sync(0xffffffffu, v[j], 4);
            if (lane < 8) {
                const int i = lane * 8 + j, half = i & 31;
                float c, s;
                if (fast) {
                    const float a = float(pos) * __powf(10000000.0f, -float(2 * half) / 64.0f);
                    c = __cosf(a);
                    s = __sinf(a);
                } else {
                    const float a = float(pos) * powf(10000000.0f, -float(2 * half) / 64.0f);
                    sincosf(a, &s, &c);
                }
                v[j] = v[j] * c + (i < 32 ? -other : other) * s;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 8; j++) p[lane * 8 + j] = v[j];
}

__global__ void silu_mul_kernel(const float *g, const float *u, float *y, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = fast_silu(g[i]) * u[i];
}
__global__ void add_kernel(float *x, const float *d, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += d[i];
}
__global__ void sigmul_kernel(float *x, const float *g, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] *= fast_sigmoid(g[i]);
}
template <bool BF16> __global__ void store_kv_kernel(const float *k, const float *v, void *kc, void *vc, int pos)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 1024) return;
    const size_t o = size_t(pos) * 1024 + i;
    if (BF16) {
        static_cast<__nv_bfloat16 *>(kc)[o] = __float2bfloat16_rn(k[i]);
        static_cast<__nv_bfloat16 *>(vc)[o] = __float2bfloat16_rn(v[i]);
    } else {
        static_cast<float *>(kc)[o] = k[i];
        static_cast<float *>(vc)[o] = v[i];
    }
}
__global__ void split_q_gate_kernel(const float *src, float *q, float *g)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < 4096) {
        const int h = i >> 8, d = i & 255;
        q[i] = src[h * 512 + d];
        g[i] = src[h * 512 + 256 + d];
    }
}
__global__ void expand_gate_kernel(const float *g, float *out)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < 4096) out[i] = g[(i >> 8) * 256];
}
__global__ void concat_kernel(const float *a, const float *b, float *out, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        out[i] = a[i];
        out[n + i] = b[i];
    }
}

// arg-max with a fixed reduction order, lowest index on ties (src/qwen_kernels.cu:20 is
// single-CTA; so is this, it is not on the engine's path)
// Convolution history after a rejected second token.  `state` holds the history after two tokens (s2, y1, y2) and
// `snapshot` the history before them (s0, s1, s2): after the first token alone it is (s1, s2, y1).
__global__ void conv_rollback_kernel(float *state, const float *snapshot, size_t channels)
{
    const size_t c = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const float y1 = state[c * 3 + 1];
    state[c * 3] = snapshot[c * 3 + 1];
    state[c * 3 + 1] = snapshot[c * 3 + 2];
    state[c * 3 + 2] = y1;
}

// One CTA per row of [count][stride] logits: the arg-max of its first n entries (lowest index on ties).
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const float *x, long long stride, int n, int *out);

// A decode batch's step end: the arg-max of every sequence becomes its next input token and is logged under the
// current position, which then advances.
__global__ void commit_tokens_kernel(const int *next, int *tokens, int *log, int capacity, int *position, int n)
{
    const int pos = *position;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int t = next[i];
        tokens[i] = t;
        if (log && pos >= 0 && pos < capacity) log[size_t(pos) * n + i] = t;
    }
    __syncthreads();
    if (threadIdx.x == 0) *position = pos + 1;
}

__global__ void __launch_bounds__(1024) argmax_kernel(const float *x, int n, int *out)
{
    __shared__ float sv[32];
    __shared__ int si[32];
    float best = -3.402823466e38f;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += 1024) {
        const float v = x[i];
        if (v > best || (v == best && i < idx)) { best = v; idx = i; }
    }
#pragma unroll
    for (int m = 16; m; m >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, m);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, m);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = best; si[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        best = sv[lane];
        idx = si[lane];
#pragma unroll
        for (int m = 16; m; m >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, m);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, m);
            if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
        }
        if (lane == 0) *out = idx == 0x7fffffff ? 0 : idx;
    }
}

// y[rows] = W_bf16[rows][cols] x : one warp per row, 16-byte loads (src/qwen_kernels.cu:25; mtp.fc 4096x8192)
__global__ void __launch_bounds__(256) bf16_gemv_kernel(const uint16_t *__restrict__ w, const float *__restrict__ x, float *__restrict__ y,
                                                        int rows, int cols)
{
    pdl_launch_dependents();
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const uint4 *wr = reinterpret_cast<const uint4 *>(w + size_t(row) * cols);
    const int nvec = cols >> 3;
    pdl_wait();
    float z = 0.f;
#pragma unroll 4
    for (int i = lane; i < nvec; i += 32) {
        const uint4 q = ldg_stream(wr + i);
        const float4 x0 = __ldcg(reinterpret_cast<const float4 *>(x) + i * 2), x1 = __ldcg(reinterpret_cast<const float4 *>(x) + i * 2 + 1);
        z = fmaf(__uint_as_float(q.x << 16), x0.x, z); z = fmaf(__uint_as_float(q.x & 0xffff0000u), x0.y, z);
        z = fmaf(__uint_as_float(q.y << 16), x0.z, z); z = fmaf(__uint_as_float(q.y & 0xffff0000u), x0.w, z);
        z = fmaf(__uint_as_float(q.z << 16), x1.x, z); z = fmaf(__uint_as_float(q.z & 0xffff0000u), x1.y, z);
        z = fmaf(__uint_as_float(q.w << 16), x1.z, z); z = fmaf(__uint_as_float(q.w & 0xffff0000u), x1.w, z);
    }
    z = warp_sum(z);
    if (lane == 0) y[row] = z;
}

static int check_launch(const char *what)
{
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? INSG_OK : cuda_fail(e, what);
}

__global__ void __launch_bounds__(1024) argmax_rows_kernel(const float *x, long long stride, int n, int *out)
{
    __shared__ float sv[32];
    __shared__ int si[32];
    x += size_t(blockIdx.x) * stride;
    float best = -3.402823466e38f;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += 1024) {
        const float v = __ldcg(x + i);
        if (v > best || (v == best && i < idx)) { best = v; idx = i; }
    }
#pragma unroll
    for (int m = 16; m; m >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, m);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, m);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 32; w++)
            if (sv[w] > best || (sv[w] == best && si[w] < idx)) { best = sv[w]; idx = si[w]; }
        out[blockIdx.x] = idx;
    }
}


} // namespace insg

using namespace insg;

extern "C" {

int insg_rmsnorm_bf16(const float *x, const uint16_t *w, const float *gate, float *y, int rows, int cols, int zero_centered,
                      insg_stream_t stream)
{
    if (!x || !w || !y || rows <= 0 || cols <= 0) return fail(INSG_E_ARG, "rmsnorm_bf16: bad argument");
    rmsnorm_kernel<false><<<rows, 256, 0, stream>>>(x, w, gate, y, cols, zero_centered, 1e-6f);
    return check_launch("rmsnorm_bf16");
}
int insg_rmsnorm_zero_centered(const float *x, const float *w, float *y, int rows, int cols, float eps, insg_stream_t stream)
{
    if (!x || !w || !y || rows <= 0 || cols <= 0) return fail(INSG_E_ARG, "rmsnorm_zero_centered: bad argument");
    rmsnorm_kernel<true><<<rows, 256, 0, stream>>>(x, w, nullptr, y, cols, 1, eps);
    return check_launch("rmsnorm_zero_centered");
}
int insg_rmsnorm_gated_silu(const float *x, const float *w, const float *gate, float *y, int rows, int cols, float eps,
                            insg_stream_t stream)
{
    if (!x || !w || !gate || !y || rows <= 0 || cols <= 0) return fail(INSG_E_ARG, "rmsnorm_gated_silu: bad argument");
    rmsnorm_kernel<true><<<rows, 256, 0, stream>>>(x, w, gate, y, cols, 0, eps);
    return check_launch("rmsnorm_gated_silu");
}
int insg_causal_conv4_silu(float *x, float *state, const uint16_t *w, int channels, insg_stream_t stream)
{
    if (!x || !state || !w || channels <= 0) return fail(INSG_E_ARG, "causal_conv4_silu: bad argument");
    conv4_silu_kernel<<<(channels + 255) / 256, 256, 0, stream>>>(x, state, w, channels);
    return check_launch("causal_conv4_silu");
}
int insg_deltanet_parameters(float *a, float *b, const float *A_log, const uint16_t *dt_bias, int heads, insg_stream_t stream)
{
    if (!a || !b || !A_log || !dt_bias || heads <= 0) return fail(INSG_E_ARG, "deltanet_parameters: bad argument");
    delta_params_kernel<<<(heads + 31) / 32, 32, 0, stream>>>(a, b, A_log, dt_bias, heads);
    return check_launch("deltanet_parameters");
}
int insg_qk_norm_rope(float *q, float *k, const uint16_t *q_w, const uint16_t *k_w, int position, int fast_trig, insg_stream_t stream)
{
    if (!q || !k || !q_w || !k_w) return fail(INSG_E_ARG, "qk_norm_rope: null pointer");
    qk_norm_rope_kernel<<<20, 32, 0, stream>>>(q, k, q_w, k_w, position, fast_trig);
    return check_launch("qk_norm_rope");
}
int insg_silu_mul(const float *gate, const float *up, float *y, int n, insg_stream_t stream)
{
    if (!gate || !up || !y || n <= 0) return fail(INSG_E_ARG, "silu_mul: bad argument");
    silu_mul_kernel<<<(n + 255) / 256, 256, 0, stream>>>(gate, up, y, n);
    return check_launch("silu_mul");
}
int insg_residual_add(float *x, const float *delta, int n, insg_stream_t stream)
{
    if (!x || !delta || n <= 0) return fail(INSG_E_ARG, "residual_add: bad argument");
    add_kernel<<<(n + 255) / 256, 256, 0, stream>>>(x, delta, n);
    return check_launch("residual_add");
}
int insg_sigmoid_mul(float *x, const float *gate, int n, insg_stream_t stream)
{
    if (!x || !gate || n <= 0) return fail(INSG_E_ARG, "sigmoid_mul: bad argument");
    sigmul_kernel<<<(n + 255) / 256, 256, 0, stream>>>(x, gate, n);
    return check_launch("sigmoid_mul");
}
int insg_store_kv(const float *k, const float *v, void *k_cache, void *v_cache, int position, int kv_dtype, insg_stream_t stream)
{
    if (!k || !v || !k_cache || !v_cache || position < 0) return fail(INSG_E_ARG, "store_kv: bad argument");
    if (kv_dtype == INSG_KV_BF16) store_kv_kernel<true><<<4, 256, 0, stream>>>(k, v, k_cache, v_cache, position);
    else store_kv_kernel<false><<<4, 256, 0, stream>>>(k, v, k_cache, v_cache, position);
    return check_launch("store_kv");
}
int insg_split_q_gate(const float *interleaved, float *q, float *gate, insg_stream_t stream)
{
    if (!interleaved || !q || !gate) return fail(INSG_E_ARG, "split_q_gate: null pointer");
    split_q_gate_kernel<<<16, 256, 0, stream>>>(interleaved, q, gate);
    return check_launch("split_q_gate");
}
int insg_expand_gate_heads(const float *head_gate, float *gate256, insg_stream_t stream)
{
    if (!head_gate || !gate256) return fail(INSG_E_ARG, "expand_gate_heads: null pointer");
    expand_gate_kernel<<<16, 256, 0, stream>>>(head_gate, gate256);
    return check_launch("expand_gate_heads");
}
int insg_concat(const float *a, const float *b, float *out, int n, insg_stream_t stream)
{
    if (!a || !b || !out || n <= 0) return fail(INSG_E_ARG, "concat: bad argument");
    concat_kernel<<<(n + 255) / 256, 256, 0, stream>>>(a, b, out, n);
    return check_launch("concat");
}
int insg_argmax_logits(const float *logits, int n, int *device_token, insg_stream_t stream)
{
    if (!logits || !device_token || n <= 0) return fail(INSG_E_ARG, "argmax_logits: bad argument");
    argmax_kernel<<<1, 1024, 0, stream>>>(logits, n, device_token);
    return check_launch("argmax_logits");
}
int insg_conv_rollback(float *state, const float *snapshot, long long channels, insg_stream_t stream)
{
    if (!state || !snapshot || channels <= 0) return fail(INSG_E_ARG, "conv_rollback: bad argument");
    conv_rollback_kernel<<<unsigned((channels + 255) / 256), 256, 0, stream>>>(state, snapshot, size_t(channels));
    return check_launch("conv_rollback");
}
int insg_argmax_rows(const float *logits, long long stride, int n, int count, int *device_tokens, insg_stream_t stream)
{
    if (!logits || !device_tokens || n <= 0 || count <= 0 || stride < n) return fail(INSG_E_ARG, "argmax_rows: bad argument");
    argmax_rows_kernel<<<count, 1024, 0, stream>>>(logits, stride, n, device_tokens);
    return check_launch("argmax_rows");
}
int insg_commit_tokens(const int *next, int *tokens, int *log, int capacity, int *position, int n, insg_stream_t stream)
{
    if (!next || !tokens || !position || n <= 0) return fail(INSG_E_ARG, "commit_tokens: bad argument");
    commit_tokens_kernel<<<1, 64, 0, stream>>>(next, tokens, log, capacity, position, n);
    return check_launch("commit_tokens");
}
int insg_bf16_gemv(const uint16_t *w, const float *x, float *y, int rows, int cols, int pdl, insg_stream_t stream)
{
    if (!w || !x || !y || rows <= 0 || cols <= 0 || (cols & 7)) return fail(INSG_E_ARG, "bf16_gemv: bad argument");
    return launch(bf16_gemv_kernel, dim3((rows + 7) / 8), dim3(256), 0, stream, pdl != 0, w, x, y, rows, cols);
}

} // extern "C"
