/*
 * CPU oracle for the Insignia decode hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C on the host, the arithmetic of the reference
 * (novysvet/insignia) kernels that make up its batch-1 token loop.  It exists so
 * the CUDA kernels of this repository can be checked against an independent
 * implementation of the same algorithm.  Nothing in the shipped library links,
 * loads or calls it: only the test-suite, the smoke check and the CPU-baseline
 * leg of the benchmark do.
 *
 * Every function names the reference file:line it follows (paths relative to
 * the reference project root).  Where the reference reduces with a fixed
 * thread/warp pattern the same pattern is emulated (fmaf per lane, xor-butterfly
 * per warp, second butterfly across warps), so that fp32 rounding follows the
 * reference as closely as a CPU can; transcendental functions use libm where
 * the reference uses the GPU's fast approximations.
 *
 * Parity pin: checked in tests against (1) the deterministic known-answer
 * fixtures of the reference's own kernel tests (src/test_mxfp4.cu,
 * src/bench_mxfp4_mlx.cu, src/test_deltanet.cu, src/test_attention.cu,
 * src/test_ops.cu) under their thresholds and (2) golden vectors produced by
 * the reference's NumPy tools (tools/reference_all_layers.py).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ codec */

/* include/insignia_layout.cuh:20-26 : E2M1 lookup, code 8 is -0.0 */
ORC_API float orc_fp4_e2m1(uint8_t code)
{
    static const float lut[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                  -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};
    return lut[code & 15];
}

/* include/insignia_layout.cuh:28-34 : helper form, 0xff -> NaN */
ORC_API float orc_e8m0(uint8_t x)
{
    uint32_t bits = x == 0xff ? 0x7fffffffu : (uint32_t)x << 23;
    float v;
    memcpy(&v, &bits, 4);
    return v;
}

/* src/mxfp4.cu:52,120,132 : the MLX kernels shift the byte straight into the
 * exponent field, so 0 -> +0.0 and 255 -> +Inf. */
ORC_API float orc_e8m0_mlx(uint8_t x)
{
    uint32_t bits = (uint32_t)x << 23;
    float v;
    memcpy(&v, &bits, 4);
    return v;
}

static inline uint8_t mlx_code(const uint32_t *row_w, int k)
{
    return (uint8_t)((row_w[k >> 3] >> ((k & 7) * 4)) & 15u);
}

/* src/mxfp4.cu:132 and tools/reference_all_layers.py:6 : full dequantisation of
 * an MLX-layout matrix (U32[rows][cols/8], U8[rows][cols/32]) to fp32. */
ORC_API void orc_mxfp4_dequant_mlx(const uint32_t *w, const uint8_t *s, float *out, int rows, int cols)
{
    const int groups = cols >> 5;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) {
        const uint32_t *rw = w + (size_t)r * groups * 4;
        const uint8_t *rs = s + (size_t)r * groups;
        float *o = out + (size_t)r * cols;
        for (int k = 0; k < cols; k++) o[k] = orc_fp4_e2m1(mlx_code(rw, k)) * orc_e8m0_mlx(rs[k >> 5]);
    }
}

/* src/mxfp4.cu:132-133 : one row (the embedding lookup). */
ORC_API void orc_mxfp4_get_row_mlx(const uint32_t *w, const uint8_t *s, float *out, int row, int cols)
{
    const int groups = cols >> 5;
    const uint32_t *rw = w + (size_t)row * groups * 4;
    const uint8_t *rs = s + (size_t)row * groups;
    for (int k = 0; k < cols; k++) out[k] = orc_fp4_e2m1(mlx_code(rw, k)) * orc_e8m0_mlx(rs[k >> 5]);
}

/* xor-butterfly over 32 lanes as __shfl_xor_sync loops of the reference do:
 * after the loop every lane holds the same tree sum. */
static float warp_butterfly_sum(float *lane)
{
    float tmp[32];
    for (int m = 16; m; m >>= 1) {
        for (int l = 0; l < 32; l++) tmp[l] = lane[l] + lane[l ^ m];
        memcpy(lane, tmp, sizeof(tmp));
    }
    return lane[0];
}

static float warp_butterfly_max(float *lane)
{
    float tmp[32];
    for (int m = 16; m; m >>= 1) {
        for (int l = 0; l < 32; l++) tmp[l] = fmaxf(lane[l], lane[l ^ m]);
        memcpy(lane, tmp, sizeof(tmp));
    }
    return lane[0];
}

/* Two-level block reduction used all over the reference: per-warp butterfly,
 * lane 0 of each warp to shared memory, warp 0 butterflies the partials. */
static float block_sum(const float *thread_vals, int nthreads)
{
    const int warps = nthreads >> 5;
    float partial[32];
    for (int i = 0; i < 32; i++) partial[i] = 0.0f;
    for (int w = 0; w < warps; w++) {
        float lane[32];
        memcpy(lane, thread_vals + w * 32, sizeof(lane));
        partial[w] = warp_butterfly_sum(lane);
    }
    if (warps == 1) return partial[0];
    return warp_butterfly_sum(partial);
}

/* src/mxfp4.cu:41-66 : y = W x with the kernel's own summation order.  Lane l
 * of warp w accumulates element l of groups w, w+WARPS, ... with fmaf, then the
 * block reduces. */
ORC_API void orc_mxfp4_gemv_mlx(const uint32_t *w, const uint8_t *s, const float *x, float *y, int rows, int cols,
                                int warps)
{
    if (rows <= 0 || cols <= 0 || (cols & 31)) return; /* src/mxfp4.cu:69 */
    if (warps != 1 && warps != 2 && warps != 8) warps = 4; /* src/mxfp4.cu:71-76 */
    const int groups = cols >> 5;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) {
        const uint32_t *rw = w + (size_t)r * groups * 4;
        const uint8_t *rs = s + (size_t)r * groups;
        float sums[256];
        for (int i = 0; i < warps * 32; i++) sums[i] = 0.0f;
        for (int g = 0; g < groups; g++) {
            const int wp = g % warps;
            const float scale = orc_e8m0_mlx(rs[g]);
            for (int l = 0; l < 32; l++) {
                const float wv = orc_fp4_e2m1(mlx_code(rw, g * 32 + l)) * scale;
                sums[wp * 32 + l] = fmaf(wv, x[g * 32 + l], sums[wp * 32 + l]);
            }
        }
        y[r] = block_sum(sums, warps * 32);
    }
}

/* Double-precision accumulation of the same contraction, as the reference's
 * tests build their expected values (src/bench_mxfp4_mlx.cu:7). */
ORC_API void orc_mxfp4_gemv_mlx_f64(const uint32_t *w, const uint8_t *s, const float *x, double *y, int rows,
                                    int cols)
{
    const int groups = cols >> 5;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) {
        const uint32_t *rw = w + (size_t)r * groups * 4;
        const uint8_t *rs = s + (size_t)r * groups;
        double z = 0.0;
        for (int k = 0; k < cols; k++)
            z += (double)(orc_fp4_e2m1(mlx_code(rw, k)) * orc_e8m0(rs[k >> 5])) * (double)x[k];
        y[r] = z;
    }
}

/* include/insignia_layout.cuh:36-43 and src/mxfp4.cu:5-30 : the 17-byte block
 * layout (scale byte, 16 bytes; lane<16 low nibble of q[lane], else high nibble
 * of q[lane-16]).  Only the reference's own kernel test uses it. */
ORC_API void orc_mxfp4_gemv_block17(const uint8_t *blocks, const float *x, float *y, int rows, int cols)
{
    if (rows <= 0 || cols <= 0 || (cols & 31)) return;
    const int bpr = cols >> 5;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) {
        float sums[256];
        for (int i = 0; i < 256; i++) sums[i] = 0.0f;
        for (int b = 0; b < bpr; b++) {
            const uint8_t *blk = blocks + ((size_t)r * bpr + b) * 17;
            const int wp = b % 8;
            const float scale = orc_e8m0(blk[0]);
            for (int l = 0; l < 32; l++) {
                const uint8_t packed = blk[1 + (l & 15)];
                const uint8_t code = l < 16 ? (packed & 15) : (packed >> 4);
                sums[wp * 32 + l] = fmaf(scale * orc_fp4_e2m1(code), x[b * 32 + l], sums[wp * 32 + l]);
            }
        }
        y[r] = block_sum(sums, 256);
    }
}

/* ------------------------------------------------------------- small ops */

static inline float bf16_to_f32(uint16_t h)
{
    uint32_t bits = (uint32_t)h << 16;
    float v;
    memcpy(&v, &bits, 4);
    return v;
}

static inline float sigmoidf_(float v) { return 1.0f / (1.0f + expf(-v)); }
static inline float siluf_(float v) { return v / (1.0f + expf(-v)); }

/* sum of squares with the 256-thread strided fmaf pattern of
 * src/qwen_kernels.cu:5 / src/ops.cu:5 */
static float strided_sumsq_256(const float *x, int cols)
{
    float t[256];
    for (int i = 0; i < 256; i++) t[i] = 0.0f;
    for (int i = 0; i < cols; i++) t[i & 255] = fmaf(x[i], x[i], t[i & 255]);
    return block_sum(t, 256);
}

/* src/qwen_kernels.cu:5-6 : RMSNorm with bf16 weight, eps 1e-6 inside the
 * root, optional 1+w, optional * silu(gate). */
ORC_API void orc_rmsnorm_bf16(const float *x, const uint16_t *w, const float *gate, float *y, int rows, int cols,
                              int zero_centered)
{
    for (int r = 0; r < rows; r++) {
        const float *xr = x + (size_t)r * cols;
        const float ss = strided_sumsq_256(xr, cols);
        const float inv = 1.0f / sqrtf(ss / (float)cols + 1e-6f);
        for (int i = 0; i < cols; i++) {
            const float wf = bf16_to_f32(w[i]);
            float z = xr[i] * inv * (zero_centered ? 1.0f + wf : wf);
            if (gate) z *= siluf_(gate[(size_t)r * cols + i]);
            y[(size_t)r * cols + i] = z;
        }
    }
}

/* src/ops.cu:5-6 : RMSNorm with fp32 weight and the 1+w convention; only the
 * reference's own ops test exercises it. */
ORC_API void orc_rmsnorm_zero_centered(const float *x, const float *w, float *y, int rows, int cols, float eps)
{
    for (int r = 0; r < rows; r++) {
        const float *xr = x + (size_t)r * cols;
        const float ss = strided_sumsq_256(xr, cols);
        const float inv = 1.0f / sqrtf(ss / (float)cols + eps);
        for (int i = 0; i < cols; i++) y[(size_t)r * cols + i] = xr[i] * inv * (1.0f + w[i]);
    }
}

/* src/qwen_kernels.cu:7 : depthwise causal conv (kernel 4) over n channels with
 * a [channel][3] fp32 history, SiLU, history shift. */
ORC_API void orc_causal_conv4_silu(float *x, float *state, const uint16_t *w, int n)
{
    for (int i = 0; i < n; i++) {
        const float z = fmaf(state[i * 3], bf16_to_f32(w[i * 4]),
                             fmaf(state[i * 3 + 1], bf16_to_f32(w[i * 4 + 1]),
                                  fmaf(state[i * 3 + 2], bf16_to_f32(w[i * 4 + 2]), x[i] * bf16_to_f32(w[i * 4 + 3]))));
        state[i * 3] = state[i * 3 + 1];
        state[i * 3 + 1] = state[i * 3 + 2];
        state[i * 3 + 2] = x[i];
        x[i] = siluf_(z);
    }
}

/* src/qwen_kernels.cu:9 : beta = sigmoid(b); g = -exp(A_log) * softplus(a+dt),
 * softplus linear above 20. */
ORC_API void orc_deltanet_parameters(float *a, float *b, const float *A_log, const uint16_t *dt_bias, int n)
{
    for (int i = 0; i < n; i++) {
        b[i] = sigmoidf_(b[i]);
        const float z = a[i] + bf16_to_f32(dt_bias[i]);
        const float soft = z > 20.0f ? z : log1pf(expf(z));
        a[i] = -expf(A_log[i]) * soft;
    }
}

/* src/deltanet.cu:4-13 : gated delta rule, one token, 32 value heads sharing 16
 * q/k heads (kh = head>>1); state [head][k][v], v contiguous.  The L2-norm
 * epsilon is added to the SUM of squares (src/deltanet.cu:8). */
ORC_API void orc_deltanet_decode(float *state, const float *q16, const float *k16, const float *v, const float *g,
                                 const float *beta, float *out)
{
#pragma omp parallel for schedule(static)
    for (int head = 0; head < 32; head++) {
        const int kh = head >> 1;
        float qt[128], kt[128];
        for (int i = 0; i < 128; i++) {
            qt[i] = q16[kh * 128 + i] * q16[kh * 128 + i];
            kt[i] = k16[kh * 128 + i] * k16[kh * 128 + i];
        }
        /* four warps butterfly, then thread 0 adds the four partials in order */
        float qp[4], kp[4];
        for (int w = 0; w < 4; w++) {
            float lane[32];
            memcpy(lane, qt + w * 32, sizeof(lane));
            qp[w] = warp_butterfly_sum(lane);
            memcpy(lane, kt + w * 32, sizeof(lane));
            kp[w] = warp_butterfly_sum(lane);
        }
        const float qa = qp[0] + qp[1] + qp[2] + qp[3], ka = kp[0] + kp[1] + kp[2] + kp[3];
        const float qs = (1.0f / sqrtf(qa + 1e-6f)) * 0.08838834764831845f;
        const float ks = 1.0f / sqrtf(ka + 1e-6f);
        float *S = state + (size_t)head * 128 * 128;
        const float decay = expf(g[head]);
        for (int j = 0; j < 128; j++) {
            float dot = 0.0f;
            for (int i = 0; i < 128; i++) dot = fmaf(S[i * 128 + j] * decay, k16[kh * 128 + i] * ks, dot);
            const float delta = (v[head * 128 + j] - dot) * beta[head];
            float acc = 0.0f;
            for (int i = 0; i < 128; i++) {
                float cell = fmaf(S[i * 128 + j], decay, k16[kh * 128 + i] * ks * delta);
                S[i * 128 + j] = cell;
                acc = fmaf(cell, q16[kh * 128 + i] * qs, acc);
            }
            out[head * 128 + j] = acc;
        }
    }
}

/* src/ops.cu:9 : per-head RMSNorm over 256 (bf16 weight, not zero-centred),
 * then for position != 0 rotate-half RoPE on dims 0..63 (pairs i, i+32),
 * inv_freq = 1e7^(-2*(i%32)/64).  Heads 0..15 are q, 16..19 are k. */
ORC_API void orc_qk_norm_rope(float *q, float *k, const uint16_t *qw, const uint16_t *kw, int pos)
{
    for (int head = 0; head < 20; head++) {
        float *p = head < 16 ? q + head * 256 : k + (head - 16) * 256;
        const uint16_t *w = head < 16 ? qw : kw;
        float sq[256];
        for (int i = 0; i < 256; i++) sq[i] = p[i] * p[i];
        const float ss = block_sum(sq, 256);
        const float inv = 1.0f / sqrtf(ss / 256.0f + 1e-6f);
        float v[256];
        for (int i = 0; i < 256; i++) v[i] = p[i] * (inv * bf16_to_f32(w[i]));
        if (pos != 0) {
            float r[64];
            for (int i = 0; i < 64; i++) {
                const int half = i & 31;
                const float invf = powf(10000000.0f, -(float)(2 * half) / 64.0f);
                const float a = (float)pos * invf, c = cosf(a), s = sinf(a);
                const float other = v[i < 32 ? i + 32 : i - 32];
                r[i] = v[i] * c + (i < 32 ? -other : other) * s;
            }
            memcpy(v, r, sizeof(r));
        }
        memcpy(p, v, sizeof(v));
    }
}

/* src/qwen_kernels.cu:31 : q_proj output is [16][q256 | gate256]. */
ORC_API void orc_split_q_gate(const float *src, float *q, float *g)
{
    for (int i = 0; i < 4096; i++) {
        const int h = i >> 8, d = i & 255;
        q[i] = src[h * 512 + d];
        g[i] = src[h * 512 + 256 + d];
    }
}

/* src/qwen_kernels.cu:15 */
ORC_API void orc_store_kv(const float *k, const float *v, float *kc, float *vc, int pos)
{
    memcpy(kc + (size_t)pos * 1024, k, 1024 * sizeof(float));
    memcpy(vc + (size_t)pos * 1024, v, 1024 * sizeof(float));
}

/* src/attention.cu:4 : 16 query heads over 4 kv heads (kvh = head>>2), d=256,
 * scale 1/16, full softmax over `tokens`, cache layout [t][4][256].
 * Thread `t%256` owns token t for the max / denominator reductions. */
ORC_API void orc_gqa_decode(const float *q, const float *kc, const float *vc, float *out, int tokens)
{
    if (tokens <= 0) return;
#pragma omp parallel for schedule(static)
    for (int head = 0; head < 16; head++) {
        const int kvh = head >> 2;
        float *score = (float *)malloc((size_t)tokens * sizeof(float));
        float tmax[256], tden[256];
        for (int i = 0; i < 256; i++) { tmax[i] = -3.402823466e+38F; tden[i] = 0.0f; }
        for (int t = 0; t < tokens; t++) {
            float z = 0.0f;
            const float *kr = kc + ((size_t)t * 4 + kvh) * 256;
            for (int d = 0; d < 256; d++) z = fmaf(q[head * 256 + d], kr[d], z);
            z *= 0.0625f;
            score[t] = z;
            tmax[t & 255] = fmaxf(tmax[t & 255], z);
        }
        float partial[32];
        for (int i = 0; i < 32; i++) partial[i] = -3.402823466e+38F;
        for (int w = 0; w < 8; w++) {
            float lane[32];
            memcpy(lane, tmax + w * 32, sizeof(lane));
            partial[w] = warp_butterfly_max(lane);
        }
        const float mx = warp_butterfly_max(partial);
        for (int t = 0; t < tokens; t++) {
            const float e = expf(score[t] - mx);
            score[t] = e;
            tden[t & 255] += e;
        }
        const float inv = 1.0f / block_sum(tden, 256);
        for (int d = 0; d < 256; d++) {
            float z = 0.0f;
            for (int t = 0; t < tokens; t++) z = fmaf(score[t] * inv, vc[((size_t)t * 4 + kvh) * 256 + d], z);
            out[head * 256 + d] = z;
        }
        free(score);
    }
}

/* src/qwen_kernels.cu:36 : element 0 of each head's gate broadcast to the
 * head's 256 lanes (the reference engine's behaviour). */
ORC_API void orc_expand_gate_heads(const float *g, float *out)
{
    for (int i = 0; i < 4096; i++) out[i] = g[(i >> 8) * 256];
}

/* src/qwen_kernels.cu:11 */
ORC_API void orc_sigmoid_mul(float *x, const float *g, int n)
{
    for (int i = 0; i < n; i++) x[i] *= sigmoidf_(g[i]);
}

/* src/ops.cu:7 */
ORC_API void orc_silu_mul(const float *g, const float *u, float *y, int n)
{
    for (int i = 0; i < n; i++) y[i] = siluf_(g[i]) * u[i];
}

/* src/ops.cu:8 */
ORC_API void orc_residual_add(float *x, const float *d, int n)
{
    for (int i = 0; i < n; i++) x[i] += d[i];
}

/* src/qwen_kernels.cu:25 : bf16 weight x fp32 activation, 256-thread strided
 * fmaf then block reduce (mtp.fc). */
ORC_API void orc_bf16_gemv(const uint16_t *w, const float *x, float *y, int rows, int cols)
{
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) {
        float t[256];
        for (int i = 0; i < 256; i++) t[i] = 0.0f;
        const uint16_t *wr = w + (size_t)r * cols;
        for (int i = 0; i < cols; i++) t[i & 255] = fmaf(bf16_to_f32(wr[i]), x[i], t[i & 255]);
        y[r] = block_sum(t, 256);
    }
}

/* src/qwen_kernels.cu:27 */
ORC_API void orc_concat(const float *a, const float *b, float *out, int n)
{
    memcpy(out, a, (size_t)n * sizeof(float));
    memcpy(out + n, b, (size_t)n * sizeof(float));
}

/* src/qwen_kernels.cu:20 : strict '>' everywhere.  A thread keeps the first
 * maximum of its stride; in the butterflies a lane keeps its own value on a
 * tie, so lane 0 ends with the maximum whose owner is earliest in lane order.
 * The emulation follows that order exactly. */
ORC_API int orc_argmax(const float *x, int n)
{
    float bv[256];
    int bi[256];
    for (int t = 0; t < 256; t++) { bv[t] = -3.402823466e38F; bi[t] = 0; }
    for (int i = 0; i < n; i++) {
        const int t = i & 255;
        if (x[i] > bv[t]) { bv[t] = x[i]; bi[t] = i; }
    }
    float wv[32];
    int wi[32];
    for (int i = 0; i < 32; i++) { wv[i] = -3.402823466e38F; wi[i] = 0; }
    for (int w = 0; w < 8; w++) {
        float v[32], tv[32];
        int id[32], ti[32];
        memcpy(v, bv + w * 32, sizeof(v));
        memcpy(id, bi + w * 32, sizeof(id));
        for (int m = 16; m; m >>= 1) {
            for (int l = 0; l < 32; l++) {
                tv[l] = v[l]; ti[l] = id[l];
                if (v[l ^ m] > v[l]) { tv[l] = v[l ^ m]; ti[l] = id[l ^ m]; }
            }
            memcpy(v, tv, sizeof(v));
            memcpy(id, ti, sizeof(id));
        }
        wv[w] = v[0];
        wi[w] = id[0];
    }
    {
        float tv[32];
        int ti[32];
        for (int m = 16; m; m >>= 1) {
            for (int l = 0; l < 32; l++) {
                tv[l] = wv[l]; ti[l] = wi[l];
                if (wv[l ^ m] > wv[l]) { tv[l] = wv[l ^ m]; ti[l] = wi[l ^ m]; }
            }
            memcpy(wv, tv, sizeof(wv));
            memcpy(wi, ti, sizeof(wi));
        }
    }
    return wi[0];
}

/* ---------------------------------------------------------------- helpers */

/* Fast GEMV for the timed CPU baseline: same contraction as
 * orc_mxfp4_gemv_mlx, fp32 accumulate per group with the scale applied once
 * per group, all host threads.  Not bit-identical to the emulated order; used
 * where the oracle is timed rather than compared bit for bit. */
ORC_API void orc_mxfp4_gemv_mlx_fast(const uint32_t *w, const uint8_t *s, const float *x, float *y, int rows,
                                     int cols)
{
    static const float lut[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                  -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};
    const int groups = cols >> 5;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) {
        const uint32_t *rw = w + (size_t)r * groups * 4;
        const uint8_t *rs = s + (size_t)r * groups;
        float total = 0.0f;
        for (int g = 0; g < groups; g++) {
            float acc = 0.0f;
            for (int i = 0; i < 4; i++) {
                const uint32_t p = rw[g * 4 + i];
                const float *xx = x + g * 32 + i * 8;
                for (int j = 0; j < 8; j++) acc += lut[(p >> (4 * j)) & 15] * xx[j];
            }
            total += acc * orc_e8m0_mlx(rs[g]);
        }
        y[r] = total;
    }
}

ORC_API int orc_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
