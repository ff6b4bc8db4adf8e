// MXFP4 weight-streaming GEMV for sm_100a (batch-1 decode and up to 4 tokens).
//
// Contraction (reference: src/mxfp4.cu:41-66): y[r] = sum_k lut[code(r,k)] * 2^(s(r,k/32)-127) * x[k].
//
// The path is HBM-bound: 17 bytes arrive per 32 weights and the SM can afford
// ~2 issue slots per weight at full bandwidth, so the scalar dequant+fmaf of the
// reference (6+ slots per weight) cannot stream at speed.  This kernel
//   * reads a tile-interleaved copy of the weights (see insg_mxfp4_repack) with
//     fully coalesced 128-bit loads, two kblocks deep per thread, issued before
//     the programmatic-dependent-launch wait so they overlap the previous
//     kernel's tail;
//   * expands E2M1 nibbles to fp16 pairs (exactly representable) with either the
//     hardware cvt.rn.f16x2.e2m1x2 or a shift/mask placement into the fp16
//     exponent field;
//   * lets mma.sync.m16n8k16 (fp16 in, fp32 accumulate) do the multiply-adds.
//     The activation vector is split into two fp16 pieces (hi + lo*2^-11, after
//     an exact power-of-two pre-scale) so the product keeps ~22 bits of x;
//   * the 8 columns of the MMA's B operand are used as (4 scale groups) x (hi,
//     lo): thread t of a quad owns scale group t of the 128-wide K block, so the
//     accumulator columns separate the four groups and the E8M0 scale is applied
//     once per (row, group) on the fp32 accumulators, not per weight.
// Prologue (RMSNorm etc.) and epilogue (residual, conv+SiLU, SwiGLU, arg-max)
// of the surrounding elementwise kernels are fused in.
#include "common.cuh"
#include "host_util.h"

#include <mutex>

namespace insg {

constexpr int kRec = 1088;            // bytes per (16-row tile, 128-k block): 1024 nibble bytes + 64 scale bytes
constexpr float kLoScale = 1.0f / 2048.0f;

struct SegDev {
    const uint8_t *packed, *packed2;
    float *out;
    float *conv_state;
    const uint16_t *conv_w;
    const float *A_log;
    const uint16_t *dt_bias;
    int tile_begin, tile_end, epilogue, rows;
};

struct GemvParams {
    const float *in, *aux;
    const uint16_t *norm_w;
    float *x_out;
    int cols, prologue, nseg, total_tiles;
    SegDev seg[4];
    float2 *argmax_partial; // [grid] (value, index as int bits)
    unsigned *ticket;
    int *token_out, *token_feedback, *token_log, *position_inout;
    int ksplit, gpc; // warps per tile group, groups per CTA
};

// ---- E2M1 x8 (one u32) -> four fp16x2 registers -----------------------------
// DEQ 0: hardware convert; register b holds elements (2b, 2b+1) at their true value.
// DEQ 1: shift/mask; register p holds elements (p, p+4) at value * 2^-14.
template <int DEQ> __device__ __forceinline__ void dequant8(uint32_t q, uint32_t (&h)[4])
{
    if constexpr (DEQ == 0) {
        asm("{\n"
            " .reg .b8 b0, b1, b2, b3;\n"
            " mov.b32 {b0, b1, b2, b3}, %4;\n"
            " cvt.rn.f16x2.e2m1x2 %0, b0;\n"
            " cvt.rn.f16x2.e2m1x2 %1, b1;\n"
            " cvt.rn.f16x2.e2m1x2 %2, b2;\n"
            " cvt.rn.f16x2.e2m1x2 %3, b3;\n"
            "}\n"
            : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
            : "r"(q));
    } else {
        h[0] = ((q << 9) & 0x0E000E00u) | ((q << 12) & 0x80008000u);
        h[1] = ((q << 5) & 0x0E000E00u) | ((q << 8) & 0x80008000u);
        h[2] = ((q << 1) & 0x0E000E00u) | ((q << 4) & 0x80008000u);
        h[3] = ((q >> 3) & 0x0E000E00u) | (q & 0x80008000u);
    }
}

// position of element j (0..7) of an 8-block inside the fp16 activation copy
template <int DEQ> __device__ __forceinline__ int xpos(int j) { return DEQ == 0 ? j : ((j & 3) * 2 + (j >> 2)); }

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int UNR> struct Chunk {
    uint4 wa[UNR], wb[UNR];
    uint32_t sc[UNR];
};

struct Cursor {
    int tile, mat, chunk;
    const uint8_t *base; // record 0 of (tile, mat)
    int seg;
    bool valid;
};

__device__ __forceinline__ int find_seg(const GemvParams &p, int tile)
{
    int s = 0;
#pragma unroll
    for (int i = 1; i < 4; i++)
        if (i < p.nseg && tile >= p.seg[i].tile_begin) s = i;
    return s;
}

__device__ __forceinline__ void cursor_set(const GemvParams &p, Cursor &c, int nkb)
{
    c.valid = c.tile < p.total_tiles;
    if (!c.valid) return;
    c.seg = find_seg(p, c.tile);
    const SegDev &s = p.seg[c.seg];
    c.base = (c.mat ? s.packed2 : s.packed) + size_t(c.tile - s.tile_begin) * nkb * kRec;
}

__device__ __forceinline__ Cursor cursor_next(const GemvParams &p, const Cursor &c, int nchunk, int nkb, int stride)
{
    Cursor n = c;
    if (c.chunk + 1 < nchunk) {
        n.chunk = c.chunk + 1;
        return n;
    }
    n.chunk = 0;
    if (c.mat == 0 && p.seg[c.seg].epilogue == INSG_EPI_SWIGLU) {
        n.mat = 1;
    } else {
        n.mat = 0;
        n.tile = c.tile + stride;
    }
    cursor_set(p, n, nkb);
    return n;
}

template <int UNR> __device__ __forceinline__ void load_chunk(Chunk<UNR> &b, const Cursor &c, int kb0, int kb1, int lane)
{
#pragma unroll
    for (int u = 0; u < UNR; u++) {
        const int kb = kb0 + c.chunk * UNR + u;
        if (kb < kb1) {
            const uint8_t *rec = c.base + size_t(kb) * kRec;
            b.wa[u] = ldg_stream(rec + lane * 16);
            b.wb[u] = ldg_stream(rec + 512 + lane * 16);
            b.sc[u] = ldg_stream_u16(rec + 1024 + lane * 2);
        } else {
            b.wa[u] = make_uint4(0, 0, 0, 0);
            b.wb[u] = make_uint4(0, 0, 0, 0);
            b.sc[u] = 0;
        }
    }
}

template <int DEQ, int UNR, int M>
__device__ __forceinline__ void compute_chunk(const Chunk<UNR> &b, const Cursor &c, int kb0, int kb1, const __half *xs,
                                              int xstride, bool bactive, int grp, int piece, float (&acc)[M][4])
{
#pragma unroll
    for (int u = 0; u < UNR; u++) {
        const int kb = kb0 + c.chunk * UNR + u;
        if (kb >= kb1) continue; // uniform per warp
        float cc[M][4];
#pragma unroll
        for (int m = 0; m < M; m++) cc[m][0] = cc[m][1] = cc[m][2] = cc[m][3] = 0.f;
        const uint32_t wa[4] = {b.wa[u].x, b.wa[u].y, b.wa[u].z, b.wa[u].w};
        const uint32_t wb[4] = {b.wb[u].x, b.wb[u].y, b.wb[u].z, b.wb[u].w};
#pragma unroll
        for (int w = 0; w < 4; w++) {
            uint32_t ha[4], hb[4];
            dequant8<DEQ>(wa[w], ha);
            dequant8<DEQ>(wb[w], hb);
#pragma unroll
            for (int m = 0; m < M; m++) {
                uint4 xv = make_uint4(0, 0, 0, 0);
                if (bactive)
                    xv = *reinterpret_cast<const uint4 *>(xs + size_t(m * 2 + piece) * xstride + kb * 128 + grp * 32 + w * 8);
                mma16816(cc[m], ha[0], hb[0], ha[1], hb[1], xv.x, xv.y);
                mma16816(cc[m], ha[2], hb[2], ha[3], hb[3], xv.z, xv.w);
            }
        }
        const float s0 = e8m0_to_float(b.sc[u] & 0xffu), s1 = e8m0_to_float(b.sc[u] >> 8);
#pragma unroll
        for (int m = 0; m < M; m++) {
            acc[m][0] = fmaf(cc[m][0], s0, acc[m][0]);
            acc[m][1] = fmaf(cc[m][1], s0, acc[m][1]);
            acc[m][2] = fmaf(cc[m][2], s1, acc[m][2]);
            acc[m][3] = fmaf(cc[m][3], s1, acc[m][3]);
        }
    }
}

// Block-wide reductions for a run-time warp count (<= 16); `scratch` needs 16 floats.
__device__ __forceinline__ float block_sum_dyn(float v, float *scratch, int nwarps)
{
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nwarps; i++) t += scratch[i];
    return t;
}
__device__ __forceinline__ float block_max_dyn(float v, float *scratch, int nwarps)
{
    v = warp_max(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = scratch[0];
    for (int i = 1; i < nwarps; i++) t = fmaxf(t, scratch[i]);
    return t;
}

// ---- activation prologue: fp32 vector -> two fp16 pieces in shared memory ----
// Returns 1/alpha (the factor that undoes the power-of-two pre-scale).  Activations are
// read with ld.global.cg: under programmatic dependent launch this CTA may have been
// resident (and its L1 filled) before the producing kernel wrote them.
template <int DEQ>
__device__ float prologue(const GemvParams &p, int m, __half *xs, int xstride, float *scratch)
{
    const int cols = p.cols, tid = threadIdx.x, lane = tid & 31, nthreads = blockDim.x, nwarps = nthreads >> 5;
    const float *in = p.in + size_t(m) * cols;
    const int nvec = cols >> 2;
    float inv_rms = 1.f;
    if (p.prologue == INSG_PRO_RMSNORM) {
        float ss = 0.f;
        for (int i = tid; i < nvec; i += nthreads) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(in) + i);
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
        ss = block_sum_dyn(ss, scratch, nwarps);
        inv_rms = rsqrtf(ss / float(cols) + 1e-6f);
    }
    // The transformed vector is evaluated twice (once for its maximum, once for the split)
    // instead of being staged in fp32: the inputs sit in L2 and K = 12288 would not fit.
    auto value4 = [&](int i) -> float4 {
        float4 v = __ldcg(reinterpret_cast<const float4 *>(in) + i);
        const int k = i << 2;
        switch (p.prologue) {
        case INSG_PRO_RMSNORM: {
            const uint2 wv = reinterpret_cast<const uint2 *>(p.norm_w)[i];
            v.x = v.x * inv_rms * bf16_bits_to_float(wv.x & 0xffff);
            v.y = v.y * inv_rms * bf16_bits_to_float(wv.x >> 16);
            v.z = v.z * inv_rms * bf16_bits_to_float(wv.y & 0xffff);
            v.w = v.w * inv_rms * bf16_bits_to_float(wv.y >> 16);
            break;
        }
        case INSG_PRO_GATED_RMSNORM: {
            // one warp covers one 128-wide head per iteration (32 lanes x float4)
            float ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
            ss = warp_sum(ss);
            const float inv = rsqrtf(ss / 128.f + 1e-6f);
            const uint2 wv = reinterpret_cast<const uint2 *>(p.norm_w)[lane];
            const float4 z = __ldcg(reinterpret_cast<const float4 *>(p.aux + size_t(m) * cols) + i);
            v.x = v.x * inv * bf16_bits_to_float(wv.x & 0xffff) * fast_silu(z.x);
            v.y = v.y * inv * bf16_bits_to_float(wv.x >> 16) * fast_silu(z.y);
            v.z = v.z * inv * bf16_bits_to_float(wv.y & 0xffff) * fast_silu(z.z);
            v.w = v.w * inv * bf16_bits_to_float(wv.y >> 16) * fast_silu(z.w);
            break;
        }
        case INSG_PRO_SIGMOID_GATE: {
            const float4 g = __ldcg(reinterpret_cast<const float4 *>(p.aux + size_t(m) * cols) + i);
            v.x *= fast_sigmoid(g.x); v.y *= fast_sigmoid(g.y); v.z *= fast_sigmoid(g.z); v.w *= fast_sigmoid(g.w);
            break;
        }
        case INSG_PRO_SIGMOID_GATE_HEAD0: {
            const float g = fast_sigmoid(__ldcg(p.aux + size_t(m) * 2 * cols + (k >> 8) * 512 + 256));
            v.x *= g; v.y *= g; v.z *= g; v.w *= g;
            break;
        }
        case INSG_PRO_SIGMOID_GATE_QPROJ: {
            const float4 g =
                __ldcg(reinterpret_cast<const float4 *>(p.aux + size_t(m) * 2 * cols + (k >> 8) * 512 + 256 + (k & 255)));
            v.x *= fast_sigmoid(g.x); v.y *= fast_sigmoid(g.y); v.z *= fast_sigmoid(g.z); v.w *= fast_sigmoid(g.w);
            break;
        }
        default: break;
        }
        return v;
    };
    float amax = 0.f;
    for (int i = tid; i < nvec; i += nthreads) {
        const float4 v = value4(i);
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        if (p.x_out && blockIdx.x == 0) reinterpret_cast<float4 *>(p.x_out + size_t(m) * cols)[i] = v;
    }
    const float tmax = block_max_dyn(amax, scratch, nwarps);
    // alpha = 2^(12 - floor(log2(max))) keeps the largest element in [2^12, 2^13)
    int eb = int((__float_as_uint(tmax) >> 23) & 0xffu);
    eb = min(max(eb, 20), 240);
    const float alpha = __uint_as_float(uint32_t(266 - eb) << 23);
    const float inv_alpha = __uint_as_float(uint32_t(eb - 12) << 23);
    __half *hi = xs + size_t(m * 2) * xstride, *lo = hi + xstride;
    for (int i = tid; i < nvec; i += nthreads) {
        const float4 v = value4(i);
        const float e[4] = {v.x * alpha, v.y * alpha, v.z * alpha, v.w * alpha};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int k = (i << 2) + j;
            const int pos = (k & ~7) + xpos<DEQ>(k & 7);
            const __half h = __float2half_rn(e[j]);
            hi[pos] = h;
            lo[pos] = __float2half_rn((e[j] - __half2float(h)) * 2048.0f);
        }
    }
    return inv_alpha;
}

__device__ __forceinline__ void group_barrier(int id, int threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Work decomposition: a GROUP of `ksplit` warps owns a 16-row tile and splits its K range;
// a CTA holds `gpc` groups; group G of the grid walks tiles G, G+groups, ...  Warps never
// meet at a CTA-wide barrier after the prologue, so while one warp waits on its weight
// loads the others compute.  Each warp runs a two-deep software pipeline (loads of chunk
// n+1 in flight while chunk n is multiplied) that continues across tile boundaries.
template <int DEQ, int UNR, int M>
__global__ void __launch_bounds__(512, 1) gemv_fused_kernel(const __grid_constant__ GemvParams p)
{
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int nkb = p.cols >> 7;
    const int xstride = p.cols + 8;
    const int ksplit = p.ksplit, gpc = p.gpc;
    __half *xs = reinterpret_cast<__half *>(smem_raw);
    float *red = reinterpret_cast<float *>(smem_raw + size_t(M) * 2 * xstride * sizeof(__half)); // [gpc][2][ksplit][M][16]
    float *scratch = red + size_t(gpc) * 2 * ksplit * M * 16;                                    // 64 floats
    __shared__ int s_last;

    pdl_launch_dependents();

    const int grp_local = warp / ksplit, wk = warp - grp_local * ksplit;
    const int kb0 = (wk * nkb) / ksplit, kb1 = ((wk + 1) * nkb) / ksplit;
    const int span = (nkb + ksplit - 1) / ksplit;
    const int nchunk = max(1, (span + UNR - 1) / UNR);
    const int stride = int(gridDim.x) * gpc;

    Cursor cur;
    cur.tile = grp_local < gpc ? int(blockIdx.x) * gpc + grp_local : p.total_tiles; // spare warps idle
    cur.mat = 0;
    cur.chunk = 0;
    cursor_set(p, cur, nkb);
    Chunk<UNR> A, B;
    if (cur.valid) load_chunk<UNR>(A, cur, kb0, kb1, lane);

    pdl_wait();

    float inv_alpha[M];
#pragma unroll
    for (int m = 0; m < M; m++) inv_alpha[m] = prologue<DEQ>(p, m, xs, xstride, scratch);
    __syncthreads();

    const bool bactive = (t == (g >> 1));
    const int piece = g & 1;
    float acc[M][4];
#pragma unroll
    for (int m = 0; m < M; m++) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
    float gate_val = 0.f; // gate_proj result held by the row's lane while up_proj streams
    float best = -3.402823466e38f;
    int best_idx = 0x7fffffff;
    int parity = 0;
    float *gred = red + size_t(grp_local) * 2 * ksplit * M * 16;

    auto finish = [&](const Cursor &c) {
        float y[M];
#pragma unroll
        for (int m = 0; m < M; m++) {
            // fold hi/lo pieces, sum the quad (4 scale groups); lanes 0..15 then hold rows 0..15 of the tile
            float v0 = fmaf(acc[m][1], kLoScale, acc[m][0]);
            float v1 = fmaf(acc[m][3], kLoScale, acc[m][2]);
            v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
            v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
            const float r0 = __shfl_sync(0xffffffffu, v0, (lane & 7) * 4);
            const float r1 = __shfl_sync(0xffffffffu, v1, (lane & 7) * 4);
            y[m] = (lane & 8) ? r1 : r0;
            acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
        }
        if (ksplit > 1) {
            float *r = gred + size_t(parity) * ksplit * M * 16;
            if (lane < 16) {
#pragma unroll
                for (int m = 0; m < M; m++) r[(wk * M + m) * 16 + lane] = y[m];
            }
            group_barrier(1 + grp_local, 32 * ksplit);
            if (wk == 0 && lane < 16) {
#pragma unroll
                for (int m = 0; m < M; m++) {
                    float z = 0.f;
                    for (int w = 0; w < ksplit; w++) z += r[(w * M + m) * 16 + lane];
                    y[m] = z;
                }
            }
            parity ^= 1;
        }
        if (wk == 0 && lane < 16) {
            const SegDev &s = p.seg[c.seg];
            const int row = (c.tile - s.tile_begin) * 16 + lane;
#pragma unroll
            for (int m = 0; m < M; m++) {
                const float v = y[m] * inv_alpha[m] * (DEQ == 1 ? 16384.0f : 1.0f);
                float *out = s.out + size_t(m) * s.rows;
                switch (s.epilogue) {
                case INSG_EPI_STORE: out[row] = v; break;
                case INSG_EPI_RESIDUAL: out[row] = __ldcg(out + row) + v; break;
                case INSG_EPI_CONV_SILU: {
                    float *st = s.conv_state + size_t(row) * 3;
                    const uint2 wv = reinterpret_cast<const uint2 *>(s.conv_w)[row];
                    const float w0 = bf16_bits_to_float(wv.x & 0xffff), w1 = bf16_bits_to_float(wv.x >> 16);
                    const float w2 = bf16_bits_to_float(wv.y & 0xffff), w3 = bf16_bits_to_float(wv.y >> 16);
                    const float s0 = __ldcg(st), s1 = __ldcg(st + 1), s2 = __ldcg(st + 2);
                    const float z = fmaf(s0, w0, fmaf(s1, w1, fmaf(s2, w2, v * w3)));
                    st[0] = s1; st[1] = s2; st[2] = v;
                    out[row] = fast_silu(z);
                    break;
                }
                case INSG_EPI_BETA: out[row] = fast_sigmoid(v); break;
                case INSG_EPI_DECAY: {
                    const float z = v + bf16_bits_to_float(s.dt_bias[row]);
                    const float soft = z > 20.f ? z : log1pf(__expf(z));
                    out[row] = -__expf(s.A_log[row]) * soft;
                    break;
                }
                case INSG_EPI_SWIGLU:
                    if (c.mat == 0) gate_val = v;
                    else out[row] = fast_silu(gate_val) * v;
                    break;
                case INSG_EPI_LOGITS:
                    out[row] = v;
                    if (v > best || (v == best && row < best_idx)) { best = v; best_idx = row; }
                    break;
                default: break;
                }
            }
        }
    };

    while (cur.valid) {
        Cursor n1 = cursor_next(p, cur, nchunk, nkb, stride);
        if (n1.valid) load_chunk<UNR>(B, n1, kb0, kb1, lane);
        compute_chunk<DEQ, UNR, M>(A, cur, kb0, kb1, xs, xstride, bactive, t, piece, acc);
        if (cur.chunk == nchunk - 1) finish(cur);
        if (!n1.valid) break;
        Cursor n2 = cursor_next(p, n1, nchunk, nkb, stride);
        if (n2.valid) load_chunk<UNR>(A, n2, kb0, kb1, lane);
        compute_chunk<DEQ, UNR, M>(B, n1, kb0, kb1, xs, xstride, bactive, t, piece, acc);
        if (n1.chunk == nchunk - 1) finish(n1);
        cur = n2;
    }

    // ---- arg-max over the rows this launch produced (lm_head) ----------------
    if (p.argmax_partial) {
        float *sv = scratch + 16;                                  // [16]
        int *si = reinterpret_cast<int *>(scratch + 32);          // [16]
#pragma unroll
        for (int mk = 8; mk; mk >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, mk);
            const int oi = __shfl_xor_sync(0xffffffffu, best_idx, mk);
            if (ov > best || (ov == best && oi < best_idx)) { best = ov; best_idx = oi; }
        }
        if (lane == 0) { sv[warp] = (wk == 0) ? best : -3.402823466e38f; si[warp] = (wk == 0) ? best_idx : 0x7fffffff; }
        __syncthreads();
        if (tid == 0) {
            float bv = sv[0];
            int bi = si[0];
            for (int w = 1; w < nwarps; w++)
                if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
            p.argmax_partial[blockIdx.x] = make_float2(bv, __int_as_float(bi));
            __threadfence();
            const unsigned ticket = atomicAdd(p.ticket, 1u);
            s_last = (ticket == gridDim.x - 1);
        }
        __syncthreads();
        if (s_last) {
            __threadfence();
            float bv = -3.402823466e38f;
            int bi = 0x7fffffff;
            for (int i = tid; i < int(gridDim.x); i += int(blockDim.x)) {
                const volatile float *e = reinterpret_cast<const volatile float *>(p.argmax_partial + i);
                const float ev = e[0];
                const int idx = __float_as_int(e[1]);
                if (ev > bv || (ev == bv && idx < bi)) { bv = ev; bi = idx; }
            }
#pragma unroll
            for (int mk = 16; mk; mk >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, mk);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, mk);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            __syncthreads();
            if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
            __syncthreads();
            if (tid == 0) {
                for (int w = 1; w < nwarps; w++)
                    if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
                *p.token_out = bi;
                if (p.token_feedback) *p.token_feedback = bi;
                if (p.position_inout) {
                    const int pos = *p.position_inout;
                    if (p.token_log) p.token_log[pos] = bi;
                    *p.position_inout = pos + 1;
                }
                *p.ticket = 0u;
            }
        }
    }
}

// ---- repack: MLX layout -> tile-interleaved records ---------------------------
__global__ void repack_kernel(const uint32_t *__restrict__ w, const uint8_t *__restrict__ s, uint8_t *__restrict__ out,
                              int rows, int cols)
{
    const int nkb = cols >> 7;
    const size_t rec_id = size_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const size_t nrec = size_t(rows >> 4) * nkb;
    if (rec_id >= nrec) return;
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int tile = int(rec_id / nkb), kb = int(rec_id % nkb);
    uint8_t *rec = out + rec_id * kRec;
    const int words_per_row = cols >> 3, groups_per_row = cols >> 5;
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const size_t row = size_t(tile) * 16 + g + half * 8;
        const uint4 v = *reinterpret_cast<const uint4 *>(w + row * words_per_row + kb * 16 + t * 4);
        *reinterpret_cast<uint4 *>(rec + half * 512 + lane * 16) = v;
        rec[1024 + lane * 2 + half] = s[row * groups_per_row + kb * 4 + t];
    }
}

// ---- plain SIMT kernel on the MLX layout (stand-alone API, any rows) ----------
// One warp per row; lane L owns scale groups L, L+32, ... (a 16-byte load is one
// whole group), fp32 fmaf, shuffle tree.
__global__ void __launch_bounds__(256) gemv_mlx_kernel(const uint32_t *__restrict__ w, const uint8_t *__restrict__ s,
                                                       const float *__restrict__ x, float *__restrict__ y, int rows,
                                                       int cols)
{
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int groups = cols >> 5;
    const uint4 *rw = reinterpret_cast<const uint4 *>(w + size_t(row) * groups * 4);
    const uint8_t *rs = s + size_t(row) * groups;
    float sum = 0.f;
    for (int gi = lane; gi < groups; gi += 32) {
        const uint4 q = ldg_stream(rw + gi);
        const float sc = e8m0_to_float(rs[gi]);
        const uint32_t qq[4] = {q.x, q.y, q.z, q.w};
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
#pragma unroll
            for (int j = 0; j < 8; j++) part = fmaf(e2m1_to_float(qq[i] >> (4 * j)), x[gi * 32 + i * 8 + j], part);
        }
        sum = fmaf(part, sc, sum);
    }
    sum = warp_sum(sum);
    if (lane == 0) y[row] = sum;
}

__global__ void get_row_kernel(const uint32_t *__restrict__ w, const uint8_t *__restrict__ s, float *__restrict__ out,
                               size_t row, int cols)
{
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= cols) return;
    const uint32_t word = w[row * (cols >> 3) + (k >> 3)];
    out[k] = e2m1_to_float(word >> ((k & 7) * 4)) * e8m0_to_float(s[row * (cols >> 5) + (k >> 5)]);
}

__global__ void embed_kernel(const uint32_t *__restrict__ w, const uint8_t *__restrict__ s, float *__restrict__ out,
                             const int *__restrict__ row_ptr, int rows, int cols)
{
    pdl_launch_dependents();
    pdl_wait();
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= cols) return;
    const int row = __ldcg(row_ptr);
    if (row < 0 || row >= rows) {
        out[k] = 0.f;
        return;
    }
    const uint32_t word = w[size_t(row) * (cols >> 3) + (k >> 3)];
    out[k] = e2m1_to_float(word >> ((k & 7) * 4)) * e8m0_to_float(s[size_t(row) * (cols >> 5) + (k >> 5)]);
}

__global__ void set_scalars_kernel(int *tok, int token, int *pos, int position)
{
    if (tok) *tok = token;
    if (pos) *pos = position;
}

__global__ void dequant_kernel(const uint32_t *__restrict__ w, const uint8_t *__restrict__ s, float *__restrict__ out,
                               size_t total_words, int cols)
{
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total_words) return;
    const uint32_t word = w[i];
    const float sc = e8m0_to_float(s[i >> 2]); // 4 words per group, rows are whole groups
    float4 a, b;
    a.x = e2m1_to_float(word) * sc; a.y = e2m1_to_float(word >> 4) * sc;
    a.z = e2m1_to_float(word >> 8) * sc; a.w = e2m1_to_float(word >> 12) * sc;
    b.x = e2m1_to_float(word >> 16) * sc; b.y = e2m1_to_float(word >> 20) * sc;
    b.z = e2m1_to_float(word >> 24) * sc; b.w = e2m1_to_float(word >> 28) * sc;
    reinterpret_cast<float4 *>(out)[i * 2] = a;
    reinterpret_cast<float4 *>(out)[i * 2 + 1] = b;
    (void)cols;
}

// ---- host side ------------------------------------------------------------------
namespace {
struct Tuning {
    int deq = 0;            // 0: cvt.e2m1x2, 1: shift/mask
    int unr = 4;            // kblocks per prefetch step
    int warps_per_sm = 16;  // warp slots per SM the decomposition is sized for
    int warps_per_cta = 16; // CTA size in warps (1 CTA per SM at 16)
} g_tune;

template <int DEQ, int UNR, int M>
int launch_variant(const GemvParams &p, int grid, int threads, size_t smem, cudaStream_t st, bool pdl)
{
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(gemv_fused_kernel<DEQ, UNR, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    });
    if (attr_err != cudaSuccess) return cuda_fail(attr_err, "cudaFuncSetAttribute(gemv)");
    return launch(gemv_fused_kernel<DEQ, UNR, M>, dim3(grid), dim3(threads), smem, st, pdl, p);
}

template <int M> int dispatch(const GemvParams &p, int grid, int threads, size_t smem, cudaStream_t st, bool pdl)
{
    const int deq = g_tune.deq, unr = g_tune.unr;
    if (deq == 0 && unr == 2) return launch_variant<0, 2, M>(p, grid, threads, smem, st, pdl);
    if (deq == 0 && unr == 4) return launch_variant<0, 4, M>(p, grid, threads, smem, st, pdl);
    if (deq == 1 && unr == 2) return launch_variant<1, 2, M>(p, grid, threads, smem, st, pdl);
    if (deq == 1 && unr == 4) return launch_variant<1, 4, M>(p, grid, threads, smem, st, pdl);
    return fail(INSG_E_ARG, "unsupported GEMV tuning");
}
} // namespace

int gemv_tune(const char *key, int value)
{
    const std::string k = key;
    if (k == "gemv_deq") g_tune.deq = value;
    else if (k == "gemv_unr") g_tune.unr = value;
    else if (k == "gemv_warps_per_sm") g_tune.warps_per_sm = std::max(1, std::min(value, 64));
    else if (k == "gemv_warps_per_cta") g_tune.warps_per_cta = std::max(1, std::min(value, 16));
    else return fail(INSG_E_ARG, "unknown tuning key");
    return INSG_OK;
}

int gemv_fused_launch(const insg_gemv_op *op, int M, cudaStream_t st)
{
    if (!op || !op->in) return fail(INSG_E_ARG, "gemv: null operand");
    if (op->cols <= 0 || (op->cols & 127) || op->cols > 16384) return fail(INSG_E_SHAPE, "gemv: cols must be a multiple of 128, <= 16384");
    if (op->n_segments < 1 || op->n_segments > 4) return fail(INSG_E_SHAPE, "gemv: 1..4 segments");
    if (M != 1 && M != 2 && M != 4) return fail(INSG_E_SHAPE, "gemv: 1, 2 or 4 tokens per launch");
    if ((op->prologue == INSG_PRO_RMSNORM || op->prologue == INSG_PRO_GATED_RMSNORM) && !op->norm_w)
        return fail(INSG_E_ARG, "gemv: norm weight missing");
    if (op->prologue >= INSG_PRO_GATED_RMSNORM && !op->aux) return fail(INSG_E_ARG, "gemv: prologue operand missing");
    if (op->prologue == INSG_PRO_GATED_RMSNORM && (op->cols & 1023)) return fail(INSG_E_SHAPE, "gemv: gated norm needs cols % 1024 == 0");
    GemvParams p = {};
    p.in = op->in; p.aux = op->aux; p.norm_w = op->norm_w; p.x_out = op->x_out;
    p.cols = op->cols; p.prologue = op->prologue; p.nseg = op->n_segments;
    int tiles = 0;
    bool logits = false;
    for (int i = 0; i < op->n_segments; i++) {
        const insg_gemv_segment &s = op->seg[i];
        if (!s.packed || !s.out || s.rows <= 0 || (s.rows & 15)) return fail(INSG_E_SHAPE, "gemv: segment rows must be a positive multiple of 16");
        if (s.epilogue == INSG_EPI_SWIGLU && !s.packed2) return fail(INSG_E_ARG, "gemv: SwiGLU needs two matrices");
        if (s.epilogue == INSG_EPI_CONV_SILU && (!s.conv_state || !s.conv_w)) return fail(INSG_E_ARG, "gemv: conv operands missing");
        if (s.epilogue == INSG_EPI_DECAY && (!s.A_log || !s.dt_bias)) return fail(INSG_E_ARG, "gemv: decay operands missing");
        if ((s.epilogue == INSG_EPI_SWIGLU || s.epilogue == INSG_EPI_LOGITS) && M != 1) return fail(INSG_E_SHAPE, "gemv: epilogue needs M == 1");
        SegDev &d = p.seg[i];
        d.packed = static_cast<const uint8_t *>(s.packed);
        d.packed2 = static_cast<const uint8_t *>(s.packed2);
        d.out = s.out; d.conv_state = s.conv_state; d.conv_w = s.conv_w; d.A_log = s.A_log; d.dt_bias = s.dt_bias;
        d.tile_begin = tiles; tiles += s.rows >> 4; d.tile_end = tiles; d.epilogue = s.epilogue; d.rows = s.rows;
        logits |= s.epilogue == INSG_EPI_LOGITS;
    }
    p.total_tiles = tiles;
    // split K over as many warps as it takes to occupy the machine once (1, 2, 3, 4 or 8 per tile)
    const int nkb = op->cols >> 7;
    const int sms = sm_count();
    const int slots = sms * g_tune.warps_per_sm;
    const int r = slots / tiles;
    int ksplit = r >= 8 ? 8 : r >= 4 ? 4 : r >= 3 ? 3 : r >= 2 ? 2 : 1;
    while (ksplit > 1 && ksplit > nkb) ksplit = ksplit == 3 ? 2 : ksplit / 2;
    const int gpc = std::max(1, g_tune.warps_per_cta / ksplit);
    const int ctas_per_sm = std::max(1, g_tune.warps_per_sm / (ksplit * gpc));
    const int grid = std::max(1, std::min((tiles + gpc - 1) / gpc, sms * ctas_per_sm));
    p.ksplit = ksplit;
    p.gpc = gpc;
    if (logits) {
        if (op->n_segments != 1) return fail(INSG_E_SHAPE, "gemv: the logits epilogue takes one segment");
        if (!op->argmax_scratch || !op->token_out) return fail(INSG_E_ARG, "gemv: arg-max scratch/token missing");
        if (grid > 4096) return fail(INSG_E_LIMIT, "gemv: arg-max scratch holds 4096 partials");
        p.ticket = static_cast<unsigned *>(op->argmax_scratch);
        p.argmax_partial = reinterpret_cast<float2 *>(static_cast<uint8_t *>(op->argmax_scratch) + 64);
        p.token_out = op->token_out;
        p.token_feedback = op->token_feedback;
        p.token_log = op->token_log;
        p.position_inout = op->position_inout;
    }
    const size_t smem = size_t(M) * 2 * (op->cols + 8) * sizeof(__half) + size_t(gpc) * 2 * ksplit * M * 16 * 4 + 64 * 4;
    const int threads = 32 * ksplit * gpc;
    const bool pdl = op->pdl != 0;
    switch (M) {
    case 1: return dispatch<1>(p, grid, threads, smem, st, pdl);
    case 2: return dispatch<2>(p, grid, threads, smem, st, pdl);
    default: return dispatch<4>(p, grid, threads, smem, st, pdl);
    }
}

} // namespace insg

using namespace insg;

extern "C" {

size_t insg_gemv_argmax_scratch_bytes(void) { return 64 + size_t(8) * 4096; }

int insg_gemv_fused(const insg_gemv_op *op, insg_stream_t stream) { return gemv_fused_launch(op, 1, stream); }

size_t insg_mxfp4_packed_bytes(int rows, int cols)
{
    if (rows <= 0 || cols <= 0 || (rows & 15) || (cols & 127)) return 0;
    return size_t(rows >> 4) * (cols >> 7) * kRec;
}

int insg_mxfp4_repack(const uint32_t *weight, const uint8_t *scales, void *packed, int rows, int cols, insg_stream_t stream)
{
    if (!weight || !scales || !packed) return fail(INSG_E_ARG, "repack: null pointer");
    if (rows <= 0 || cols <= 0 || (rows & 15) || (cols & 127)) return fail(INSG_E_SHAPE, "repack: rows % 16 and cols % 128 must be 0");
    const size_t nrec = size_t(rows >> 4) * (cols >> 7);
    const unsigned blocks = unsigned((nrec + 7) / 8);
    repack_kernel<<<blocks, 256, 0, stream>>>(weight, scales, static_cast<uint8_t *>(packed), rows, cols);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? INSG_OK : cuda_fail(e, "repack launch");
}

int insg_mxfp4_gemv_packed(const void *packed, const float *x, float *y, int rows, int cols, int M, insg_stream_t stream)
{
    if (M < 1 || M > 8) return fail(INSG_E_SHAPE, "gemv_packed: 1 <= M <= 8");
    for (int m0 = 0; m0 < M;) {
        const int left = M - m0;
        const int mm = left >= 4 ? 4 : (left >= 2 ? 2 : 1);
        insg_gemv_op op = {};
        op.in = x + size_t(m0) * cols;
        op.cols = cols;
        op.prologue = INSG_PRO_PLAIN;
        op.n_segments = 1;
        op.seg[0].packed = packed;
        op.seg[0].out = y + size_t(m0) * rows;
        op.seg[0].rows = rows;
        op.seg[0].epilogue = INSG_EPI_STORE;
        const int rc = gemv_fused_launch(&op, mm, stream);
        if (rc) return rc;
        m0 += mm;
    }
    return INSG_OK;
}

int insg_mxfp4_gemv_mlx(const uint32_t *weight, const uint8_t *scales, const float *x, float *y, int rows, int cols,
                        insg_stream_t stream)
{
    if (rows <= 0 || cols <= 0 || (cols & 31)) return fail(INSG_E_SHAPE, "gemv_mlx: cols must be a positive multiple of 32");
    if (!weight || !scales || !x || !y) return fail(INSG_E_ARG, "gemv_mlx: null pointer");
    gemv_mlx_kernel<<<(rows + 7) / 8, 256, 0, stream>>>(weight, scales, x, y, rows, cols);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? INSG_OK : cuda_fail(e, "gemv_mlx launch");
}

int insg_mxfp4_get_row_mlx(const uint32_t *weight, const uint8_t *scales, float *out, int row, int cols, insg_stream_t stream)
{
    if (row < 0 || cols <= 0 || (cols & 31)) return fail(INSG_E_SHAPE, "get_row: bad row/cols");
    if (!weight || !scales || !out) return fail(INSG_E_ARG, "get_row: null pointer");
    get_row_kernel<<<(cols + 255) / 256, 256, 0, stream>>>(weight, scales, out, size_t(row), cols);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? INSG_OK : cuda_fail(e, "get_row launch");
}

int insg_mxfp4_embed(const uint32_t *weight, const uint8_t *scales, float *out, const int *device_row, int rows, int cols,
                     int pdl, insg_stream_t stream)
{
    if (!weight || !scales || !out || !device_row) return fail(INSG_E_ARG, "embed: null pointer");
    if (rows <= 0 || cols <= 0 || (cols & 31)) return fail(INSG_E_SHAPE, "embed: bad rows/cols");
    return launch(embed_kernel, dim3((cols + 255) / 256), dim3(256), 0, stream, pdl != 0, weight, scales, out, device_row, rows, cols);
}

int insg_set_scalars(int *device_token, int token, int *device_position, int position, insg_stream_t stream)
{
    set_scalars_kernel<<<1, 1, 0, stream>>>(device_token, token, device_position, position);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? INSG_OK : cuda_fail(e, "set_scalars launch");
}

int insg_mxfp4_dequant_mlx(const uint32_t *weight, const uint8_t *scales, float *out, int rows, int cols, insg_stream_t stream)
{
    if (rows <= 0 || cols <= 0 || (cols & 31)) return fail(INSG_E_SHAPE, "dequant: cols must be a positive multiple of 32");
    if (!weight || !scales || !out) return fail(INSG_E_ARG, "dequant: null pointer");
    const size_t words = size_t(rows) * (cols >> 3);
    dequant_kernel<<<unsigned((words + 255) / 256), 256, 0, stream>>>(weight, scales, out, words, cols);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? INSG_OK : cuda_fail(e, "dequant launch");
}

} // extern "C"
