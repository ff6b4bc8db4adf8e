// Device-side body of the fused MXFP4 weight-streaming GEMV, shared by the stand-alone kernel (gemv_fused.cu) and by
// the persistent token kernel (persistent.cu), which runs the same stages as phases of one launch.
//
// Contraction (reference: src/mxfp4.cu:41-66): y[r] = sum_k lut[code(r,k)] * 2^(s(r,k/32)-127) * x[k].
//
// Stages, in the order a launch (or a phase) runs them:
//   gemv_range        this CTA's share of the record sequence (whole output tiles) and this warp's part of it
//   gemv_issue_first  the first two chunks of weight records into registers (no dependency on activations)
//   gemv_activation   the fused prologue: fp32 vector (or a prepared fp16 image) -> two fp16 pieces in shared memory
//   gemv_stream       the record loop: E2M1 -> fp16 by cvt, multiply-adds on mma.sync, partial sums parked per run
//   gemv_finish       after one CTA barrier: runs summed over the warps in warp order, epilogues, arg-max
#pragma once
#include "common.cuh"
#include "gemv_prologue.cuh"

namespace insg {

constexpr int kRec = 1088;  // bytes per (16-row tile, 128-k block) record
constexpr int kWarps = 16;  // warps per CTA, one CTA per SM
constexpr int kThreads = kWarps * 32;
constexpr float kLoScale = 1.0f / 2048.0f;
constexpr int kMaxGrid = 296;
constexpr int kUnr = 3;     // records per register prefetch chunk (2 / 3 / 4 measured 580 / 584 / 569 tokens/s in the engine)
// Fixed pre-scale of a prepared activation image: the producer cannot know the vector's maximum, so instead of the
// adaptive power of two of the in-kernel prologue the image holds x / 16.  fp16 then covers |x| from 1e-3 (below that
// the low piece loses bits that are far under the fp32 rounding of a 4096-term dot product) to 1e6 (saturating).
constexpr float kPrepScale = 0.0625f, kPrepInv = 16.0f;

struct SegDev {
    const uint8_t *packed, *packed2;
    float *out;
    float *conv_state;
    const uint16_t *conv_w;
    const float *A_log;
    const uint16_t *dt_bias;
    int tm_begin; // first (tile, matrix) index of the segment
    int nmat;     // 1, or 2 for the gate/up pair of SwiGLU
    int epilogue, rows;
    __half *prep;            // optional fp16 image [2][rows] of out * prep_w / 16 for a later INSG_PRO_PREPARED launch
    const uint16_t *prep_w;  // bf16 [rows] or null
    long long conv_stride;   // CONV_SILU with several tokens: 0 = one sequence (history carried through the tokens in order),
                             // else the tokens are independent sequences and token m's history is conv_state + m * conv_stride
};

struct GemvParams {
    const float *in, *aux;
    const uint16_t *norm_w;
    float *x_out;
    int cols, nkb, prologue, nseg;
    int total_units, total_tm, slots; // records in the launch, (tile, matrix) runs, shared slots per warp
    int total_etiles, etile_units;    // output tiles (a run, or a gate/up pair of runs) and records per tile
    SegDev seg[4];
    float2 *argmax_partial; // [grid] (value, index as int bits)
    unsigned *argmax_ticket;
    int *token_out, *token_feedback, *token_log, *position_inout;
    int token_log_capacity;        // entries of token_log; positions beyond it are not logged
    const float *prep_partials_in; // INSG_PRO_PREPARED: [kMaxGrid] per-CTA sums of squares of the producer, or null
    int prep_rms;                  // INSG_PRO_PREPARED: scale by rsqrt(mean square + 1e-6) (the RMSNorm case)
    float *prep_partials_out;      // RESIDUAL with prep: [kMaxGrid], this launch's per-CTA sums of out^2
};

// Small shared state of the body (the large buffers are carved from dynamic shared memory by the caller).
struct GemvShared {
    int wa[kWarps + 1], tmf[kWarps]; // warp boundaries in the record sequence, first run of each warp
    int last;
};

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void dequant8(uint32_t q, uint32_t (&h)[4])
{
    // register b holds elements (2b, 2b+1) of the 8-nibble word at their true value
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
}

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Position in the linear record sequence.
struct UnitIt {
    int u;   // record index in the launch
    int tm;  // (tile, matrix) run
    int kb;  // k-block inside the run
    const uint8_t *ptr;
};

__device__ __forceinline__ int seg_of(const GemvParams &p, int tm)
{
    int s = 0;
#pragma unroll
    for (int i = 1; i < 4; i++)
        if (i < p.nseg && tm >= p.seg[i].tm_begin) s = i;
    return s;
}

__device__ __forceinline__ const uint8_t *run_base(const GemvParams &p, int tm)
{
    const SegDev &s = p.seg[seg_of(p, tm)];
    const int local = tm - s.tm_begin;
    if (s.nmat == 2) return ((local & 1) ? s.packed2 : s.packed) + size_t(local >> 1) * p.nkb * kRec;
    return s.packed + size_t(local) * p.nkb * kRec;
}

__device__ __forceinline__ void it_set(const GemvParams &p, UnitIt &it, int u)
{
    it.u = u;
    it.tm = u / p.nkb;
    it.kb = u - it.tm * p.nkb;
    it.ptr = u < p.total_units ? run_base(p, it.tm) + size_t(it.kb) * kRec : nullptr;
}

// nkb and total_units are p's, passed by value: the record loop then keeps them in registers wherever p itself lives.
__device__ __forceinline__ void it_next(const GemvParams &p, UnitIt &it, int nkb, int total_units)
{
    it.u++;
    it.kb++;
    it.ptr += kRec;
    if (it.kb == nkb) {
        it.kb = 0;
        it.tm++;
        it.ptr = it.u < total_units ? run_base(p, it.tm) : nullptr;
    }
}

template <int UNR> struct Chunk {
    uint4 wa[UNR], wb[UNR];
    uint32_t sc[UNR];
};

// Issues the loads of the next UNR records (those below `end`) and advances the iterator past them.
template <int UNR>
__device__ __forceinline__ void load_chunk(const GemvParams &p, Chunk<UNR> &b, UnitIt &it, int end, int lane, int nkb, int total_units)
{
#pragma unroll
    for (int j = 0; j < UNR; j++) {
        if (it.u < end) {
            b.wa[j] = ldg_stream(it.ptr + lane * 16);
            b.wb[j] = ldg_stream(it.ptr + 512 + lane * 16);
            b.sc[j] = ldg_stream_u16(it.ptr + 1024 + lane * 2);
            it_next(p, it, nkb, total_units);
        } else {
            b.wa[j] = make_uint4(0, 0, 0, 0);
            b.wb[j] = make_uint4(0, 0, 0, 0);
            b.sc[j] = 0;
        }
    }
}

// This CTA's share [a, b) of the record sequence and this warp's part [ua, ub) of it.
struct GemvRange {
    int a, b, ua, ub, tm_first;
};

// CTA ranges end on tile boundaries (a tile = one run, or the gate/up pair): no tile is shared between CTAs.  The CTAs
// that get one tile more are the lowest-numbered ones: those are placed first, on the SMs the previous kernel left
// first, so the extra tile goes where the head start is (and the stragglers' SMs get the short ranges).
__device__ __forceinline__ GemvRange gemv_range(const GemvParams &p, int G, int c, int warp)
{
    GemvRange r;
    const int tq = p.total_etiles / G, tr = p.total_etiles % G;
    r.a = (c * tq + min(c, tr)) * p.etile_units;
    r.b = ((c + 1) * tq + min(c + 1, tr)) * p.etile_units;
    r.ua = r.a + (((r.b - r.a) * warp) >> 4); // kWarps == 16
    r.ub = r.a + (((r.b - r.a) * (warp + 1)) >> 4);
    r.tm_first = r.ua / p.nkb;
    return r;
}

template <int UNR>
__device__ __forceinline__ void gemv_issue_first(const GemvParams &p, const GemvRange &r, Chunk<UNR> &A, Chunk<UNR> &B, UnitIt &lit, int lane)
{
    const int nkb = p.nkb, total_units = p.total_units;
    it_set(p, lit, r.ua);
    load_chunk<UNR>(p, A, lit, r.ub, lane, nkb, total_units);
    load_chunk<UNR>(p, B, lit, r.ub, lane, nkb, total_units);
}

__device__ __forceinline__ void gemv_publish_range(const GemvRange &r, GemvShared &sh, int lane, int warp)
{
    if (lane == 0) {
        sh.wa[warp] = r.ua;
        sh.tmf[warp] = r.tm_first;
        if (warp == kWarps - 1) sh.wa[kWarps] = r.ub;
    }
}

// ---- activation prologue: fp32 vector -> two fp16 pieces in shared memory ----
// Returns 1/alpha, which undoes the power-of-two pre-scale.
__device__ __forceinline__ float prologue(const GemvParams &p, const ProIn &pin, int m, __half *xs, int xstride, const uint2 (&wpre)[kPreVec],
                                          float *scratch)
{
    float4 v[kMaxVec];
    load_activation(pin, m, v);
    const float tmax = transform_activation(pin, m, v, wpre, scratch);
    const int tid = threadIdx.x, nvec = p.cols >> 2;
    // alpha = 2^(12 - floor(log2(max))) puts the largest element in [2^12, 2^13): fp16 holds it with room to spare
    int eb = int((__float_as_uint(tmax) >> 23) & 0xffu);
    eb = min(max(eb, 20), 240);
    const float alpha = __uint_as_float(uint32_t(266 - eb) << 23);
    __half *hi = xs + size_t(m * 2) * xstride, *lo = hi + xstride;
#pragma unroll
    for (int j = 0; j < kMaxVec; j++) {
        const int i = tid + j * kThreads;
        if (i < nvec) {
            const float e[4] = {v[j].x * alpha, v[j].y * alpha, v[j].z * alpha, v[j].w * alpha};
            __half h[4], l[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                h[q] = __float2half_rn(e[q]);
                l[q] = __float2half_rn((e[q] - __half2float(h[q])) * 2048.0f);
            }
            *reinterpret_cast<uint2 *>(hi + (i << 2)) = *reinterpret_cast<const uint2 *>(h);
            *reinterpret_cast<uint2 *>(lo + (i << 2)) = *reinterpret_cast<const uint2 *>(l);
        }
    }
    return __uint_as_float(uint32_t(eb - 12) << 23);
}

// The whole activation stage for M tokens; ends with a CTA barrier (the pieces are then visible to every warp).
template <int M>
__device__ __forceinline__ void gemv_activation(const GemvParams &p, __half *xs, int xstride, float *scratch, uint2 (&wpre)[kPreVec],
                                                float (&inv_alpha)[M])
{
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (p.prologue == INSG_PRO_PREPARED) {
        // The producer left both fp16 pieces ready: copy them (16-byte asynchronous copies through L2, no registers,
        // no reductions) and fold the RMS factor, when there is one, into the output scale.
        const int n16 = p.cols >> 3; // 16-byte chunks per piece
        const uint4 *src = reinterpret_cast<const uint4 *>(p.in);
        for (int i = tid; i < 2 * n16; i += kThreads) {
            const int piece = i >= n16, k = i - piece * n16;
            const uint32_t dst = smem_addr(xs + size_t(piece) * xstride + k * 8);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src + i) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (warp == 0) {
            float f = 1.0f, ok = 1.0f;
            if (p.prep_partials_in) {
                float a = 0.f;
#pragma unroll
                for (int j = 0; j < (kMaxGrid + 31) / 32; j++)
                    if (lane + 32 * j < kMaxGrid) a += __ldcg(p.prep_partials_in + lane + 32 * j);
                a = warp_sum(a);
                const float ms = a / float(p.cols);
                if (p.prep_rms) f = rsqrtf(ms + 1e-6f);
                // The image has a fixed scale: it is exact enough for a root mean square between 1e-3 and 1e5 and
                // when no element saturated (the producer then left an infinite sum).  Outside that, use the fp32 vector.
                ok = (ms >= 1e-6f && ms <= 1e10f) ? 1.0f : 0.0f;
            }
            if (lane == 0) { scratch[0] = f * kPrepInv; scratch[1] = ok; }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (scratch[1] == 0.0f && p.aux) { // CTA-uniform and the same in every CTA: it depends on global sums only
            const ProIn q{p.aux, nullptr, p.norm_w, p.x_out, p.cols, p.norm_w ? INSG_PRO_RMSNORM : INSG_PRO_PLAIN};
            preload_norm_weights(q, wpre);
            __syncthreads(); // every thread has read scratch[1]
#pragma unroll
            for (int m = 0; m < M; m++) inv_alpha[m] = prologue(p, q, m, xs, xstride, wpre, scratch);
        } else {
#pragma unroll
            for (int m = 0; m < M; m++) inv_alpha[m] = scratch[0];
        }
    } else {
        const ProIn pin{p.in, p.aux, p.norm_w, p.x_out, p.cols, p.prologue};
#pragma unroll
        for (int m = 0; m < M; m++) inv_alpha[m] = prologue(p, pin, m, xs, xstride, wpre, scratch);
    }
    __syncthreads();
}

// The two fp16 pieces of v * w / 16 (see kPrepScale) into a prepared image of `rows` elements.
// Returns false when the value does not fit (the consumer is then told, through an infinite sum of squares, to read the
// fp32 vector instead).
__device__ __forceinline__ bool prep_store(const SegDev &s, int row, float v)
{
    const float w = s.prep_w ? bf16_bits_to_float(s.prep_w[row]) : 1.0f;
    const float raw = v * w * kPrepScale;
    const float e = fminf(fmaxf(raw, -65504.0f), 65504.0f);
    const __half hi = __float2half_rn(e);
    s.prep[row] = hi;
    s.prep[s.rows + row] = __float2half_rn((e - __half2float(hi)) * 2048.0f);
    return fabsf(raw) <= 65504.0f; // false for NaN too
}

// One output row of one token through the epilogue of its segment.
__device__ __forceinline__ void row_epilogue(const SegDev &s, int row, int m, float y0, float y1, float &best, int &best_idx, float &ss)
{
    float *out = s.out + size_t(m) * s.rows;
    switch (s.epilogue) {
    case INSG_EPI_STORE: out[row] = y0; break;
    case INSG_EPI_RESIDUAL: {
        const float h = __ldcg(out + row) + y0;
        out[row] = h;
        if (s.prep) ss = prep_store(s, row, h) ? fmaf(h, h, ss) : __int_as_float(0x7f800000);
        break;
    }
    case INSG_EPI_CONV_SILU: {
        float *st = s.conv_state + size_t(m) * s.conv_stride + size_t(row) * 3;
        const uint2 wv = reinterpret_cast<const uint2 *>(s.conv_w)[row];
        const float w0 = bf16_bits_to_float(wv.x & 0xffff), w1 = bf16_bits_to_float(wv.x >> 16);
        const float w2 = bf16_bits_to_float(wv.y & 0xffff), w3 = bf16_bits_to_float(wv.y >> 16);
        const float s0 = __ldcg(st), s1 = __ldcg(st + 1), s2 = __ldcg(st + 2);
        const float z = fmaf(s0, w0, fmaf(s1, w1, fmaf(s2, w2, y0 * w3)));
        st[0] = s1; st[1] = s2; st[2] = y0;
        out[row] = fast_silu(z);
        break;
    }
    case INSG_EPI_BETA: out[row] = fast_sigmoid(y0); break;
    case INSG_EPI_DECAY: {
        const float z = y0 + bf16_bits_to_float(s.dt_bias[row]);
        const float soft = z > 20.f ? z : log1pf(__expf(z));
        out[row] = -__expf(s.A_log[row]) * soft;
        break;
    }
    case INSG_EPI_SWIGLU: {
        const float act = fast_silu(y0) * y1;
        out[row] = act;
        if (s.prep) ss = prep_store(s, row, act) ? fmaf(act, act, ss) : __int_as_float(0x7f800000);
        break;
    }
    case INSG_EPI_LOGITS:
        out[row] = y0;
        if (y0 > best || (y0 == best && row < best_idx)) { best = y0; best_idx = row; }
        break;
    default: break;
    }
}

// The record loop of one warp over [r.ua, r.ub).  A and B hold the first two chunks (gemv_issue_first); `lit` is the
// load iterator past them.  `wrec` is this warp's slot array [slots][M][16].
template <int UNR, int M>
__device__ __forceinline__ void gemv_stream(const GemvParams &p, const GemvRange &r, Chunk<UNR> &A, Chunk<UNR> &B, UnitIt &lit,
                                            const __half *xs, int xstride, float *wrec, const float (&inv_alpha)[M], int lane)
{
    const int g = lane >> 2, t = lane & 3;
    const int nkb = p.nkb, total_units = p.total_units, ub = r.ub, tm_first = r.tm_first;
    const bool bactive = (t == (g >> 1));
    const int piece = g & 1;
    float acc[M][4];
#pragma unroll
    for (int m = 0; m < M; m++) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;

    // consume one chunk: multiply its records, closing a (tile, matrix) run whenever one ends
    UnitIt cit;
    it_set(p, cit, r.ua);
    auto compute = [&](const Chunk<UNR> &ch) {
#pragma unroll
        for (int j = 0; j < UNR; j++) {
            if (cit.u >= ub) break; // warp-uniform
            float cc[M][4];
#pragma unroll
            for (int m = 0; m < M; m++) cc[m][0] = cc[m][1] = cc[m][2] = cc[m][3] = 0.f;
            const uint32_t wa[4] = {ch.wa[j].x, ch.wa[j].y, ch.wa[j].z, ch.wa[j].w};
            const uint32_t wb[4] = {ch.wb[j].x, ch.wb[j].y, ch.wb[j].z, ch.wb[j].w};
            const int xoff = cit.kb * 128 + t * 32;
#pragma unroll
            for (int w = 0; w < 4; w++) {
                uint32_t ha[4], hb[4];
                dequant8(wa[w], ha);
                dequant8(wb[w], hb);
#pragma unroll
                for (int m = 0; m < M; m++) {
                    uint4 xv = make_uint4(0, 0, 0, 0);
                    if (bactive) xv = *reinterpret_cast<const uint4 *>(xs + size_t(m * 2 + piece) * xstride + xoff + w * 8);
                    mma16816(cc[m], ha[0], hb[0], ha[1], hb[1], xv.x, xv.y);
                    mma16816(cc[m], ha[2], hb[2], ha[3], hb[3], xv.z, xv.w);
                }
            }
            const float s0 = e8m0_to_float(ch.sc[j] & 0xffu), s1 = e8m0_to_float(ch.sc[j] >> 8);
#pragma unroll
            for (int m = 0; m < M; m++) {
                acc[m][0] = fmaf(cc[m][0], s0, acc[m][0]);
                acc[m][1] = fmaf(cc[m][1], s0, acc[m][1]);
                acc[m][2] = fmaf(cc[m][2], s1, acc[m][2]);
                acc[m][3] = fmaf(cc[m][3], s1, acc[m][3]);
            }
            if (cit.kb == nkb - 1 || cit.u == ub - 1) {
                // fold hi/lo, sum the quad (4 scale groups), gather rows 0..15 into lanes 0..15, park in this run's slot
                float *slot = wrec + size_t(cit.tm - tm_first) * M * 16;
#pragma unroll
                for (int m = 0; m < M; m++) {
                    float v0 = fmaf(acc[m][1], kLoScale, acc[m][0]);
                    float v1 = fmaf(acc[m][3], kLoScale, acc[m][2]);
                    v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
                    v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
                    v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
                    v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
                    const float r0 = __shfl_sync(0xffffffffu, v0, (lane & 7) * 4);
                    const float r1 = __shfl_sync(0xffffffffu, v1, (lane & 7) * 4);
                    if (lane < 16) slot[m * 16 + lane] = ((lane & 8) ? r1 : r0) * inv_alpha[m];
                    acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
                }
            }
            it_next(p, cit, nkb, total_units);
        }
    };

    while (cit.u < ub) {
        compute(A);
        load_chunk<UNR>(p, A, lit, ub, lane, nkb, total_units);
        if (cit.u >= ub) break;
        compute(B);
        load_chunk<UNR>(p, B, lit, ub, lane, nkb, total_units);
    }
}

// Everything after the CTA barrier that follows the record loop: every tile this CTA touched has its runs summed over
// the warps in warp order and goes through its epilogue; then the per-CTA sum of squares (prepared output) and the
// arg-max (lm_head).  `G` CTAs take part, this one is `c`.
template <int M>
__device__ __forceinline__ void gemv_finish(const GemvParams &p, const GemvRange &r, int G, int c, const float *rec, float *scratch,
                                            GemvShared &sh)
{
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nkb = p.nkb, a = r.a, b = r.b;
    float best = -3.402823466e38f;
    int best_idx = 0x7fffffff;
    float ss = 0.f; // sum of squares of the residual-stream rows this thread produced (prepared output only)
    if (b > a) {
        const int tm_lo = a / nkb, tm_hi = (b - 1) / nkb;
        const int row = lane & 15;
        // warp boundaries into registers once: the sums below then issue their shared-memory reads together
        int wr[kWarps + 1], tf[kWarps];
#pragma unroll
        for (int w = 0; w < kWarps; w++) { wr[w] = sh.wa[w]; tf[w] = sh.tmf[w]; }
        wr[kWarps] = sh.wa[kWarps];
        // tasks are tiles: a run for plain segments, the (gate, up) pair of runs for SwiGLU
        for (int tmq = tm_lo + warp; tmq <= tm_hi; tmq += kWarps) {
            const SegDev &s = p.seg[seg_of(p, tmq)];
            const int local = tmq - s.tm_begin;
            if (s.nmat == 2 && (local & 1)) continue; // the pair is handled from its gate run
            const int tm0 = tmq - (s.nmat == 2 ? (local & 1) : 0);
            // Tokens are independent except for the convolution, whose history is carried from one token to the next:
            // there the 16 row lanes walk the tokens in order, elsewhere the two half-warps take alternate tokens.
            const bool serial = M > 1 && s.epilogue == INSG_EPI_CONV_SILU && s.conv_stride == 0;
            for (int m = serial ? (lane < 16 ? 0 : M) : lane >> 4; m < M; m += serial ? 1 : 2) {
                float y[2] = {0.f, 0.f};
                for (int mat = 0; mat < s.nmat; mat++) {
                    const int tm = tm0 + mat, lo = max(tm * nkb, a), hi = min((tm + 1) * nkb, b);
                    float part[kWarps];
#pragma unroll
                    for (int w = 0; w < kWarps; w++) {
                        const bool on = hi > lo && wr[w + 1] > wr[w] && wr[w] < hi && wr[w + 1] > lo;
                        part[w] = on ? rec[((w * p.slots + (tm - tf[w])) * M + m) * 16 + row] : 0.f;
                    }
                    float z = 0.f;
#pragma unroll
                    for (int w = 0; w < kWarps; w++) z += part[w]; // warp order, whatever the schedule
                    y[mat] = z;
                }
                row_epilogue(s, (tm0 - s.tm_begin) / s.nmat * 16 + row, m, y[0], y[1], best, best_idx, ss);
            }
        }
    }

    // ---- this CTA's share of sum(out^2), for the RMSNorm of the launch that consumes the prepared image ----
    if (p.prep_partials_out && c < G) {
        ss = warp_sum(ss);
        __syncthreads(); // scratch[0] was the prologue's
        if (lane == 0) scratch[warp] = ss;
        __syncthreads();
        if (tid == 0) {
            float tot = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; w++) tot += scratch[w];
            p.prep_partials_out[c] = tot;
        }
        if (c == 0)
            for (int i = G + tid; i < kMaxGrid; i += kThreads) p.prep_partials_out[i] = 0.f;
    }
    // ---- arg-max over the rows this launch produced (lm_head) ----------------
    if (p.argmax_partial && c < G) { // CTA-uniform (a persistent grid may be larger than the G CTAs that take part)
        float *sv = scratch + 16;
        int *si = reinterpret_cast<int *>(scratch + 32);
#pragma unroll
        for (int mk = 16; mk; mk >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, mk);
            const int oi = __shfl_xor_sync(0xffffffffu, best_idx, mk);
            if (ov > best || (ov == best && oi < best_idx)) { best = ov; best_idx = oi; }
        }
        if (lane == 0) { sv[warp] = best; si[warp] = best_idx; }
        __syncthreads();
        if (tid == 0) {
            float bv = sv[0];
            int bi = si[0];
            for (int w = 1; w < kWarps; w++)
                if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
            p.argmax_partial[c] = make_float2(bv, __int_as_float(bi));
            __threadfence();
            const unsigned ticket = atomicAdd(p.argmax_ticket, 1u);
            sh.last = (ticket == unsigned(G) - 1u);
        }
        __syncthreads();
        if (sh.last) {
            __threadfence();
            float bv = -3.402823466e38f;
            int bi = 0x7fffffff;
            for (int i = tid; i < G; i += kThreads) {
                const float ev = __ldcg(reinterpret_cast<const float *>(p.argmax_partial + i));
                const int idx = __float_as_int(__ldcg(reinterpret_cast<const float *>(p.argmax_partial + i) + 1));
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
                for (int w = 1; w < kWarps; w++)
                    if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
                *p.token_out = bi;
                if (p.token_feedback) *p.token_feedback = bi;
                if (p.position_inout) {
                    // read past L1: inside a persistent launch another CTA wrote the position one token earlier
                    const int pos = __ldcg(p.position_inout);
                    if (p.token_log && pos >= 0 && pos < p.token_log_capacity) p.token_log[pos] = bi;
                    *p.position_inout = pos + 1;
                }
                *p.argmax_ticket = 0u;
            }
        }
    }
}

// Dynamic shared memory of the body: the activation pieces, the per-warp slots, 64 floats of scratch.
__host__ __device__ inline size_t gemv_smem_bytes(int M, int cols, int slots)
{
    return size_t(M) * 2 * (cols + 8) * sizeof(__half) + size_t(kWarps) * slots * M * 16 * 4 + 64 * 4;
}

} // namespace insg
