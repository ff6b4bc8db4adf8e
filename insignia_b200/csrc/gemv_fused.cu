// Fused MXFP4 weight-streaming GEMV for sm_100a (batch-1 decode, up to 4 tokens per launch).
//
// Contraction (reference: src/mxfp4.cu:41-66): y[r] = sum_k lut[code(r,k)] * 2^(s(r,k/32)-127) * x[k].
//
// The path is HBM-bound: 17 bytes arrive per 32 weights, so the kernel is built around the byte
// stream, not around the arithmetic:
//   * weights come from the tile-interleaved copy made by insg_mxfp4_repack: one (16 rows x 128 k)
//     record is 1088 contiguous bytes, read by a warp with two coalesced 512-byte loads + 64 scale
//     bytes (ld.global.nc, no L1 allocation); every warp keeps two chunks of UNR records in flight,
//     both issued BEFORE the programmatic-dependent-launch wait so they overlap the previous kernel;
//   * the launch's records form one linear sequence (segment, tile, matrix, k-block).  Output tiles
//     are dealt evenly to the CTAs (one per SM, whole tiles only, so no CTA ever waits for another)
//     and a CTA's records are then divided evenly over its 16 warps, so every warp of a CTA streams
//     the same number of bytes whatever the matrix shape.  A warp folds each (tile, matrix) run it
//     finishes into a shared-memory slot; after one CTA barrier the slots are summed in warp order,
//     so the result does not depend on scheduling (a ticketed split of tiles across CTAs was
//     measured: its fence + atomic + re-read chain cost ~2.5 us per launch, more than the <=15 %
//     imbalance of whole tiles);
//   * E2M1 nibbles become fp16 pairs with cvt.rn.f16x2.e2m1x2 (exact); the multiply-adds run on
//     mma.sync.m16n8k16 (fp16 in, fp32 accumulate) purely as a cheap FMA engine.  The fp32 activation
//     is split into two fp16 pieces (hi + lo * 2^-11 after an exact power-of-two pre-scale) so the
//     products keep ~22 bits of x; the 8 columns of the MMA's B operand hold (4 scale groups) x
//     (hi, lo): thread t of a quad owns scale group t of the 128-wide k-block, so accumulator
//     columns separate the groups and the E8M0 scale is applied once per (row, group) in fp32;
//   * the elementwise kernels around the GEMV are fused in: RMSNorm / gated RMSNorm / sigmoid-gate
//     prologues on the activation, residual / conv+SiLU / decay / beta / SwiGLU / logits+arg-max
//     epilogues on the rows.
#include "common.cuh"
#include "gemv_prologue.cuh"
#include "host_util.h"

#include <algorithm>
#include <mutex>

namespace insg {

constexpr int kRec = 1088;  // bytes per (16-row tile, 128-k block) record
constexpr int kWarps = 16;  // warps per CTA, one CTA per SM
constexpr int kThreads = kWarps * 32;
constexpr float kLoScale = 1.0f / 2048.0f;
constexpr int kMaxGrid = 296;
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
    unsigned long long *trace; // optional [grid][8] phase timestamps (ns), or null
    int *error_flag;           // RING: raised when a bounded wait expires
    const float *prep_partials_in; // INSG_PRO_PREPARED: [kMaxGrid] per-CTA sums of squares of the producer, or null
    int prep_rms;                  // INSG_PRO_PREPARED: scale by rsqrt(mean square + 1e-6) (the RMSNorm case)
    float *prep_partials_out;      // RESIDUAL with prep: [kMaxGrid], this launch's per-CTA sums of out^2
};

__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define INSG_TRACE(slot)                                                   \
    do {                                                                   \
        if (p.trace && threadIdx.x == 0) p.trace[blockIdx.x * 8 + (slot)] = global_ns(); \
    } while (0)

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

__device__ __forceinline__ void it_next(const GemvParams &p, UnitIt &it)
{
    it.u++;
    it.kb++;
    it.ptr += kRec;
    if (it.kb == p.nkb) {
        it.kb = 0;
        it.tm++;
        it.ptr = it.u < p.total_units ? run_base(p, it.tm) : nullptr;
    }
}

template <int UNR> struct Chunk {
    uint4 wa[UNR], wb[UNR];
    uint32_t sc[UNR];
};

// Issues the loads of the next UNR records (those below `end`) and advances the iterator past them.
template <int UNR> __device__ __forceinline__ void load_chunk(const GemvParams &p, Chunk<UNR> &b, UnitIt &it, int end, int lane)
{
#pragma unroll
    for (int j = 0; j < UNR; j++) {
        if (it.u < end) {
            b.wa[j] = ldg_stream(it.ptr + lane * 16);
            b.wb[j] = ldg_stream(it.ptr + 512 + lane * 16);
            b.sc[j] = ldg_stream_u16(it.ptr + 1024 + lane * 2);
            it_next(p, it);
        } else {
            b.wa[j] = make_uint4(0, 0, 0, 0);
            b.wb[j] = make_uint4(0, 0, 0, 0);
            b.sc[j] = 0;
        }
    }
}

// ---- shared-memory ring helpers (RING variant) ----------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void ring_bar_init(uint64_t *b) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(b))); }
// one record HBM -> shared memory; the stage's mbarrier completes when all 1088 bytes have landed
__device__ __forceinline__ void ring_issue(void *dst, const void *src, uint64_t *bar)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(kRec) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(dst)), "l"(src), "r"(kRec), "r"(smem_addr(bar)) : "memory");
}
// bounded wait; false (and the CTA-wide abort flag raised) if the data never arrives
__device__ __forceinline__ bool ring_wait(uint64_t *bar, uint32_t parity, int *abort_flag)
{
    for (uint32_t it = 0; it < (1u << 22); it++) {
        uint32_t done;
        asm volatile("{\n.reg .pred q;\nmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\nselp.u32 %0, 1, 0, q;\n}"
                     : "=r"(done) : "r"(smem_addr(bar)), "r"(parity) : "memory");
        if (done) return true;
    }
    *abort_flag = 1;
    return false;
}

// ---- activation prologue: fp32 vector -> two fp16 pieces in shared memory ----
// Returns 1/alpha, which undoes the power-of-two pre-scale.
__device__ float prologue(const GemvParams &p, int m, __half *xs, int xstride, const uint2 (&wpre)[kPreVec], float *scratch)
{
    const ProIn pin{p.in, p.aux, p.norm_w, p.x_out, p.cols, p.prologue};
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

// One output row of one token through the epilogue of its segment.
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
        float *st = s.conv_state + size_t(row) * 3;
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

// RING = false: weights prefetched into registers (two chunks of UNR records per warp).
// RING = true : weights prefetched into a per-warp shared-memory ring of UNR stages by cp.async.bulk with mbarrier
//               completion; the kernel then needs half the registers, so two CTAs (this launch's and, under programmatic
//               dependent launch, the next one's, already filling its ring) fit on an SM.
template <int UNR, int M, bool RING>
__global__ void __launch_bounds__(kThreads, RING ? 2 : 1) gemv_fused_kernel(const __grid_constant__ GemvParams p)
{
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int nkb = p.nkb;
    const int xstride = p.cols + 8;
    __half *xs = reinterpret_cast<__half *>(smem_raw);
    float *rec = reinterpret_cast<float *>(smem_raw + size_t(M) * 2 * xstride * sizeof(__half)); // [16 warps][slots][M][16]
    float *scratch = rec + size_t(kWarps) * p.slots * M * 16;                                    // 64 floats
    __shared__ int s_last;
    __shared__ int s_wa[kWarps + 1], s_tmf[kWarps]; // warp boundaries in the record sequence, first run of each warp
    __shared__ __align__(8) uint64_t s_bar[RING ? kWarps * UNR : 1];
    __shared__ int s_abort;
    uint8_t *wring = reinterpret_cast<uint8_t *>(scratch + 64) + size_t(warp) * UNR * kRec; // RING: this warp's stages

    INSG_TRACE(0);
    pdl_launch_dependents();

    // this CTA's and this warp's share of the record sequence
    const int G = int(gridDim.x), c = int(blockIdx.x);
    // CTA ranges end on tile boundaries (a tile = one run, or the gate/up pair): no tile is shared between CTAs
    // The CTAs that get one tile more are the lowest-numbered ones: those are placed first, on the SMs the previous
    // kernel left first, so the extra tile goes where the head start is (and the stragglers' SMs get the short ranges).
    const int tq = p.total_etiles / G, tr = p.total_etiles % G;
    const int a = (c * tq + min(c, tr)) * p.etile_units, b = ((c + 1) * tq + min(c + 1, tr)) * p.etile_units;
    const int ua = a + (((b - a) * warp) >> 4), ub = a + (((b - a) * (warp + 1)) >> 4); // kWarps == 16
    const int tm_first = ua / nkb;
    if (lane == 0) {
        s_wa[warp] = ua;
        s_tmf[warp] = tm_first;
        if (warp == kWarps - 1) s_wa[kWarps] = ub;
    }

    UnitIt lit;
    it_set(p, lit, ua);
    Chunk<RING ? 1 : UNR> A, B;
    if constexpr (RING) {
        if (tid == 0) s_abort = 0;
        if (lane == 0) {
            for (int d = 0; d < UNR; d++) ring_bar_init(&s_bar[warp * UNR + d]);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
        // weights do not depend on the previous kernel: fill the ring before the dependency wait
        for (int d = 0; d < UNR; d++) {
            if (lit.u < ub) {
                if (lane == 0) ring_issue(wring + size_t(d) * kRec, lit.ptr, &s_bar[warp * UNR + d]);
                it_next(p, lit);
            }
        }
    } else {
        load_chunk<UNR>(p, A, lit, ub, lane);
        load_chunk<UNR>(p, B, lit, ub, lane);
    }
    uint2 wpre[kPreVec];
    preload_norm_weights(ProIn{p.in, p.aux, p.norm_w, p.x_out, p.cols, p.prologue}, wpre);
    INSG_TRACE(1);

    pdl_wait();
    INSG_TRACE(2);

    float inv_alpha[M];
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
            GemvParams q = p;
            q.in = p.aux;
            q.aux = nullptr;
            q.prologue = p.norm_w ? INSG_PRO_RMSNORM : INSG_PRO_PLAIN;
            preload_norm_weights(ProIn{q.in, q.aux, q.norm_w, nullptr, q.cols, q.prologue}, wpre);
            __syncthreads(); // every thread has read scratch[1]
#pragma unroll
            for (int m = 0; m < M; m++) inv_alpha[m] = prologue(q, m, xs, xstride, wpre, scratch);
        } else {
#pragma unroll
            for (int m = 0; m < M; m++) inv_alpha[m] = scratch[0];
        }
    } else {
#pragma unroll
        for (int m = 0; m < M; m++) inv_alpha[m] = prologue(p, m, xs, xstride, wpre, scratch);
    }
    __syncthreads();
    INSG_TRACE(3);

    const bool bactive = (t == (g >> 1));
    const int piece = g & 1;
    float acc[M][4];
#pragma unroll
    for (int m = 0; m < M; m++) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
    float *wrec = rec + size_t(warp) * p.slots * M * 16;

    // consume one chunk: multiply its records, closing a (tile, matrix) run whenever one ends
    UnitIt cit;
    it_set(p, cit, ua);
    auto compute = [&](const Chunk<RING ? 1 : UNR> &ch) {
#pragma unroll
        for (int j = 0; j < (RING ? 1 : UNR); j++) {
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
            it_next(p, cit);
        }
    };

    if constexpr (RING) {
        for (int idx = 0; cit.u < ub; idx++) {
            const int st = idx % UNR;
            uint64_t *bar = &s_bar[warp * UNR + st];
            if (!ring_wait(bar, (idx / UNR) & 1, &s_abort)) break;
            const uint8_t *stage = wring + size_t(st) * kRec;
            A.wa[0] = *reinterpret_cast<const uint4 *>(stage + lane * 16);
            A.wb[0] = *reinterpret_cast<const uint4 *>(stage + 512 + lane * 16);
            A.sc[0] = *reinterpret_cast<const uint16_t *>(stage + 1024 + lane * 2);
            __syncwarp(); // every lane has its copy: the stage may be overwritten
            if (lit.u < ub) {
                if (lane == 0) ring_issue(wring + size_t(st) * kRec, lit.ptr, bar);
                it_next(p, lit);
            }
            compute(A);
        }
    } else {
        while (cit.u < ub) {
            compute(A);
            load_chunk<UNR>(p, A, lit, ub, lane);
            if (cit.u >= ub) break;
            compute(B);
            load_chunk<UNR>(p, B, lit, ub, lane);
        }
    }
    if constexpr (RING) {
        if (tid == 0 && s_abort && p.error_flag) *p.error_flag = 1;
    }
    INSG_TRACE(4);
    __syncthreads();
    INSG_TRACE(5);

    // ---- combine: every (tile) this CTA touched, its runs summed over the warps in warp order --------
    float best = -3.402823466e38f;
    int best_idx = 0x7fffffff;
    float ss = 0.f; // sum of squares of the residual-stream rows this thread produced (prepared output only)
    if (b > a) {
        const int tm_lo = a / nkb, tm_hi = (b - 1) / nkb;
        const int row = lane & 15;
        // warp boundaries into registers once: the sums below then issue their shared-memory reads together
        int wr[kWarps + 1], tf[kWarps];
#pragma unroll
        for (int w = 0; w < kWarps; w++) { wr[w] = s_wa[w]; tf[w] = s_tmf[w]; }
        wr[kWarps] = s_wa[kWarps];
        // tasks are tiles: a run for plain segments, the (gate, up) pair of runs for SwiGLU
        for (int tmq = tm_lo + warp; tmq <= tm_hi; tmq += kWarps) {
            const SegDev &s = p.seg[seg_of(p, tmq)];
            const int local = tmq - s.tm_begin;
            if (s.nmat == 2 && (local & 1)) continue; // the pair is handled from its gate run
            const int tm0 = tmq - (s.nmat == 2 ? (local & 1) : 0);
            // Tokens are independent except for the convolution, whose history is carried from one token to the next:
            // there the 16 row lanes walk the tokens in order, elsewhere the two half-warps take alternate tokens.
            const bool serial = M > 1 && s.epilogue == INSG_EPI_CONV_SILU;
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
                if (tmq == tm_lo) INSG_TRACE(7);
                row_epilogue(s, (tm0 - s.tm_begin) / s.nmat * 16 + row, m, y[0], y[1], best, best_idx, ss);
            }
        }
    }

    INSG_TRACE(6);
    // ---- this CTA's share of sum(out^2), for the RMSNorm of the launch that consumes the prepared image ----
    if (p.prep_partials_out) {
        ss = warp_sum(ss);
        __syncthreads(); // scratch[0] was the prologue's
        if (lane == 0) scratch[warp] = ss;
        __syncthreads();
        if (tid == 0) {
            float tot = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; w++) tot += scratch[w];
            p.prep_partials_out[blockIdx.x] = tot;
        }
        if (blockIdx.x == 0)
            for (int i = G + tid; i < kMaxGrid; i += kThreads) p.prep_partials_out[i] = 0.f;
    }
    // ---- arg-max over the rows this launch produced (lm_head) ----------------
    if (p.argmax_partial) {
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
            p.argmax_partial[blockIdx.x] = make_float2(bv, __int_as_float(bi));
            __threadfence();
            const unsigned ticket = atomicAdd(p.argmax_ticket, 1u);
            s_last = (ticket == gridDim.x - 1);
        }
        __syncthreads();
        if (s_last) {
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
                    const int pos = *p.position_inout;
                    if (p.token_log) p.token_log[pos] = bi;
                    *p.position_inout = pos + 1;
                }
                *p.argmax_ticket = 0u;
            }
        }
    }
}

// ---- host side ------------------------------------------------------------------
namespace {
struct Tuning {
    int unr = 3;  // records per prefetch chunk (register variant): 3 measured best in the engine (2: 580, 3: 584, 4: 569 tok/s)
    int ring = 0; // > 0: shared-memory ring variant with up to this many stages per warp
    int ctas_per_sm = 1;
} g_tune;


template <int UNR, int M, bool RING> int launch_variant(const GemvParams &p, int grid, size_t smem, cudaStream_t st, bool pdl)
{
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(gemv_fused_kernel<UNR, M, RING>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    });
    if (attr_err != cudaSuccess) return cuda_fail(attr_err, "cudaFuncSetAttribute(gemv)");
    return launch(gemv_fused_kernel<UNR, M, RING>, dim3(grid), dim3(kThreads), smem + (RING ? size_t(kWarps) * UNR * kRec : 0), st, pdl, p);
}

template <int M> int dispatch(const GemvParams &p, int grid, size_t smem, cudaStream_t st, bool pdl)
{
    if (g_tune.ring) {
        // stages per warp: as deep as fits next to the activation copy while leaving room for a second CTA on the SM
        if (smem + size_t(kWarps) * 4 * kRec <= 112 * 1024 && g_tune.ring >= 4) return launch_variant<4, M, true>(p, grid, smem, st, pdl);
        if (smem + size_t(kWarps) * 3 * kRec <= 112 * 1024 && g_tune.ring >= 3) return launch_variant<3, M, true>(p, grid, smem, st, pdl);
        return launch_variant<2, M, true>(p, grid, smem, st, pdl);
    }
    if (g_tune.unr == 2 || M == 4) return launch_variant<2, M, false>(p, grid, smem, st, pdl); // four tokens: registers for accumulators
    if (g_tune.unr == 3) return launch_variant<3, M, false>(p, grid, smem, st, pdl);
    return launch_variant<4, M, false>(p, grid, smem, st, pdl);
}
} // namespace

int gemv_umma_launch(const insg_gemv_op *op, cudaStream_t st);

int gemv_tune(const char *key, int value)
{
    const std::string k = key;
    if (k == "gemv_unr") g_tune.unr = std::max(2, std::min(value, 4));
    else if (k == "gemv_ring") g_tune.ring = std::max(0, std::min(value, 4));
    else if (k == "gemv_ctas_per_sm") g_tune.ctas_per_sm = std::max(1, std::min(value, 2));
    else return fail(INSG_E_ARG, "unknown tuning key");
    return INSG_OK;
}

int gemv_fused_launch(const insg_gemv_op *op, int M, cudaStream_t st)
{
    if (!op || !op->in) return fail(INSG_E_ARG, "gemv: null operand");
    if (op->cols <= 0 || (op->cols & 127) || op->cols > kMaxVec * kThreads * 4)
        return fail(INSG_E_SHAPE, "gemv: cols must be a multiple of 128, <= 12288");
    if (op->n_segments < 1 || op->n_segments > 4) return fail(INSG_E_SHAPE, "gemv: 1..4 segments");
    if (M != 1 && M != 2 && M != 4) return fail(INSG_E_SHAPE, "gemv: 1, 2 or 4 tokens per launch");
    if ((op->prologue == INSG_PRO_RMSNORM || op->prologue == INSG_PRO_GATED_RMSNORM) && !op->norm_w)
        return fail(INSG_E_ARG, "gemv: norm weight missing");
    if (op->prologue >= INSG_PRO_GATED_RMSNORM && op->prologue != INSG_PRO_PREPARED && !op->aux)
        return fail(INSG_E_ARG, "gemv: prologue operand missing");
    if (op->prologue < 0 || op->prologue > INSG_PRO_PREPARED) return fail(INSG_E_ARG, "gemv: unknown prologue");
    if (op->prologue == INSG_PRO_PREPARED && M != 1) return fail(INSG_E_SHAPE, "gemv: a prepared input carries one token");
    if (op->prologue == INSG_PRO_GATED_RMSNORM && (op->cols & 127)) return fail(INSG_E_SHAPE, "gemv: gated norm needs cols % 128 == 0");
    GemvParams p = {};
    p.in = op->in; p.aux = op->aux; p.norm_w = op->norm_w; p.x_out = op->x_out;
    p.cols = op->cols; p.nkb = op->cols >> 7; p.prologue = op->prologue; p.nseg = op->n_segments;
    int tm = 0, nmat_all = 0;
    bool logits = false;
    for (int i = 0; i < op->n_segments; i++) {
        const insg_gemv_segment &s = op->seg[i];
        if (!s.packed || !s.out || s.rows <= 0 || (s.rows & 15)) return fail(INSG_E_SHAPE, "gemv: segment rows must be a positive multiple of 16");
        if (s.epilogue == INSG_EPI_SWIGLU && !s.packed2) return fail(INSG_E_ARG, "gemv: SwiGLU needs two matrices");
        if (s.epilogue == INSG_EPI_CONV_SILU && (!s.conv_state || !s.conv_w)) return fail(INSG_E_ARG, "gemv: conv operands missing");
        if (s.epilogue == INSG_EPI_DECAY && (!s.A_log || !s.dt_bias)) return fail(INSG_E_ARG, "gemv: decay operands missing");
        if (s.epilogue == INSG_EPI_LOGITS && M != 1) return fail(INSG_E_SHAPE, "gemv: the logits epilogue needs M == 1");
        SegDev &d = p.seg[i];
        d.packed = static_cast<const uint8_t *>(s.packed);
        d.packed2 = static_cast<const uint8_t *>(s.packed2);
        d.out = s.out; d.conv_state = s.conv_state; d.conv_w = s.conv_w; d.A_log = s.A_log; d.dt_bias = s.dt_bias;
        if (s.prep) {
            if (s.epilogue != INSG_EPI_RESIDUAL && s.epilogue != INSG_EPI_SWIGLU) return fail(INSG_E_ARG, "gemv: prepared output needs the residual or SwiGLU epilogue");
            if (M != 1) return fail(INSG_E_SHAPE, "gemv: a prepared output carries one token");
            if (s.prep_partials && op->n_segments != 1) return fail(INSG_E_ARG, "gemv: sums of squares come from a single-segment launch");
            d.prep = static_cast<__half *>(s.prep);
            d.prep_w = s.prep_w;
            if (s.prep_partials) p.prep_partials_out = s.prep_partials;
        }
        d.nmat = s.epilogue == INSG_EPI_SWIGLU ? 2 : 1;
        d.tm_begin = tm; tm += (s.rows >> 4) * d.nmat; d.epilogue = s.epilogue; d.rows = s.rows;
        if (nmat_all && nmat_all != d.nmat) return fail(INSG_E_SHAPE, "gemv: SwiGLU segments cannot be mixed with others");
        nmat_all = d.nmat;
        logits |= s.epilogue == INSG_EPI_LOGITS;
    }
    const long long units = (long long)tm * p.nkb;
    if (units > 0x7fffffffLL) return fail(INSG_E_LIMIT, "gemv: more than 2^31 records");
    p.total_tm = tm;
    p.total_units = int(units);
    // one CTA per SM, each owning whole output tiles; its 16 warps split the tiles' records evenly
    p.etile_units = nmat_all * p.nkb;
    p.total_etiles = tm / nmat_all;
    const int grid = std::max(1, std::min(std::min(sm_count() * (g_tune.ring ? g_tune.ctas_per_sm : 1), kMaxGrid), p.total_etiles));
    const int per_cta = (p.total_etiles + grid - 1) / grid * p.etile_units;
    p.slots = (per_cta / kWarps + 1 + p.nkb - 1) / p.nkb + 1;
    if (logits) {
        if (op->n_segments != 1) return fail(INSG_E_SHAPE, "gemv: the logits epilogue takes one segment");
        if (!op->argmax_scratch || !op->token_out) return fail(INSG_E_ARG, "gemv: arg-max scratch/token missing");
        p.argmax_ticket = static_cast<unsigned *>(op->argmax_scratch);
        p.argmax_partial = reinterpret_cast<float2 *>(static_cast<uint8_t *>(op->argmax_scratch) + 64);
        p.token_out = op->token_out;
        p.token_feedback = op->token_feedback;
        p.token_log = op->token_log;
        p.position_inout = op->position_inout;
    }
    p.trace = static_cast<unsigned long long *>(op->trace);
    p.error_flag = op->error_flag;
    p.prep_partials_in = op->prologue == INSG_PRO_PREPARED ? op->prep_partials : nullptr;
    p.prep_rms = op->prep_rms != 0;
    const size_t smem = size_t(M) * 2 * (op->cols + 8) * sizeof(__half) + size_t(kWarps) * p.slots * M * 16 * 4 + 64 * 4;
    if (smem > 220 * 1024) return fail(INSG_E_LIMIT, "gemv: shared memory beyond 220 KB");
    const bool pdl = op->pdl != 0;
    switch (M) {
    case 1: return dispatch<1>(p, grid, smem, st, pdl);
    case 2: return dispatch<2>(p, grid, smem, st, pdl);
    default: return dispatch<4>(p, grid, smem, st, pdl);
    }
}

} // namespace insg

using namespace insg;

extern "C" {

size_t insg_gemv_argmax_scratch_bytes(void) { return 64 + size_t(8) * 512; }

int insg_gemv_fused(const insg_gemv_op *op, insg_stream_t stream)
{
    if (op && op->layout == 1) {
        if (op->tokens > 1) return fail(INSG_E_SHAPE, "gemv: the tcgen05 layout takes one token per launch");
        return gemv_umma_launch(op, stream);
    }
    return gemv_fused_launch(op, op && op->tokens > 1 ? op->tokens : 1, stream);
}

int insg_mxfp4_gemv_packed(const void *packed, const float *x, float *y, int rows, int cols, int M, insg_stream_t stream)
{
    if (M < 1 || M > 4096) return fail(INSG_E_SHAPE, "gemv_packed: 1 <= M <= 4096");
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

} // extern "C"
