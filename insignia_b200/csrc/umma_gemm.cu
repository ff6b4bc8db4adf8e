// MXFP4 weights x several tokens on the 5th-generation tensor cores (tcgen05, sm_100a): the M >= 5 form of the GEMV.
//
// y[m][r] = sum_k e2m1(code(r,k)) * 2^(s(r,k/32)-127) * x[m][k]                 (reference: src/mxfp4.cu:41-66, M times)
//
// With several tokens the contraction is a real (if skinny) GEMM, and it runs where a GEMM belongs:
// tcgen05.mma.kind::mxf4.block_scale, weights as the A operand in their native packed E2M1 + UE8M0 form (the tile
// layout of insg_mxfp4_repack_umma, nothing dequantised), accumulators in tensor memory.  The activations are the
// B operand.  kind::mxf4 wants E2M1 there too, so each fp32 activation is written as a 25-bit signed fixed-point
// number (relative to its token's largest element) in balanced base 9: eight digits -4..4, every one exact in E2M1.
// Column j of a token holds digit j of every element; the eight columns are combined as sum_j 9^j D_j in fp32 by the
// epilogue, which gives the product to ~1e-7.  A token takes 8 columns of N: SIXTEEN tokens share one M128 x N128 x K64
// instruction (eight tokens an N64 one), which costs the tensor pipe what the one-token instruction costs.
//
// Kernels:
//   umma_digitize_kernel  one CTA per token: the fused activation prologue (RMSNorm, gates, ...), then the digit
//                         image of the token in global memory, laid out as the shared-memory image the MMA reads
//                         ([k-block][group of tokens][512 bytes x tokens per group], canonical K-major, no swizzle);
//   umma_gemm_kernel      one CTA per SM.  The work is the sequence of all (tile of 128 rows, token group, matrix,
//                         k-block) stages; every CTA takes an equal contiguous share of it (stream-K), so SMs are
//                         busy whatever the number of tiles.  A ring of stages, each one weight record + the group's
//                         digit block of the same k-block, both fetched by cp.async.bulk with mbarrier completion
//                         (local, no multicast); one thread issues the scale copies and the MMAs; accumulators double
//                         buffered so that four epilogue warps (tensor memory lane = output row) work on one run
//                         while the next one multiplies.  A (tile, group) that lies inside one CTA's share goes
//                         straight through the fused epilogue; one that is cut by a share boundary leaves per-CTA
//                         partial sums in scratch, and the CTA that arrives last (a ticket per cut unit) adds them
//                         in share order -- the result does not depend on which CTA that is -- and runs the
//                         epilogue.  Every wait is bounded: on expiry an error flag is raised and all roles drain.
//   conv_tokens_kernel    the causal convolution + SiLU over consecutive tokens of one sequence (the history runs
//                         through the tokens in order, so it cannot live in a per-unit epilogue).
#include "gemv_prologue.cuh"
#include "host_util.h"
#include "umma_common.cuh"

#include <algorithm>
#include <mutex>

namespace insg {

constexpr int kGThreads = kProThreads;     // digitize kernel: the activation prologue is written for this many threads
constexpr int kGemmThreads = 192;          // GEMM kernel: four epilogue warps, the MMA issuer, the producer
constexpr int kDigits = 8;                 // balanced base-9 digits per activation = N columns per token
constexpr int kGSfaBufs = 8;               // scale-factor column sets cycled by k-block
constexpr int kGTmemCols = 512;            // accumulators [0,256), weight scale factors [256,320), digit scale factors [320,324)
constexpr int kGMaxStages = 16;
constexpr int kGMaxGrid = 256;             // partial-sum slots and tickets are sized for this many CTAs
constexpr int kSlotFloats = 128 * 16;      // one partial: 128 rows x up to 16 tokens

// Development aid, compiled in only with -DINSG_PHASE_TIMES: clock stamps of the roles of every CTA of the last launch.
#ifdef INSG_PHASE_TIMES
__device__ unsigned long long g_gemm_stamps[kGMaxGrid * 16 + 4];
#define GEMM_STAMP(slot)                                                                                   \
    do {                                                                                                   \
        unsigned long long t_;                                                                             \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                            \
        g_gemm_stamps[blockIdx.x * 16 + (slot)] = t_;                                                      \
    } while (0)
#else
#define GEMM_STAMP(slot) \
    do {                 \
    } while (0)
#endif

struct GSeg {
    const uint8_t *packed, *packed2;
    float *out;
    float *conv_state;
    const uint16_t *conv_w;
    const float *A_log;
    const uint16_t *dt_bias;
    long long conv_stride; // 0: one sequence (the epilogue stores the raw product, conv_tokens_kernel follows); else token m's history at conv_state + m * stride
    int tile_begin, ntiles, nmat, epilogue, rows;
};

struct GParams {
    const uint8_t *bimg;    // [nkb][ngroups][512 * tpg]
    const float *inv_alpha; // [ngroups * tpg]
    float *partials;        // [grid][2 cut units][2 matrices][2 tiles][128 rows][tpg]
    int *tickets;           // [grid], zero between launches
    int nkb, nseg, total_tiles, stages, ngroups, tokens, sfa_lookahead, tpg, nmat;
    int total_stages, share, share_rem; // CTA c owns stages [share * c + share_rem * c / G, ...): all products stay in 32 bits
    GSeg seg[4];
    int *error_flag;
};

struct DigitizeParams {
    ProIn pro;
    uint8_t *bimg;
    float *inv_alpha;
    int *tickets;
    int tokens, ngroups, tpg, parts; // a token's digits are written by `parts` CTAs, each a slice of the columns
};

// Eight balanced base-9 digits of round(x * alpha) (|.| < 2^24) as E2M1 codes, digit j in nibble j.
__device__ __forceinline__ uint32_t digit_codes9(float x, float alpha)
{
    const int v = max(-0xFFFFFF, min(__float2int_rn(x * alpha), 0xFFFFFF));
    uint32_t u = uint32_t(v + 21523360); // + 4 * (9^8 - 1) / 8: plain base-9 digits 0..8 of u are the balanced digits + 4
    uint32_t codes = 0;
#pragma unroll
    for (int j = 0; j < kDigits; j++) {
        const uint32_t q = u / 9u, e = u - 9u * q; // digit + 4
        u = q;
        const int d = int(e) - 4;
        const uint32_t mag = uint32_t(d < 0 ? -d : d);                         // 0..4 -> E2M1 codes 0, 2, 4, 5, 6 (0, 1, 2, 3, 4)
        const uint32_t code = (mag < 3u ? 2u * mag : mag + 2u) | (d < 0 ? 8u : 0u);
        codes |= code << (4 * j);
    }
    return codes;
}

// `parts` CTAs per token slot (slots beyond `tokens` are written as zeros so that their columns contribute nothing).  Every
// CTA of a token runs the whole prologue (the norm and the token's largest element need all columns; that part is a few
// loads and one reduction) and writes the digits of its slice of the columns only: the digit extraction is the long part.
__global__ void __launch_bounds__(kGThreads, 2) umma_digitize_kernel(const __grid_constant__ DigitizeParams p)
{
    __shared__ float scratch[64];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); // the GEMM may set itself up and fetch weights meanwhile
#ifdef INSG_PHASE_TIMES
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t_;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));
        g_gemm_stamps[kGMaxGrid * 16] = t_;
    }
#endif
    const int m = blockIdx.x / p.parts, part = blockIdx.x - m * p.parts, grp = m / p.tpg, ms = m - grp * p.tpg;
    const int tid = threadIdx.x;
    const bool live = m < p.tokens;
    if (blockIdx.x == 0 && tid < kGMaxGrid) p.tickets[tid] = 0;
    float4 v[kMaxVec];
    float alpha = 0.f;
    if (live) {
        ProIn pin = p.pro;
        pin.x_out = nullptr;
        uint2 wpre[kPreVec];
        preload_norm_weights(pin, wpre);
        load_activation(pin, m, v);
        const float tmax = transform_activation(pin, m, v, wpre, scratch);
        int eb = int((__float_as_uint(tmax) >> 23) & 0xffu);
        eb = min(max(eb, 24), 230);
        alpha = __uint_as_float(uint32_t(127 + 23 - (eb - 127)) << 23); // max * alpha in [2^23, 2^24)
        if (tid == 0 && part == 0) p.inv_alpha[m] = __uint_as_float(uint32_t(eb - 23) << 23);
    } else {
#pragma unroll
        for (int j = 0; j < kMaxVec; j++) v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tid == 0 && part == 0) p.inv_alpha[m] = 0.f;
    }
    const int nvec = p.pro.cols >> 2;
    const int block = 512 * p.tpg, kstep = 256 * p.tpg;
    const int per = (nvec + p.parts - 1) / p.parts, v0 = part * per, v1 = min(nvec, v0 + per);
#pragma unroll
    for (int j = 0; j < kMaxVec; j++) {
        const int i = tid + j * kGThreads;
        if (i >= v0 && i < v1) {
            uint32_t c[4];
            c[0] = digit_codes9(v[j].x, alpha);
            c[1] = digit_codes9(v[j].y, alpha);
            c[2] = digit_codes9(v[j].z, alpha);
            c[3] = digit_codes9(v[j].w, alpha);
            // 4 consecutive k -> 2 bytes per column.  Block image: [2 K-steps][tpg column groups][2 k cores][8 columns][16 B];
            // the token's eight digit columns are one column group.
            const int k = i << 2, kb = k >> 7, kk = k & 127;
            const int half = (kk & 63) >> 1; // byte index of these k inside the 32-byte row of a K-step
            uint8_t *base = p.bimg + (size_t(kb) * p.ngroups + grp) * block + (kk >> 6) * kstep + ms * 256 + (half >> 4) * 128 + (half & 15);
#pragma unroll
            for (int col = 0; col < kDigits; col++) {
                const int sh = col * 4;
                const uint32_t two = ((c[0] >> sh) & 0xFu) | (((c[1] >> sh) & 0xFu) << 4) | (((c[2] >> sh) & 0xFu) << 8) | (((c[3] >> sh) & 0xFu) << 12);
                *reinterpret_cast<uint16_t *>(base + col * 16) = uint16_t(two);
            }
        }
    }
#ifdef INSG_PHASE_TIMES
    if (threadIdx.x == 0) {
        unsigned long long t_;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));
        atomicMax(&g_gemm_stamps[kGMaxGrid * 16 + 1], t_);
    }
#endif
}

// Causal convolution (kernel 4) + SiLU over `tokens` consecutive tokens of one sequence, in place: io[m][c] holds the raw
// projection on entry and the activation on return; the three-value history per channel is read and left updated.
// The filter is not recursive (out[m] needs raw[m-3..m] only), so a thread takes one channel and up to 32 tokens at a
// time: all their loads are in flight together, then the outputs are stored.  (reference: src/qwen_kernels.cu:31, once per token)
__global__ void conv_tokens_kernel(float *io, float *conv_state, const uint16_t *conv_w, int channels, int tokens)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    float *st = conv_state + size_t(c) * 3;
    float h0 = st[0], h1 = st[1], h2 = st[2];
    const uint2 wv = reinterpret_cast<const uint2 *>(conv_w)[c];
    const float w0 = bf16_bits_to_float(wv.x & 0xffff), w1 = bf16_bits_to_float(wv.x >> 16);
    const float w2 = bf16_bits_to_float(wv.y & 0xffff), w3 = bf16_bits_to_float(wv.y >> 16);
    for (int m0 = 0; m0 < tokens; m0 += 32) {
        float x[32];
#pragma unroll
        for (int j = 0; j < 32; j++) x[j] = m0 + j < tokens ? __ldcg(io + size_t(m0 + j) * channels + c) : 0.f;
#pragma unroll
        for (int j = 0; j < 32; j++) {
            if (m0 + j < tokens) {
                const float z = fmaf(h0, w0, fmaf(h1, w1, fmaf(h2, w2, x[j] * w3)));
                h0 = h1; h1 = h2; h2 = x[j];
                io[size_t(m0 + j) * channels + c] = fast_silu(z);
            }
        }
    }
    st[0] = h0; st[1] = h1; st[2] = h2;
}

__device__ __forceinline__ int gseg_of(const GParams &p, int tile)
{
    int s = 0;
#pragma unroll
    for (int i = 1; i < 4; i++)
        if (i < p.nseg && tile >= p.seg[i].tile_begin) s = i;
    return s;
}

// ---- the stream-K schedule ----------------------------------------------------------------------------------------------
// Stage g of the launch: unit = g / L (L = nmat * nkb), unit = tile * ngroups + group; inside the unit matrix 0's k-blocks,
// then matrix 1's.  CTA c owns stages [share_begin(c), share_begin(c + 1)).  A run = the part of one (unit, matrix) inside
// one share; it has its own accumulator.
__device__ __forceinline__ int share_begin(const GParams &p, int c, int G) { return p.share * c + (p.share_rem * c) / G; }
__device__ __forceinline__ int cta_of_stage(const GParams &p, int g, int G)
{
    int c = min(G - 1, g / p.share); // share >= 1; the remainder term moves the answer down by a few at most
    while (share_begin(p, c, G) > g) c--;
    while (c + 1 < G && share_begin(p, c + 1, G) <= g) c++;
    return c;
}

struct GRun {
    int g0;         // first stage
    int len;        // stages
    int unit, mat, kb0;
};
__device__ __forceinline__ GRun run_at(const GParams &p, int g, int end)
{
    const int q = g / p.nkb;                 // (unit, matrix) index
    const int qend = (q + 1) * p.nkb;
    GRun r;
    r.g0 = g;
    r.len = min(qend, end) - g;
    r.unit = p.nmat == 2 ? q >> 1 : q;
    r.mat = p.nmat == 2 ? q & 1 : 0;
    r.kb0 = g - q * p.nkb;
    return r;
}

// The fused epilogue of one row for the tokens of one group; y[] are finished sums (before the per-token scale).
// Everything stays in registers (fully unrolled, predicated): with nearly all of the SM's memory configured as shared
// memory, the little L1 that is left cannot hold a stack frame per thread, and spilled arrays would go to L2 and back.
// The switch sits outside the token loops so that a launch runs through one short straight-line piece only.
template <int TPG>
__device__ __forceinline__ void finish_row(const GParams &p, const GSeg &s, int row, int grp, const float (&y)[TPG], const float (&gate)[TPG],
                                           const float (&ia)[TPG])
{
    const int m0 = grp * TPG, live = min(TPG, p.tokens - m0);
    float *out = s.out + size_t(m0) * s.rows + row;
    const size_t ld = size_t(s.rows);
    switch (s.epilogue) {
    case INSG_EPI_RESIDUAL: {
        float r[TPG];
#pragma unroll
        for (int t = 0; t < TPG; t++) r[t] = t < live ? __ldcg(out + t * ld) : 0.f;
#pragma unroll
        for (int t = 0; t < TPG; t++)
            if (t < live) out[t * ld] = r[t] + y[t] * ia[t];
        break;
    }
    case INSG_EPI_CONV_SILU:
        if (s.conv_stride != 0) { // independent sequences: each token has its own history
            const uint2 wv = reinterpret_cast<const uint2 *>(s.conv_w)[row];
            const float cw0 = bf16_bits_to_float(wv.x & 0xffff), cw1 = bf16_bits_to_float(wv.x >> 16);
            const float cw2 = bf16_bits_to_float(wv.y & 0xffff), cw3 = bf16_bits_to_float(wv.y >> 16);
#pragma unroll
            for (int t = 0; t < TPG; t++) {
                if (t < live) {
                    float *st = s.conv_state + size_t(m0 + t) * s.conv_stride + size_t(row) * 3;
                    const float h0 = __ldcg(st), h1 = __ldcg(st + 1), h2 = __ldcg(st + 2), yv = y[t] * ia[t];
                    st[0] = h1; st[1] = h2; st[2] = yv;
                    out[t * ld] = fast_silu(fmaf(h0, cw0, fmaf(h1, cw1, fmaf(h2, cw2, yv * cw3))));
                }
            }
            break;
        }
        // one sequence: the raw product is stored, the convolution over the tokens follows as its own kernel
        [[fallthrough]];
    case INSG_EPI_STORE:
#pragma unroll
        for (int t = 0; t < TPG; t++)
            if (t < live) out[t * ld] = y[t] * ia[t];
        break;
    case INSG_EPI_BETA:
#pragma unroll
        for (int t = 0; t < TPG; t++)
            if (t < live) out[t * ld] = fast_sigmoid(y[t] * ia[t]);
        break;
    case INSG_EPI_DECAY: {
        const float bias = bf16_bits_to_float(s.dt_bias[row]), a = -__expf(s.A_log[row]);
#pragma unroll
        for (int t = 0; t < TPG; t++) {
            const float z = y[t] * ia[t] + bias;
            if (t < live) out[t * ld] = a * (z > 20.f ? z : log1pf(__expf(z)));
        }
        break;
    }
    case INSG_EPI_SWIGLU:
#pragma unroll
        for (int t = 0; t < TPG; t++)
            if (t < live) out[t * ld] = fast_silu(gate[t] * ia[t]) * (y[t] * ia[t]);
        break;
    default: break;
    }
}

// The sums of the TPG tokens of one accumulator (TMEM lane = row, eight digit columns per token), digits combined.
template <int TPG>
__device__ __forceinline__ void load_sums(uint32_t taddr, float (&y)[TPG])
{
#pragma unroll
    for (int t0 = 0; t0 < TPG; t0 += 8) { // eight tokens (two loads of 32 columns) per wait
        uint32_t d[2][32];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                         "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                         : "=r"(d[h][0]), "=r"(d[h][1]), "=r"(d[h][2]), "=r"(d[h][3]), "=r"(d[h][4]), "=r"(d[h][5]), "=r"(d[h][6]), "=r"(d[h][7]),
                           "=r"(d[h][8]), "=r"(d[h][9]), "=r"(d[h][10]), "=r"(d[h][11]), "=r"(d[h][12]), "=r"(d[h][13]), "=r"(d[h][14]), "=r"(d[h][15]),
                           "=r"(d[h][16]), "=r"(d[h][17]), "=r"(d[h][18]), "=r"(d[h][19]), "=r"(d[h][20]), "=r"(d[h][21]), "=r"(d[h][22]), "=r"(d[h][23]),
                           "=r"(d[h][24]), "=r"(d[h][25]), "=r"(d[h][26]), "=r"(d[h][27]), "=r"(d[h][28]), "=r"(d[h][29]), "=r"(d[h][30]), "=r"(d[h][31])
                         : "r"(taddr + kDigits * (t0 + 4 * h)));
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int t = 0; t < 8; t++) {
            const uint32_t *q = &d[t >> 2][(t & 3) * 8];
            // least significant digit first; 9^j is exact in fp32
            float ya = __uint_as_float(q[0]);
            ya = fmaf(__uint_as_float(q[1]), 9.f, ya);
            ya = fmaf(__uint_as_float(q[2]), 81.f, ya);
            ya = fmaf(__uint_as_float(q[3]), 729.f, ya);
            ya = fmaf(__uint_as_float(q[4]), 6561.f, ya);
            ya = fmaf(__uint_as_float(q[5]), 59049.f, ya);
            ya = fmaf(__uint_as_float(q[6]), 531441.f, ya);
            ya = fmaf(__uint_as_float(q[7]), 4782969.f, ya);
            y[t0 + t] = ya;
        }
    }
}

// Where the weight records of one (tile pair, matrix) start, and whether the pair has its second tile.
struct PairSrc {
    const uint8_t *a0, *a1;
    bool has1;
};
__device__ __forceinline__ PairSrc pair_src(const GParams &p, int pair, int mat, int kb)
{
    PairSrc q;
    const int t0 = 2 * pair, t1 = t0 + 1;
    const GSeg &s0 = p.seg[gseg_of(p, t0)];
    q.a0 = (mat ? s0.packed2 : s0.packed) + (size_t(t0 - s0.tile_begin) * p.nkb + kb) * kURec;
    q.has1 = t1 < p.total_tiles;
    q.a1 = q.a0;
    if (q.has1) {
        const GSeg &s1 = p.seg[gseg_of(p, t1)];
        q.a1 = (mat ? s1.packed2 : s1.packed) + (size_t(t1 - s1.tile_begin) * p.nkb + kb) * kURec;
    }
    return q;
}

template <int TPG, int NMAT>
__global__ void __launch_bounds__(kGemmThreads, 1) umma_gemm_kernel(const __grid_constant__ GParams p)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr int kBBlock = 512 * TPG;              // digits of the group's tokens for one k-block: 8 * TPG columns x 128 k x 4 bit
    constexpr int kGStage = 2 * kURec + kBBlock;    // one ring stage: the weight records of a pair of row tiles + the digit block both multiply
    constexpr int N = kDigits * TPG;
    // Tensor memory: accumulator sets of 2 tiles x N columns from column 0 (two sets of 2 x 64, or one of 2 x 128), the
    // weights' scale factors at [256, 320) (8 k-blocks x 2 tiles x 4 columns), the digits' (all 1) at [320, 324).
    constexpr int NB = TPG == 8 ? 2 : 1;
    constexpr uint32_t kSfaCol = 256, kSfbCol = 320;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nkb = p.nkb, S = p.stages;
    uint8_t *ring = smem;                          // S stages of kGStage bytes
    uint8_t *sfb = ring + size_t(S) * kGStage;     // 512 bytes
    __shared__ __align__(8) uint64_t full[kGMaxStages], empty[kGMaxStages], dfull[2], dempty[2];
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort, s_last;

    if (tid == 0) GEMM_STAMP(0);
    const int G = int(gridDim.x), c = int(blockIdx.x);
    const int begin = share_begin(p, c, G), end = share_begin(p, c + 1, G);
    const int total_kb = int(end - begin);
    constexpr int kNmat = NMAT;
    const int L = kNmat * nkb;

    if (tid == 0) {
        for (int i = 0; i < S; i++) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        for (int i = 0; i < 2; i++) { mbar_init(&dfull[i], 1); mbar_init(&dempty[i], 4); }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(kGTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    // column block scales: all 1 (the digit weights 9^j are not powers of two; the epilogue applies them)
    if (tid < 128) reinterpret_cast<uint32_t *>(sfb)[tid] = 0x7F7F7F7Fu;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    const uint32_t tmem = s_tmem;
    volatile int *abort_flag = &s_abort;
    if (tid == 0) GEMM_STAMP(1);

    if (warp == 5) {
        // ---- producer: the pair's two weight records + the token group's digit block per stage -----------------------
        // The weights do not depend on the launch before this one (the digit image does): the first ring of weight
        // records is requested before the programmatic-dependency wait, the digit blocks of those stages after it.
        // The first ring is requested by one lane per stage (a bulk copy takes the issuing thread a few hundred cycles).
        const int first = min(S, total_kb);
        const uint8_t *b0 = nullptr;
        uint8_t *dst0 = nullptr;
        if (lane < first) {
            const GRun r = run_at(p, begin + lane, end);
            const int pair = r.unit / p.ngroups, grp = r.unit - pair * p.ngroups;
            const PairSrc q = pair_src(p, pair, r.mat, r.kb0);
            b0 = p.bimg + (size_t(r.kb0) * p.ngroups + grp) * kBBlock;
            dst0 = ring + size_t(lane) * kGStage;
            mbar_expect_tx(&full[lane], (q.has1 ? 2 : 1) * kURec + kBBlock);
            bulk_load(dst0, q.a0, kURec, &full[lane]);
            if (q.has1) bulk_load(dst0 + kURec, q.a1, kURec, &full[lane]);
        }
        if (tid == 160) GEMM_STAMP(2);
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (tid == 160) GEMM_STAMP(3);
        if (lane < first) bulk_load(dst0 + 2 * kURec, b0, kBBlock, &full[lane]);
        if (lane == 0) {
            int g = begin + first, i = first;
            bool ok = true;
            while (g < end && ok) {
                const GRun r = run_at(p, g, end);
                const int pair = r.unit / p.ngroups, grp = r.unit - pair * p.ngroups;
                const PairSrc q = pair_src(p, pair, r.mat, r.kb0);
                const uint8_t *b_src = p.bimg + (size_t(r.kb0) * p.ngroups + grp) * kBBlock;
                const uint32_t bytes = (q.has1 ? 2 : 1) * kURec + kBBlock;
                for (int k = 0; k < r.len; k++, i++) {
                    const int st = i % S;
                    if (!mbar_wait(&empty[st], ((i / S) - 1) & 1, abort_flag)) { ok = false; break; }
                    uint8_t *dst = ring + size_t(st) * kGStage;
                    mbar_expect_tx(&full[st], bytes);
                    bulk_load(dst, q.a0 + size_t(k) * kURec, kURec, &full[st]);
                    if (q.has1) bulk_load(dst + kURec, q.a1 + size_t(k) * kURec, kURec, &full[st]);
                    bulk_load(dst + 2 * kURec, b_src + size_t(k) * p.ngroups * kBBlock, kBBlock, &full[st]);
                }
                g += r.len;
            }
            GEMM_STAMP(4);
        }
    } else if (warp == 4) {
        // ---- MMA issuer --------------------------------------------------------------------------------------------------
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            // E2M1 x E2M1, UE8M0 scales, N columns, M = 128
            const uint32_t idesc_base = (1u << 7) | (1u << 10) | ((uint32_t(N) >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24);
            asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem + kSfbCol), "l"(umma_desc(smem_u32(sfb), 16, 128)));
            // The scale-factor copies of a k-block are issued `la` k-blocks ahead of its MMAs: the tensor pipe runs its
            // work in order, and a copy placed right in front of the MMAs that need it puts its whole latency on the chain.
            // (A missing second tile's copy and MMAs read ring bytes nobody wrote; their results are never looked at.)
            const int la = p.sfa_lookahead;
            int i = 0, j = 0; // next stage to multiply, next stage whose scale factors are copied
            bool ok = true;
            auto copy_scales = [&](int upto) {
                for (; j <= upto && j < total_kb && ok; j++) {
                    const int st = j % S;
                    ok = mbar_wait(&full[st], (j / S) & 1, abort_flag);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sbase = smem_u32(ring + size_t(st) * kGStage);
#pragma unroll
                    for (int h = 0; h < 2; h++)
                        asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem + kSfaCol + 8 * (j % kGSfaBufs) + 4 * h),
                                     "l"(umma_desc(sbase + h * kURec + 8192, 16, 128)));
                }
            };
            int g = begin;
            for (int run = 0; g < end && ok; run++) {
                const GRun r = run_at(p, g, end);
                const bool has1 = 2 * (r.unit / p.ngroups) + 1 < p.total_tiles;
                const int buf = run % NB;
                ok = mbar_wait(&dempty[buf], ((run / NB) & 1) ^ 1, abort_flag); // first use of each set passes at once
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int k = 0; k < r.len; k++, i++) {
                    copy_scales(i + la);
                    if (!ok) break;
                    if (i == 0) GEMM_STAMP(5);
                    const int st = i % S;
                    const uint32_t sbase = smem_u32(ring + size_t(st) * kGStage);
#pragma unroll
                    for (int s = 0; s < 2; s++) {
                        const uint64_t db = umma_desc(sbase + 2 * kURec + s * (kBBlock / 2), 128, 256);
                        const uint32_t idesc = idesc_base | (uint32_t(2 * s) << 29); // A scales: bytes 2s, 2s+1; B scales: byte 0 (all equal)
                        const uint32_t acc = (k > 0 || s > 0) ? 1u : 0u;             // the run's first MMA overwrites
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            if (h == 1 && !has1) break;
                            const uint64_t da = umma_desc(sbase + h * kURec + s * 4096, 128, 256);
                            asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %4, 0;\n"
                                         "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], q;\n}"
                                         ::"r"(tmem + uint32_t((buf * 2 + h) * N)), "l"(da), "l"(db), "r"(idesc), "r"(acc),
                                           "r"(tmem + kSfaCol + 8 * (i % kGSfaBufs) + 4 * h), "r"(tmem + kSfbCol)
                                         : "memory");
                        }
                    }
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&empty[st])) : "memory");
                }
                if (ok) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&dfull[buf])) : "memory");
                g += r.len;
            }
            GEMM_STAMP(6);
        }
    } else if (warp < 4) {
        // ---- epilogue: tensor-memory lane = row of the tile; token t of the group = columns 8t .. 8t+7 --------------------
        float gate_val[NMAT == 2 ? 2 : 1][NMAT == 2 ? TPG : 1], zero[TPG];
#pragma unroll
        for (int t = 0; t < TPG; t++) zero[t] = 0.f;
        if (NMAT == 2) {
#pragma unroll
            for (int t = 0; t < TPG; t++) gate_val[0][NMAT == 2 ? t : 0] = gate_val[NMAT == 2 ? 1 : 0][NMAT == 2 ? t : 0] = 0.f;
        }
        asm volatile("griddepcontrol.wait;" ::: "memory"); // per-token scales, residual inputs and tickets come from earlier launches
        bool ok = true;
        int g = begin;
        for (int run = 0; g < end && ok; run++) {
            const GRun r = run_at(p, g, end);
            g += r.len;
            const int buf = run % NB;
            const int pair = r.unit / p.ngroups, grp = r.unit - pair * p.ngroups;
            float ia[TPG]; // the group's per-token scales: fetched while the run multiplies
#pragma unroll
            for (int t = 0; t < TPG; t += 4) {
                const float4 q = __ldcg(reinterpret_cast<const float4 *>(p.inv_alpha + grp * TPG) + (t >> 2));
                ia[t] = q.x; ia[t + 1] = q.y; ia[t + 2] = q.z; ia[t + 3] = q.w;
            }
            ok = mbar_wait(&dfull[buf], (run / NB) & 1, abort_flag);
            {   // the 128 epilogue threads go on or give up together (they meet at named barriers below)
                uint32_t all;
                asm volatile("{\n.reg .pred q, r;\nsetp.ne.b32 q, %1, 0;\nbar.red.and.pred r, 1, 128, q;\nselp.u32 %0, 1, 0, r;\n}"
                             : "=r"(all) : "r"(uint32_t(ok)) : "memory");
                ok = all != 0;
            }
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (tid == 0 && g >= end) GEMM_STAMP(7); // the last run's accumulators are complete
            const bool has1 = 2 * pair + 1 < p.total_tiles;
            float y[2][TPG];
            load_sums<TPG>(tmem + uint32_t((buf * 2) * N) + (uint32_t(warp * 32) << 16), y[0]);
            if (has1) load_sums<TPG>(tmem + uint32_t((buf * 2 + 1) * N) + (uint32_t(warp * 32) << 16), y[1]);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&dempty[buf]);
            if (tid == 0 && g >= end) GEMM_STAMP(10); // the last run's sums are in registers

            const int ubegin = r.unit * L, uend = ubegin + L;
            const bool whole = begin <= ubegin && uend <= end; // the whole unit lies in this CTA's share
            bool last = false;
            int c_first = 0, c_last = 0;
            if (!whole) {
                // ---- a unit cut by a share boundary: leave the partial sums; the CTA that arrives last adds them up ----
                c_first = cta_of_stage(p, ubegin, G);
                c_last = cta_of_stage(p, uend - 1, G);
                const int which = (begin > ubegin) ? 0 : 1; // the unit that contains this share's first stage, or a later one
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    if (h == 1 && !has1) break;
                    float *slot = p.partials + (((size_t(c) * 2 + which) * 2 + r.mat) * 2 + h) * kSlotFloats + size_t(tid) * TPG;
#pragma unroll
                    for (int t = 0; t < TPG; t += 4)
                        __stcg(reinterpret_cast<float4 *>(slot + t), make_float4(y[h][t], y[h][t + 1], y[h][t + 2], y[h][t + 3]));
                }
                const bool my_last_of_unit = g == end || g == uend;
                if (!my_last_of_unit) continue;
                // The barrier makes the 128 threads' partial stores visible to thread 0; its release at GPU scope is cumulative
                // over them, and the last arriver's acquire + the next barrier hand the other CTAs' stores to its 128 readers.
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (tid == 0) {
                    int seen;
                    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(seen) : "l"(p.tickets + c_first) : "memory");
                    s_last = seen == c_last - c_first;
                    if (s_last) p.tickets[c_first] = 0; // ready for the next launch
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                last = s_last != 0;
                asm volatile("bar.sync 1, 128;" ::: "memory"); // s_last may be rewritten by the next cut unit
                if (tid == 0 && g >= end) GEMM_STAMP(11);      // the last run's ticket is drawn
                if (!last) continue;
            } else if (NMAT == 2 && r.mat == 0) {
#pragma unroll
                for (int t = 0; t < TPG; t++) { gate_val[0][NMAT == 2 ? t : 0] = y[0][t]; gate_val[NMAT == 2 ? 1 : 0][NMAT == 2 ? t : 0] = y[1][t]; }
                continue;
            }
            if (whole) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    if (h == 1 && !has1) break;
                    const int tile = 2 * pair + h;
                    const GSeg &s = p.seg[gseg_of(p, tile)];
                    const int row = (tile - s.tile_begin) * 128 + tid;
                    if (row < s.rows) {
                        if constexpr (NMAT == 2) finish_row<TPG>(p, s, row, grp, y[h], gate_val[h], ia);
                        else finish_row<TPG>(p, s, row, grp, y[h], zero, ia);
                    }
                }
                continue;
            }
            // the last arriver: add the parts in share order (the sum does not depend on who arrived last)
#pragma unroll
            for (int h = 0; h < 2; h++) {
                if (h == 1 && !has1) break;
                float acc[NMAT][TPG]; // [matrix][token]
#pragma unroll
                for (int t = 0; t < TPG; t++) acc[0][t] = acc[NMAT - 1][t] = 0.f;
                int b = share_begin(p, c_first, G);
                for (int cc = c_first; cc <= c_last; cc++) {
                    const int e = share_begin(p, cc + 1, G);
                    const int which = (b > ubegin) ? 0 : 1;
#pragma unroll
                    for (int mat = 0; mat < NMAT; mat++) {
                        const int mb = ubegin + mat * nkb, me = mb + nkb;
                        if (max(b, mb) >= min(e, me)) continue; // that share holds nothing of this matrix
                        if (cc == c && mat == r.mat) { // this CTA's newest partial is still in registers
#pragma unroll
                            for (int t = 0; t < TPG; t++) acc[mat][t] += y[h][t];
                            continue;
                        }
                        const float *slot = p.partials + (((size_t(cc) * 2 + which) * 2 + mat) * 2 + h) * kSlotFloats + size_t(tid) * TPG;
                        float4 q[TPG / 4];
#pragma unroll
                        for (int t = 0; t < TPG / 4; t++) q[t] = __ldcg(reinterpret_cast<const float4 *>(slot) + t);
#pragma unroll
                        for (int t = 0; t < TPG / 4; t++) {
                            acc[mat][4 * t] += q[t].x; acc[mat][4 * t + 1] += q[t].y; acc[mat][4 * t + 2] += q[t].z; acc[mat][4 * t + 3] += q[t].w;
                        }
                    }
                    b = e;
                }
                if (tid == 0 && g >= end && h == 0) GEMM_STAMP(12); // first tile's parts added
                const int tile = 2 * pair + h;
                const GSeg &s = p.seg[gseg_of(p, tile)];
                const int row = (tile - s.tile_begin) * 128 + tid;
                if (row < s.rows) {
                    if constexpr (NMAT == 2) finish_row<TPG>(p, s, row, grp, acc[1], acc[0], ia);
                    else finish_row<TPG>(p, s, row, grp, acc[0], zero, ia);
                }
                if (tid == 0 && g >= end && h == 0) GEMM_STAMP(13); // first tile finished
            }
        }
    }
    if (tid == 0) GEMM_STAMP(8); // epilogue role done
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kGTmemCols));
    if (tid == 0 && s_abort && p.error_flag) *p.error_flag = 1;
    if (tid == 0) GEMM_STAMP(9);
}

// ---- host side --------------------------------------------------------------------------------------------------------
namespace {
std::mutex g_gemm_attr_mutex;
bool g_gemm_attr_done[64] = {false}; // the shared-memory opt-in is a per-device function attribute
constexpr int kGemmLookahead = 4; // k-blocks the scale-factor copies run ahead of the MMAs (0, 1, 2, 4, 6 measured alike within 2 %)

int tokens_per_group(int tokens) { return tokens <= 8 ? 8 : 16; }
size_t image_bytes(int cols, int tokens)
{
    const int tpg = tokens_per_group(tokens);
    const size_t groups = size_t(tokens + tpg - 1) / tpg;
    return size_t(cols >> 7) * groups * 512 * tpg;
}
constexpr size_t kPartialBytes = size_t(kGMaxGrid) * 2 * 2 * 2 * kSlotFloats * sizeof(float); // [CTA][cut unit][matrix][tile of the pair]
} // namespace


// digit image | per-token scales | partial sums of cut units | tickets
size_t umma_gemm_scratch(int cols, int tokens)
{
    if (cols <= 0 || (cols & 127) || tokens <= 0) return 0;
    const int tpg = tokens_per_group(tokens);
    const size_t groups = size_t(tokens + tpg - 1) / tpg;
    return image_bytes(cols, tokens) + ((groups * tpg * sizeof(float) + 255) & ~size_t(255)) + kPartialBytes + kGMaxGrid * sizeof(int);
}

int gemm_umma_launch(const insg_gemv_op *op, cudaStream_t st)
{
    if (!op || !op->in) return fail(INSG_E_ARG, "gemm: null operand");
    const int tokens = op->tokens;
    if (tokens < 1 || tokens > 4096) return fail(INSG_E_SHAPE, "gemm: 1 <= tokens <= 4096");
    if (op->cols <= 0 || (op->cols & 127) || op->cols > kMaxVec * kGThreads * 4) return fail(INSG_E_SHAPE, "gemm: cols must be a multiple of 128, <= 12288");
    if (op->n_segments < 1 || op->n_segments > 4) return fail(INSG_E_SHAPE, "gemm: 1..4 segments");
    if (op->prologue < 0 || op->prologue >= INSG_PRO_PREPARED) return fail(INSG_E_ARG, "gemm: prologue not available for several tokens");
    if ((op->prologue == INSG_PRO_RMSNORM || op->prologue == INSG_PRO_GATED_RMSNORM) && !op->norm_w) return fail(INSG_E_ARG, "gemm: norm weight missing");
    if (op->prologue >= INSG_PRO_GATED_RMSNORM && !op->aux) return fail(INSG_E_ARG, "gemm: prologue operand missing");
    const size_t need = umma_gemm_scratch(op->cols, tokens);
    if (!op->umma_scratch || op->umma_scratch_bytes < need) return fail(INSG_E_ARG, "gemm: scratch missing or too small (insg_umma_gemm_scratch_bytes)");
    if (reinterpret_cast<uintptr_t>(op->umma_scratch) & 255) return fail(INSG_E_ARG, "gemm: scratch must be 256-byte aligned");
    const int tpg = tokens_per_group(tokens);
    const int ngroups = (tokens + tpg - 1) / tpg, nkb = op->cols >> 7;

    DigitizeParams d = {};
    d.pro = ProIn{op->in, op->aux, op->norm_w, nullptr, op->cols, op->prologue};
    d.bimg = static_cast<uint8_t *>(op->umma_scratch);
    d.inv_alpha = reinterpret_cast<float *>(d.bimg + image_bytes(op->cols, tokens));
    d.tokens = tokens;
    d.ngroups = ngroups;
    d.tpg = tpg;
    // about one CTA per SM, a slice of at least 64 float4 columns each
    d.parts = std::max(1, std::min((op->cols >> 2) / 64, sm_count() / (ngroups * tpg)));

    GParams p = {};
    p.bimg = d.bimg;
    p.inv_alpha = d.inv_alpha;
    p.partials = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(d.inv_alpha) + ((size_t(ngroups) * tpg * sizeof(float) + 255) & ~size_t(255)));
    p.tickets = reinterpret_cast<int *>(reinterpret_cast<uint8_t *>(p.partials) + kPartialBytes);
    d.tickets = p.tickets;
    p.nkb = nkb;
    p.nseg = op->n_segments;
    p.ngroups = ngroups;
    p.tokens = tokens;
    p.tpg = tpg;
    int tiles = 0, nmat_all = 0;
    for (int i = 0; i < op->n_segments; i++) {
        const insg_gemv_segment &s = op->seg[i];
        if (!s.packed || !s.out || s.rows <= 0) return fail(INSG_E_SHAPE, "gemm: bad segment");
        if (s.epilogue == INSG_EPI_LOGITS) return fail(INSG_E_SHAPE, "gemm: the logits epilogue takes one token");
        if (s.prep) return fail(INSG_E_SHAPE, "gemm: a prepared output carries one token");
        if (s.epilogue == INSG_EPI_SWIGLU && !s.packed2) return fail(INSG_E_ARG, "gemm: SwiGLU needs two matrices");
        if (s.epilogue == INSG_EPI_CONV_SILU && (!s.conv_state || !s.conv_w)) return fail(INSG_E_ARG, "gemm: conv operands missing");
        if (s.epilogue == INSG_EPI_DECAY && (!s.A_log || !s.dt_bias)) return fail(INSG_E_ARG, "gemm: decay operands missing");
        GSeg &g = p.seg[i];
        g.packed = static_cast<const uint8_t *>(s.packed);
        g.packed2 = static_cast<const uint8_t *>(s.packed2);
        g.out = s.out; g.conv_state = s.conv_state; g.conv_w = s.conv_w; g.A_log = s.A_log; g.dt_bias = s.dt_bias;
        g.conv_stride = s.conv_token_stride;
        g.nmat = s.epilogue == INSG_EPI_SWIGLU ? 2 : 1;
        if (nmat_all && nmat_all != g.nmat) return fail(INSG_E_SHAPE, "gemm: SwiGLU segments cannot be mixed with others");
        nmat_all = g.nmat;
        g.tile_begin = tiles; g.ntiles = (s.rows + 127) >> 7; tiles += g.ntiles; g.epilogue = s.epilogue; g.rows = s.rows;
    }
    p.total_tiles = tiles;
    p.nmat = nmat_all;
    const long long total = (long long)((tiles + 1) / 2) * ngroups * nmat_all * nkb; // a unit = (pair of tiles, token group)
    if (total > (1ll << 30)) return fail(INSG_E_LIMIT, "gemm: more than 2^30 (tile, group, k-block) stages");
    p.total_stages = int(total);
    p.error_flag = op->error_flag;
    const int stage_bytes = 2 * kURec + 512 * tpg;
    p.stages = std::min(kGMaxStages, (224 * 1024 - 512) / stage_bytes);
    p.sfa_lookahead = std::max(0, std::min(kGemmLookahead, kGSfaBufs - 2));
    const size_t smem = size_t(p.stages) * stage_bytes + 512;
    auto kernel = tpg == 8 ? (nmat_all == 2 ? umma_gemm_kernel<8, 2> : umma_gemm_kernel<8, 1>) : (nmat_all == 2 ? umma_gemm_kernel<16, 2> : umma_gemm_kernel<16, 1>);
    {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
        if (dev < 0 || dev >= 64) return fail(INSG_E_LIMIT, "gemm: device ordinal beyond 63");
        std::lock_guard<std::mutex> lock(g_gemm_attr_mutex);
        if (!g_gemm_attr_done[dev]) {
            e = cudaFuncSetAttribute(umma_gemm_kernel<8, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(umma_gemm_kernel<8, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(umma_gemm_kernel<16, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(umma_gemm_kernel<16, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
            if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(umma gemm)");
            g_gemm_attr_done[dev] = true;
        }
    }
    // the digitize kernel is in plain stream order (its input comes from whatever ran before); the GEMM is its programmatic
    // dependent: it allocates tensor memory and requests its first weight records while the digits are being written
    int rc = launch(umma_digitize_kernel, dim3(ngroups * tpg * d.parts), dim3(kGThreads), 0, st, false, d);
    if (rc != INSG_OK) return rc;
    const int grid = std::max(1, std::min(std::min(sm_count(), kGMaxGrid), p.total_stages));
    p.share = p.total_stages / grid;
    p.share_rem = p.total_stages % grid;
    rc = launch(kernel, dim3(grid), dim3(kGemmThreads), smem, st, true, p); // may start while the digits are being written
    if (rc != INSG_OK) return rc;
    for (int i = 0; i < op->n_segments; i++) {
        const insg_gemv_segment &s = op->seg[i];
        if (s.epilogue == INSG_EPI_CONV_SILU && s.conv_token_stride == 0) { // one sequence: the history runs through the tokens
            rc = launch(conv_tokens_kernel, dim3((s.rows + 63) / 64), dim3(64), 0, st, false, s.out, s.conv_state, s.conv_w, s.rows, tokens);
            if (rc != INSG_OK) return rc;
        }
    }
    return INSG_OK;
}

} // namespace insg

using namespace insg;

extern "C" {

#ifdef INSG_PHASE_TIMES
// development builds: the stamps of the last launch -> host array of 256 * 16 + 4 values
__attribute__((visibility("default"))) int insg_debug_gemm_stamps(unsigned long long *host_out)
{
    return cudaMemcpyFromSymbol(host_out, g_gemm_stamps, sizeof(g_gemm_stamps)) == cudaSuccess ? 0 : 1;
}
__attribute__((visibility("default"))) int insg_debug_gemm_stamps_clear()
{
    static unsigned long long zeros[kGMaxGrid * 16 + 4];
    return cudaMemcpyToSymbol(g_gemm_stamps, zeros, sizeof(zeros)) == cudaSuccess ? 0 : 1;
}
#endif

size_t insg_umma_gemm_scratch_bytes(int cols, int tokens) { return umma_gemm_scratch(cols, tokens); }

int insg_mxfp4_gemm_umma(const void *packed_umma, const float *x, float *y, int rows, int cols, int M, void *scratch, size_t scratch_bytes,
                         insg_stream_t stream)
{
    insg_gemv_op op = {};
    op.in = x;
    op.cols = cols;
    op.prologue = INSG_PRO_PLAIN;
    op.n_segments = 1;
    op.seg[0].packed = packed_umma;
    op.seg[0].out = y;
    op.seg[0].rows = rows;
    op.seg[0].epilogue = INSG_EPI_STORE;
    op.tokens = M;
    op.layout = 1;
    op.umma_scratch = scratch;
    op.umma_scratch_bytes = scratch_bytes;
    return gemm_umma_launch(&op, stream);
}

} // extern "C"
