// MXFP4 weights x several tokens on the 5th-generation tensor cores (tcgen05, sm_100a): the M >= 8 form of the GEMV.
//
// y[m][r] = sum_k e2m1(code(r,k)) * 2^(s(r,k/32)-127) * x[m][k]                 (reference: src/mxfp4.cu:41-66, M times)
//
// With several tokens the contraction is a real (if skinny) GEMM, and it runs where a GEMM belongs:
// tcgen05.mma.kind::mxf4.block_scale, weights as the A operand in their native packed E2M1 + UE8M0 form (the tile
// layout of insg_mxfp4_repack_umma, nothing dequantised), accumulators in tensor memory.  The activations are the
// B operand.  kind::mxf4 wants E2M1 there too, so each fp32 activation is written as a 24-bit fixed-point number
// (relative to its token's largest element) cut into twelve base-4 digits: a digit 0..3 is exact in E2M1, column j
// of a token holds digit j of every element, the column's block scale is 4^j, and the twelve columns summed in fp32
// give the product to ~1e-7.  A token takes 16 columns of N (twelve digits, four empty); EIGHT tokens share one
// M128 x N128 x K64 instruction, which costs the tensor pipe what the one-token instruction costs.
//
// Two kernels:
//   umma_digitize_kernel  one CTA per token: the fused activation prologue (RMSNorm, gates, ...), then the digit
//                         image of the token in global memory, laid out as the shared-memory image the MMA reads
//                         ([k-block][group of 8 tokens][8192 bytes], canonical K-major, no swizzle);
//   umma_gemm_kernel      one CTA per SM over (tile of 128 rows) x (group of 8 tokens): a ring of stages, each
//                         one weight record + the group's digit block of the same k-block, both fetched by
//                         cp.async.bulk with mbarrier completion (local, no multicast); one thread issues the scale
//                         copies and the MMAs; accumulators double buffered so that four epilogue warps (tensor
//                         memory lane = output row) run the fused epilogues of one group while the next one
//                         multiplies.  Every wait is bounded: on expiry an error flag is raised and all roles drain.
#include "gemv_prologue.cuh"
#include "host_util.h"
#include "umma_common.cuh"

#include <algorithm>
#include <mutex>

namespace insg {

constexpr int kGThreads = kProThreads;
constexpr int kTokPerMma = 8;
constexpr int kBBlock = 8192;              // digits of 8 tokens for one k-block: 128 columns x 128 k x 4 bit
constexpr int kGStage = kURec + kBBlock;   // one ring stage
constexpr int kGSfaBufs = 8;               // scale-factor column sets cycled by k-block
constexpr int kGTmemCols = 512;            // D buffer 0 [0,128), D buffer 1 [128,256), SFA [256,288), SFB [288,292)

struct GSeg {
    const uint8_t *packed, *packed2;
    float *out;
    float *conv_state;
    const uint16_t *conv_w;
    const float *A_log;
    const uint16_t *dt_bias;
    long long conv_stride; // 0: one sequence (history carried through the tokens); else token m's history at conv_state + m * stride
    int tile_begin, ntiles, nmat, epilogue, rows;
};

struct GParams {
    const uint8_t *bimg;    // [nkb][ngroups][kBBlock]
    const float *inv_alpha; // [ngroups * 8]
    int nkb, nseg, total_tiles, stages, ngroups, tokens, sfa_lookahead, tile_major;
    GSeg seg[4];
    int *error_flag;
};

struct DigitizeParams {
    ProIn pro;
    uint8_t *bimg;
    float *inv_alpha;
    int tokens, ngroups;
};

// One CTA per token slot (slots beyond `tokens` are written as zeros so that their columns contribute nothing).
__global__ void __launch_bounds__(kGThreads) umma_digitize_kernel(const __grid_constant__ DigitizeParams p)
{
    __shared__ float scratch[64];
    const int m = blockIdx.x, grp = m >> 3, ms = m & 7;
    const int tid = threadIdx.x;
    const bool live = m < p.tokens;
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
        if (tid == 0) p.inv_alpha[m] = __uint_as_float(uint32_t(eb - 23) << 23);
    } else {
#pragma unroll
        for (int j = 0; j < kMaxVec; j++) v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tid == 0) p.inv_alpha[m] = 0.f;
    }
    const int nvec = p.pro.cols >> 2;
#pragma unroll
    for (int j = 0; j < kMaxVec; j++) {
        const int i = tid + j * kGThreads;
        if (i < nvec) {
            uint32_t lo[4], hi[4];
            digit_codes(v[j].x, alpha, lo[0], hi[0]);
            digit_codes(v[j].y, alpha, lo[1], hi[1]);
            digit_codes(v[j].z, alpha, lo[2], hi[2]);
            digit_codes(v[j].w, alpha, lo[3], hi[3]);
            // 4 consecutive k -> 2 bytes per column.  Block image: [2 K-steps][16 column groups][2 k cores][8 columns][16 B]
            const int k = i << 2, kb = k >> 7, kk = k & 127;
            const int half = (kk & 63) >> 1; // byte index of these k inside the 32-byte row of a K-step
            uint8_t *base = p.bimg + (size_t(kb) * p.ngroups + grp) * kBBlock + (kk >> 6) * 4096 + (half >> 4) * 128 + (half & 15);
#pragma unroll
            for (int col = 0; col < 16; col++) {
                const int n = 16 * ms + col;
                uint32_t two = 0;
                if (col < 12) {
                    const int sh = (col & 7) * 4;
                    const uint32_t *w = col < 8 ? lo : hi;
                    two = ((w[0] >> sh) & 0xFu) | (((w[1] >> sh) & 0xFu) << 4) | (((w[2] >> sh) & 0xFu) << 8) | (((w[3] >> sh) & 0xFu) << 12);
                }
                *reinterpret_cast<uint16_t *>(base + (n >> 3) * 256 + (n & 7) * 16) = uint16_t(two);
            }
        }
    }
}

__device__ __forceinline__ int gseg_of(const GParams &p, int tile)
{
    int s = 0;
#pragma unroll
    for (int i = 1; i < 4; i++)
        if (i < p.nseg && tile >= p.seg[i].tile_begin) s = i;
    return s;
}

__device__ __forceinline__ const uint8_t *grun_base(const GParams &p, int tile, int mat)
{
    const GSeg &s = p.seg[gseg_of(p, tile)];
    return (mat ? s.packed2 : s.packed) + size_t(tile - s.tile_begin) * p.nkb * kURec;
}

// Work is dealt to the CTAs in items.  Tile-major (a segment carries the convolution history from token to token, so all
// token groups of a tile stay in one CTA, in order): item = tile, CTA c takes tiles c, c + G, ..., each with its
// ngroups x nmat runs.  Otherwise item = (tile, token group), dealt round-robin: a 4096-row matrix (32 tiles) with four
// token groups then occupies 128 SMs instead of 32.
struct GRun {
    int tile, grp, mat;
};
__device__ __forceinline__ GRun grun_of(const GParams &p, int r, int c, int G, int nmat)
{
    if (p.tile_major) {
        const int per_tile = p.ngroups * nmat;
        const int ti = r / per_tile, rem = r - ti * per_tile;
        return GRun{c + ti * G, rem / nmat, rem % nmat};
    }
    const int item = c + (r / nmat) * G;
    return GRun{item / p.ngroups, item % p.ngroups, r % nmat};
}

__global__ void __launch_bounds__(kGThreads, 1) umma_gemm_kernel(const __grid_constant__ GParams p)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nkb = p.nkb, S = p.stages;
    uint8_t *ring = smem;                          // S stages of kGStage bytes
    uint8_t *sfb = ring + size_t(S) * kGStage;     // 512 bytes
    __shared__ __align__(8) uint64_t full[16], empty[16], dfull[2], dempty[2];
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;

    const int G = int(gridDim.x), c = int(blockIdx.x);
    const int nmat = p.seg[0].nmat;
    const int total_items = p.tile_major ? p.total_tiles : p.total_tiles * p.ngroups;
    const int my_items = c < total_items ? (total_items - c + G - 1) / G : 0;
    const int nruns = my_items * (p.tile_major ? p.ngroups : 1) * nmat;
    const int total_kb = nruns * nkb;

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
    // column block scales: column n = 16 * token + digit: 4^digit for the twelve digit columns, 1 for the empty ones.
    // Image [32 rows][4 quarters] of four equal bytes, column n at row n & 31, quarter n >> 5.
    if (tid < 128) {
        const int n = tid, digit = n & 15;
        reinterpret_cast<uint32_t *>(sfb)[(n & 31) * 4 + (n >> 5)] = digit < 12 ? 0x01010101u * uint32_t(127 + 2 * digit) : 0x7F7F7F7Fu;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    const uint32_t tmem = s_tmem;
    volatile int *abort_flag = &s_abort;

    if (warp == 5) {
        // ---- producer: one weight record + the token group's digit block per stage ------------------------------------
        if (lane == 0) {
            for (int i = 0; i < total_kb; i++) {
                const int st = i % S;
                if (i >= S && !mbar_wait(&empty[st], ((i / S) - 1) & 1, abort_flag)) break;
                const int run = i / nkb, kb = i - run * nkb;
                const GRun r = grun_of(p, run, c, G, nmat);
                const uint8_t *a_src = grun_base(p, r.tile, r.mat) + size_t(kb) * kURec;
                const uint8_t *b_src = p.bimg + (size_t(kb) * p.ngroups + r.grp) * kBBlock;
                uint8_t *dst = ring + size_t(st) * kGStage;
                mbar_expect_tx(&full[st], kGStage);
                bulk_load(dst, a_src, kURec, &full[st]);
                bulk_load(dst + kURec, b_src, kBBlock, &full[st]);
            }
        }
    } else if (warp == 4) {
        // ---- MMA issuer --------------------------------------------------------------------------------------------------
        if (lane == 0) {
            // E2M1 x E2M1, UE8M0 scales, N = 128, M = 128
            const uint32_t idesc_base = (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24);
            asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem + 288), "l"(umma_desc(smem_u32(sfb), 16, 128)));
            // The scale-factor copy of a k-block is issued `la` k-blocks ahead of its MMAs: the tensor pipe runs its
            // work in order, and a copy placed right in front of the MMAs that need it puts its whole latency on the chain.
            const int la = p.sfa_lookahead;
            int i = 0, j = 0; // next k-block to multiply, next k-block whose scale factors are copied
            bool ok = true;
            auto copy_scales = [&](int upto) {
                for (; j <= upto && j < total_kb && ok; j++) {
                    const int st = j % S;
                    ok = mbar_wait(&full[st], (j / S) & 1, abort_flag);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sbase = smem_u32(ring + size_t(st) * kGStage);
                    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem + 256 + 4 * (j % kGSfaBufs)),
                                 "l"(umma_desc(sbase + 8192, 16, 128)));
                }
            };
            for (int run = 0; run < nruns && ok; run++) {
                const int buf = run & 1;
                ok = mbar_wait(&dempty[buf], ((run >> 1) & 1) ^ 1, abort_flag); // first use of each buffer passes at once
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int kb = 0; kb < nkb; kb++, i++) {
                    copy_scales(i + la);
                    if (!ok) break;
                    const int st = i % S;
                    const uint32_t sbase = smem_u32(ring + size_t(st) * kGStage);
                    const uint32_t t_sfa = tmem + 256 + 4 * (i % kGSfaBufs);
#pragma unroll
                    for (int s = 0; s < 2; s++) {
                        const uint64_t da = umma_desc(sbase + s * 4096, 128, 256), db = umma_desc(sbase + kURec + s * 4096, 128, 256);
                        const uint32_t idesc = idesc_base | (uint32_t(2 * s) << 29); // A scales: bytes 2s, 2s+1; B scales: byte 0 (all equal)
                        const uint32_t acc = (kb > 0 || s > 0) ? 1u : 0u;            // the run's first MMA overwrites
                        asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %4, 0;\n"
                                     "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], q;\n}"
                                     ::"r"(tmem + 128 * buf), "l"(da), "l"(db), "r"(idesc), "r"(acc), "r"(t_sfa), "r"(tmem + 288)
                                     : "memory");
                    }
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&empty[st])) : "memory");
                }
                if (ok) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&dfull[buf])) : "memory");
            }
        }
    } else if (warp < 4) {
        // ---- epilogue: tensor-memory lane = row of the tile; token t of the group = columns 16t .. 16t+11 ----------------
        float gate_val[kTokPerMma];
#pragma unroll
        for (int t = 0; t < kTokPerMma; t++) gate_val[t] = 0.f;
        bool ok = true;
        for (int run = 0; run < nruns && ok; run++) {
            const int buf = run & 1;
            ok = mbar_wait(&dfull[buf], (run >> 1) & 1, abort_flag);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float y[kTokPerMma];
#pragma unroll
            for (int t = 0; t < kTokPerMma; t++) {
                uint32_t r[16];
                const uint32_t taddr = tmem + 128 * buf + 16 * t + (uint32_t(warp * 32) << 16);
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                               "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                             : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                float ya = 0.f;
#pragma unroll
                for (int j = 0; j < 12; j++) ya += __uint_as_float(r[j]); // least significant digit first
                y[t] = ya;
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&dempty[buf]);
            const GRun rr = grun_of(p, run, c, G, nmat);
            const GSeg &s = p.seg[gseg_of(p, rr.tile)];
            const int row = (rr.tile - s.tile_begin) * 128 + tid;
            if (row < s.rows) {
                // tokens in order: the convolution history is carried from one token to the next, in registers
                float h0 = 0.f, h1 = 0.f, h2 = 0.f, cw0 = 0.f, cw1 = 0.f, cw2 = 0.f, cw3 = 0.f;
                const bool carried = s.epilogue == INSG_EPI_CONV_SILU && s.conv_stride == 0;
                if (s.epilogue == INSG_EPI_CONV_SILU) {
                    if (carried) {
                        const float *st = s.conv_state + size_t(row) * 3;
                        h0 = __ldcg(st); h1 = __ldcg(st + 1); h2 = __ldcg(st + 2);
                    }
                    const uint2 wv = reinterpret_cast<const uint2 *>(s.conv_w)[row];
                    cw0 = bf16_bits_to_float(wv.x & 0xffff); cw1 = bf16_bits_to_float(wv.x >> 16);
                    cw2 = bf16_bits_to_float(wv.y & 0xffff); cw3 = bf16_bits_to_float(wv.y >> 16);
                }
#pragma unroll
                for (int t = 0; t < kTokPerMma; t++) {
                    const int m = rr.grp * kTokPerMma + t;
                    if (m >= p.tokens) break;
                    const float yv = y[t] * __ldg(p.inv_alpha + m);
                    float *out = s.out + size_t(m) * s.rows;
                    switch (s.epilogue) {
                    case INSG_EPI_STORE: out[row] = yv; break;
                    case INSG_EPI_RESIDUAL: out[row] = __ldcg(out + row) + yv; break;
                    case INSG_EPI_CONV_SILU: {
                        if (!carried) { // independent sequences: each token has its own history
                            float *st = s.conv_state + size_t(m) * s.conv_stride + size_t(row) * 3;
                            h0 = __ldcg(st); h1 = __ldcg(st + 1); h2 = __ldcg(st + 2);
                            st[0] = h1; st[1] = h2; st[2] = yv;
                        }
                        const float z = fmaf(h0, cw0, fmaf(h1, cw1, fmaf(h2, cw2, yv * cw3)));
                        h0 = h1; h1 = h2; h2 = yv;
                        out[row] = fast_silu(z);
                        break;
                    }
                    case INSG_EPI_BETA: out[row] = fast_sigmoid(yv); break;
                    case INSG_EPI_DECAY: {
                        const float z = yv + bf16_bits_to_float(s.dt_bias[row]);
                        const float soft = z > 20.f ? z : log1pf(__expf(z));
                        out[row] = -__expf(s.A_log[row]) * soft;
                        break;
                    }
                    case INSG_EPI_SWIGLU:
                        if (rr.mat == 0) gate_val[t] = yv;
                        else out[row] = fast_silu(gate_val[t]) * yv;
                        break;
                    default: break;
                    }
                }
                if (carried) {
                    float *st = s.conv_state + size_t(row) * 3;
                    st[0] = h0; st[1] = h1; st[2] = h2;
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kGTmemCols));
    if (tid == 0 && s_abort && p.error_flag) *p.error_flag = 1;
}

// ---- host side --------------------------------------------------------------------------------------------------------
namespace {
std::mutex g_gemm_attr_mutex;
bool g_gemm_attr_done[64] = {false}; // the shared-memory opt-in is a per-device function attribute
int g_gemm_lookahead = 4;
} // namespace

int umma_gemm_tune(const char *key, int value)
{
    if (std::string(key) == "umma_gemm_lookahead") { g_gemm_lookahead = value; return INSG_OK; }
    return INSG_E_ARG;
}

size_t umma_gemm_scratch(int cols, int tokens)
{
    if (cols <= 0 || (cols & 127) || tokens <= 0) return 0;
    const size_t groups = size_t(tokens + kTokPerMma - 1) / kTokPerMma;
    return size_t(cols >> 7) * groups * kBBlock + groups * kTokPerMma * sizeof(float);
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
    const int ngroups = (tokens + kTokPerMma - 1) / kTokPerMma, nkb = op->cols >> 7;

    DigitizeParams d = {};
    d.pro = ProIn{op->in, op->aux, op->norm_w, nullptr, op->cols, op->prologue};
    d.bimg = static_cast<uint8_t *>(op->umma_scratch);
    d.inv_alpha = reinterpret_cast<float *>(d.bimg + size_t(nkb) * ngroups * kBBlock);
    d.tokens = tokens;
    d.ngroups = ngroups;

    GParams p = {};
    p.bimg = d.bimg;
    p.inv_alpha = d.inv_alpha;
    p.nkb = nkb;
    p.nseg = op->n_segments;
    p.ngroups = ngroups;
    p.tokens = tokens;
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
    // (tile, token group) items only where whole tiles would leave SMs idle: the groups of a tile then run on different SMs
    // at different times and each streams the tile's weights again
    p.tile_major = tiles >= sm_count() ? 1 : 0;
    for (int i = 0; i < op->n_segments; i++) p.tile_major |= op->seg[i].epilogue == INSG_EPI_CONV_SILU && op->seg[i].conv_token_stride == 0;
    p.error_flag = op->error_flag;
    p.stages = 12;
    p.sfa_lookahead = std::max(0, std::min(g_gemm_lookahead, kGSfaBufs - 2));
    const size_t smem = size_t(p.stages) * kGStage + 512;
    {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
        if (dev < 0 || dev >= 64) return fail(INSG_E_LIMIT, "gemm: device ordinal beyond 63");
        std::lock_guard<std::mutex> lock(g_gemm_attr_mutex);
        if (!g_gemm_attr_done[dev]) {
            e = cudaFuncSetAttribute(umma_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
            if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(umma gemm)");
            g_gemm_attr_done[dev] = true;
        }
    }
    // plain stream order for both launches: neither kernel waits on a dependency of its own
    int rc = launch(umma_digitize_kernel, dim3(ngroups * kTokPerMma), dim3(kGThreads), 0, st, false, d);
    if (rc != INSG_OK) return rc;
    const int grid = std::max(1, std::min(sm_count(), p.tile_major ? tiles : tiles * ngroups));
    return launch(umma_gemm_kernel, dim3(grid), dim3(kGThreads), smem, st, false, p);
}

} // namespace insg

using namespace insg;

extern "C" {

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
