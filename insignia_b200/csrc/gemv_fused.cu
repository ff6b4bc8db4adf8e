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
#include "gemv_body.cuh"
#include "host_util.h"

#include <algorithm>
#include <mutex>

namespace insg {

// One launch = the stages of gemv_body.cuh in order.  The weight loads are issued before the programmatic-dependent-
// launch wait, so they overlap the tail of the previous kernel in the stream.
template <int UNR, int M>
__global__ void __launch_bounds__(kThreads, 1) gemv_fused_kernel(const __grid_constant__ GemvParams p)
{
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __shared__ GemvShared sh;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int xstride = p.cols + 8;
    __half *xs = reinterpret_cast<__half *>(smem_raw);
    float *rec = reinterpret_cast<float *>(smem_raw + size_t(M) * 2 * xstride * sizeof(__half)); // [16 warps][slots][M][16]
    float *scratch = rec + size_t(kWarps) * p.slots * M * 16;                                    // 64 floats

    pdl_launch_dependents();

    const int G = int(gridDim.x), c = int(blockIdx.x);
    const GemvRange r = gemv_range(p, G, c, warp);
    gemv_publish_range(r, sh, lane, warp);
    UnitIt lit;
    Chunk<UNR> A, B;
    gemv_issue_first<UNR>(p, r, A, B, lit, lane);
    uint2 wpre[kPreVec];
    preload_norm_weights(ProIn{p.in, p.aux, p.norm_w, p.x_out, p.cols, p.prologue}, wpre);

    pdl_wait();

    float inv_alpha[M];
    gemv_activation<M>(p, xs, xstride, scratch, wpre, inv_alpha);
    gemv_stream<UNR, M>(p, r, A, B, lit, xs, xstride, rec + size_t(warp) * p.slots * M * 16, inv_alpha, lane);
    __syncthreads();
    gemv_finish<M>(p, r, G, c, rec, scratch, sh);
}

// ---- host side ------------------------------------------------------------------
namespace {

// The opt-in to more than 48 KB of dynamic shared memory is a per-device function attribute: set once per
// (kernel variant, device).
template <int UNR, int M> int launch_variant(const GemvParams &p, int grid, size_t smem, cudaStream_t st, bool pdl)
{
    static std::mutex mu;
    static bool done[64] = {false};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(INSG_E_LIMIT, "gemv: device ordinal beyond 63");
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!done[dev]) {
            e = cudaFuncSetAttribute(gemv_fused_kernel<UNR, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
            if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(gemv)");
            done[dev] = true;
        }
    }
    return launch(gemv_fused_kernel<UNR, M>, dim3(grid), dim3(kThreads), smem, st, pdl, p);
}

} // namespace

int gemv_umma_launch(const insg_gemv_op *op, cudaStream_t st);
int gemm_umma_launch(const insg_gemv_op *op, cudaStream_t st);

// Validates a fused-GEMV description and turns it into the kernel's parameter block for a grid of at most `max_grid`
// CTAs (one per SM); *grid and *smem receive the launch shape.
int gemv_build_params(const insg_gemv_op *op, int M, int max_grid, GemvParams *out, int *grid_out, size_t *smem_out)
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
        d.conv_stride = s.conv_token_stride;
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
    const int grid = std::max(1, std::min(std::min(max_grid, kMaxGrid), p.total_etiles));
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
        p.token_log_capacity = op->token_log_capacity;
        if (op->token_log && op->token_log_capacity <= 0) return fail(INSG_E_ARG, "gemv: token_log needs its capacity");
        p.position_inout = op->position_inout;
    }
    p.prep_partials_in = op->prologue == INSG_PRO_PREPARED ? op->prep_partials : nullptr;
    p.prep_rms = op->prep_rms != 0;
    const size_t smem = gemv_smem_bytes(M, op->cols, p.slots);
    if (smem > 220 * 1024) return fail(INSG_E_LIMIT, "gemv: shared memory beyond 220 KB");
    *out = p;
    *grid_out = grid;
    *smem_out = smem;
    return INSG_OK;
}

int gemv_fused_launch(const insg_gemv_op *op, int M, cudaStream_t st)
{
    GemvParams p;
    int grid = 0;
    size_t smem = 0;
    const int rc = gemv_build_params(op, M, sm_count(), &p, &grid, &smem);
    if (rc != INSG_OK) return rc;
    const bool pdl = op->pdl != 0;
    switch (M) {
    case 1: return launch_variant<kUnr, 1>(p, grid, smem, st, pdl);
    case 2: return launch_variant<kUnr, 2>(p, grid, smem, st, pdl);
    default: return launch_variant<2, 4>(p, grid, smem, st, pdl); // four tokens: registers go to the accumulators
    }
}

} // namespace insg

using namespace insg;

extern "C" {

size_t insg_gemv_argmax_scratch_bytes(void) { return 64 + size_t(8) * 512; }

int insg_gemv_fused(const insg_gemv_op *op, insg_stream_t stream)
{
    if (op && op->layout == 1) return op->tokens > 1 ? gemm_umma_launch(op, stream) : gemv_umma_launch(op, stream);
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
