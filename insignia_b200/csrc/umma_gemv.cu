// MXFP4 GEMV on the 5th-generation tensor cores (tcgen05, sm_100a), batch 1.
//
// y[r] = sum_k e2m1(code(r,k)) * 2^(s(r,k/32)-127) * x[k]            (reference: src/mxfp4.cu:41-66)
//
// The checkpoint's weights ARE the A operand of tcgen05.mma kind::mxf4.block_scale: packed E2M1 with
// one UE8M0 scale per 32 values along K.  Nothing is dequantised in registers: weights go
// HBM -> shared memory with cp.async.bulk (TMA, mbarrier completion) and are read from there by the
// tensor core, with their scale bytes copied shared -> tensor memory by tcgen05.cp.  The stream is HBM
// bound (17 bytes per 32 weights) and the SM's instruction slots stay free.
//
// The activation is the B operand, which for kind::mxf4 must be E2M1 as well.  It is written as a
// 24-bit fixed-point number (relative to the largest element of the vector) cut into twelve base-4
// digits: a digit 0..3 is exactly representable in E2M1, so column j of B holds digit j of every
// element with the column's block scale set to 4^j, and y = sum_j D[:, j] / alpha is an exact
// positional recombination in fp32.  (N = 16 columns are required by the M = 128 instruction shape;
// the last four are zero.)
//
// Layout of the weights for this kernel (insg_mxfp4_repack_umma), same 17 bytes per 32 weights: rows
// in tiles of 128, K in blocks of 128; one (tile, block) record is 8704 contiguous bytes = the shared
// memory image the MMA reads: 2 K-steps of 64 x [16 row groups][2 k cores][8 rows][16 bytes]
// (canonical K-major, no swizzle: leading byte offset 128, stride byte offset 256), then the 512-byte
// scale block [32 rows][4 row quarters][4 groups] that tcgen05.cp.32x128b.warpx4 expects.
//
// CTA roles (512 threads): every warp takes part in the activation prologue; then one thread issues
// bulk copies into a ring of stages, one thread issues tcgen05.cp + tcgen05.mma and commits stage
// releases, warps 0-3 read the accumulators (tcgen05.ld, TMEM lane = output row) and run the fused
// epilogue.  Accumulators are double buffered so a tile's epilogue overlaps the next tile's MMAs.
// Every wait is bounded: on expiry a flag is raised in global memory and all roles drain.
#include "gemv_prologue.cuh"
#include "umma_common.cuh"
#include "host_util.h"

#include <algorithm>
#include <mutex>

namespace insg {

constexpr int kUThreads = kProThreads;
constexpr int kBImgPerKb = 1024;     // activation digits: 16 columns x 128 k x 4 bit
constexpr int kAccMax = 8;           // independent accumulators per tile: consecutive MMAs must not wait on each other's result
constexpr int kSfaBufs = 8;          // scale-factor column sets cycled by k-block
constexpr int kTmemCols = 512;       // D set 0 [0,128) D set 1 [128,256) SFA [256,288) SFB [288,292)

struct USeg {
    const uint8_t *packed, *packed2;
    float *out;
    float *conv_state;
    const uint16_t *conv_w;
    const float *A_log;
    const uint16_t *dt_bias;
    int tile_begin, ntiles, nmat, epilogue, rows;
};

struct UParams {
    ProIn pro;
    int nkb, nseg, total_tiles, stages, nacc, prefetch;
    USeg seg[4];
    float2 *argmax_partial;
    unsigned *argmax_ticket;
    int *token_out, *token_feedback, *token_log, *position_inout;
    int *error_flag;
    int token_log_capacity;
};

// kblock i of this CTA's sequence -> global address of its record and its place in the tile sequence
struct URun {
    const uint8_t *rec;
    int run;  // index of the (tile, matrix) run inside this CTA
    int kb;
};

__device__ __forceinline__ int useg_of(const UParams &p, int tile)
{
    int s = 0;
#pragma unroll
    for (int i = 1; i < 4; i++)
        if (i < p.nseg && tile >= p.seg[i].tile_begin) s = i;
    return s;
}

// Run r of CTA c: tile = c + (r / nmat) * G, matrix r % nmat (nmat is the same for all segments of a launch).
__device__ __forceinline__ const uint8_t *run_base(const UParams &p, int tile, int mat)
{
    const USeg &s = p.seg[useg_of(p, tile)];
    return (mat ? s.packed2 : s.packed) + size_t(tile - s.tile_begin) * p.nkb * kURec;
}

__global__ void __launch_bounds__(kUThreads, 1) umma_gemv_kernel(const __grid_constant__ UParams p)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nkb = p.nkb, S = p.stages;
    uint8_t *ring = smem;                                   // S stages of kURec bytes
    uint8_t *bimg = ring + size_t(S) * kURec;               // nkb x 1024 bytes of activation digits
    uint8_t *sfb = bimg + size_t(nkb) * kBImgPerKb;         // 512 bytes
    float *scratch = reinterpret_cast<float *>(sfb + 512);  // 64 floats
    __shared__ __align__(8) uint64_t full[32], empty[32], dfull[2], dempty[2];
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort, s_last;

    pdl_launch_dependents();

    const int G = int(gridDim.x), c = int(blockIdx.x);
    const int nmat = p.seg[0].nmat;
    const int my_tiles = c < p.total_tiles ? (p.total_tiles - c + G - 1) / G : 0;
    const int nruns = my_tiles * nmat;
    const int total_kb = nruns * nkb;

    if (tid == 0) {
        for (int i = 0; i < S; i++) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        for (int i = 0; i < 2; i++) { mbar_init(&dfull[i], 1); mbar_init(&dempty[i], 4); }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(kTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    __syncthreads();

    // weights do not depend on the previous kernel: start the stream before the dependency wait
    if (warp == 5 && lane == 0) {
        for (int i = 0; i < p.prefetch && i < total_kb; i++) {
            const int run = i / nkb, kb = i - run * nkb;
            const uint8_t *src = run_base(p, c + (run / nmat) * G, run % nmat) + size_t(kb) * kURec;
            mbar_expect_tx(&full[i], kURec);
            bulk_load(ring + size_t(i) * kURec, src, kURec, &full[i]);
        }
    }
    uint2 wpre[kPreVec];
    preload_norm_weights(p.pro, wpre);
    pdl_wait();

    // ---- activation prologue: fp32 vector -> 24-bit fixed point -> twelve E2M1 digit columns ---------
    float4 v[kMaxVec];
    load_activation(p.pro, 0, v);
    const float tmax = transform_activation(p.pro, 0, v, wpre, scratch);
    int eb = int((__float_as_uint(tmax) >> 23) & 0xffu);
    eb = min(max(eb, 24), 230);
    const float alpha = __uint_as_float(uint32_t(127 + 23 - (eb - 127)) << 23); // max * alpha in [2^23, 2^24)
    const float inv_alpha = __uint_as_float(uint32_t(eb - 23) << 23);
    {
        const int nvec = p.pro.cols >> 2;
#pragma unroll
        for (int j = 0; j < kMaxVec; j++) {
            const int i = tid + j * kUThreads;
            if (i < nvec) {
                uint32_t lo[4], hi[4];
                digit_codes(v[j].x, alpha, lo[0], hi[0]);
                digit_codes(v[j].y, alpha, lo[1], hi[1]);
                digit_codes(v[j].z, alpha, lo[2], hi[2]);
                digit_codes(v[j].w, alpha, lo[3], hi[3]);
                // 4 consecutive k -> 2 bytes per column; image: [kblock][2 steps][2 col groups][2 k cores][8 cols][16 B]
                const int k = i << 2, kb = k >> 7, kk = k & 127;
                uint8_t *base = bimg + size_t(kb) * kBImgPerKb + (kk >> 6) * 512 + (((kk & 63) >> 1) >> 4) * 128 + (((kk & 63) >> 1) & 15);
#pragma unroll
                for (int col = 0; col < 12; col++) {
                    const int sh = (col & 7) * 4;
                    const uint32_t *w = col < 8 ? lo : hi;
                    const uint32_t two = ((w[0] >> sh) & 0xFu) | (((w[1] >> sh) & 0xFu) << 4) | (((w[2] >> sh) & 0xFu) << 8) |
                                         (((w[3] >> sh) & 0xFu) << 12);
                    *reinterpret_cast<uint16_t *>(base + (col >> 3) * 256 + (col & 7) * 16) = uint16_t(two);
                }
#pragma unroll
                for (int col = 12; col < 16; col++) *reinterpret_cast<uint16_t *>(base + 256 + (col & 7) * 16) = 0;
            }
        }
        // column block scales: 4^j for the digit columns, 1 elsewhere; [32 rows][16 B], row = column, byte = (quarter, group)
        if (tid < 128) reinterpret_cast<uint32_t *>(sfb)[tid] = ((tid >> 2) < 12 && (tid & 3) == 0) ? 0x01010101u * uint32_t(127 + 2 * (tid >> 2)) : 0x7F7F7F7Fu;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    const uint32_t tmem = s_tmem;
    volatile int *abort_flag = &s_abort;

    if (warp == 5) {
        // ---- producer: refill a stage as soon as the MMAs that read it have retired ------------------
        if (lane == 0) {
            for (int i = p.prefetch; i < total_kb; i++) {
                const int st = i % S;
                if (i >= S && !mbar_wait(&empty[st], ((i / S) - 1) & 1, abort_flag)) break;
                const int run = i / nkb, kb = i - run * nkb;
                const uint8_t *src = run_base(p, c + (run / nmat) * G, run % nmat) + size_t(kb) * kURec;
                mbar_expect_tx(&full[st], kURec);
                bulk_load(ring + size_t(st) * kURec, src, kURec, &full[st]);
            }
        }
    } else if (warp == 4) {
        // ---- MMA issuer ------------------------------------------------------------------------------
        if (lane == 0) {
            const uint32_t idesc_base = (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24);
            asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem + 288), "l"(umma_desc(smem_u32(sfb), 16, 128)));
            int i = 0;
            bool ok = true;
            for (int run = 0; run < nruns && ok; run++) {
                const int buf = run & 1;
                ok = mbar_wait(&dempty[buf], ((run >> 1) & 1) ^ 1, abort_flag); // first use of each buffer passes at once
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int kb = 0; kb < nkb; kb++, i++) {
                    const int st = i % S;
                    ok = mbar_wait(&full[st], (i / S) & 1, abort_flag);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sbase = smem_u32(ring + size_t(st) * kURec);
                    const uint32_t t_sfa = tmem + 256 + 4 * (i % kSfaBufs);
                    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(t_sfa), "l"(umma_desc(sbase + 8192, 16, 128)));
                    const uint32_t bbase = smem_u32(bimg + size_t(kb) * kBImgPerKb);
#pragma unroll
                    for (int s = 0; s < 2; s++) {
                        const uint64_t da = umma_desc(sbase + s * 4096, 128, 256), db = umma_desc(bbase + s * 512, 128, 256);
                        const uint32_t idesc = idesc_base | (uint32_t(2 * s) << 29); // A scales: bytes 2s, 2s+1; B scales: byte 0 (all equal)
                        const int a = (2 * kb + s) % p.nacc;               // accumulator of this MMA
                        const uint32_t acc = (2 * kb + s) >= p.nacc ? 1u : 0u;  // its first use overwrites
                        asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %4, 0;\n"
                                     "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], q;\n}"
                                     ::"r"(tmem + 128 * buf + 16 * a), "l"(da), "l"(db), "r"(idesc), "r"(acc), "r"(t_sfa), "r"(tmem + 288)
                                     : "memory");
                    }
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&empty[st])) : "memory");
                }
                if (ok) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&dfull[buf])) : "memory");
            }
        }
    } else if (warp < 4) {
        // ---- epilogue: TMEM lane = row of the tile; 16 columns = 12 digit sums (already weighted by 4^j) ----
        float best = -3.402823466e38f;
        int best_idx = 0x7fffffff;
        float gate_val = 0.f;
        bool ok = true;
        for (int run = 0; run < nruns && ok; run++) {
            const int buf = run & 1;
            ok = mbar_wait(&dfull[buf], (run >> 1) & 1, abort_flag);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float y = 0.f;
            const int nused = min(p.nacc, 2 * nkb);
            for (int a = 0; a < nused; a++) { // fixed order: accumulator 0 first, least significant digit first
                uint32_t r[16];
                const uint32_t taddr = tmem + 128 * buf + 16 * a + (uint32_t(warp * 32) << 16);
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                               "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                             : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                float ya = 0.f;
#pragma unroll
                for (int j = 0; j < 12; j++) ya += __uint_as_float(r[j]);
                y += ya;
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&dempty[buf]);
            y *= inv_alpha;
            const int tile = c + (run / nmat) * G, mat = run % nmat;
            const USeg &s = p.seg[useg_of(p, tile)];
            const int row = (tile - s.tile_begin) * 128 + tid;
            if (row < s.rows) {
                float *out = s.out;
                switch (s.epilogue) {
                case INSG_EPI_STORE: out[row] = y; break;
                case INSG_EPI_RESIDUAL: out[row] = __ldcg(out + row) + y; break;
                case INSG_EPI_CONV_SILU: {
                    float *st = s.conv_state + size_t(row) * 3;
                    const uint2 wv = reinterpret_cast<const uint2 *>(s.conv_w)[row];
                    const float w0 = bf16_bits_to_float(wv.x & 0xffff), w1 = bf16_bits_to_float(wv.x >> 16);
                    const float w2 = bf16_bits_to_float(wv.y & 0xffff), w3 = bf16_bits_to_float(wv.y >> 16);
                    const float s0 = __ldcg(st), s1 = __ldcg(st + 1), s2 = __ldcg(st + 2);
                    const float z = fmaf(s0, w0, fmaf(s1, w1, fmaf(s2, w2, y * w3)));
                    st[0] = s1; st[1] = s2; st[2] = y;
                    out[row] = fast_silu(z);
                    break;
                }
                case INSG_EPI_BETA: out[row] = fast_sigmoid(y); break;
                case INSG_EPI_DECAY: {
                    const float z = y + bf16_bits_to_float(s.dt_bias[row]);
                    const float soft = z > 20.f ? z : log1pf(__expf(z));
                    out[row] = -__expf(s.A_log[row]) * soft;
                    break;
                }
                case INSG_EPI_SWIGLU:
                    if (mat == 0) gate_val = y;
                    else out[row] = fast_silu(gate_val) * y;
                    break;
                case INSG_EPI_LOGITS:
                    out[row] = y;
                    if (y > best || (y == best && row < best_idx)) { best = y; best_idx = row; }
                    break;
                default: break;
                }
            }
        }
        // per-warp arg-max candidates for the logits epilogue
        if (p.argmax_partial) {
#pragma unroll
            for (int mk = 16; mk; mk >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, mk);
                const int oi = __shfl_xor_sync(0xffffffffu, best_idx, mk);
                if (ov > best || (ov == best && oi < best_idx)) { best = ov; best_idx = oi; }
            }
            if (lane == 0) { scratch[32 + warp] = best; reinterpret_cast<int *>(scratch)[40 + warp] = best_idx; }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
    if (tid == 0 && s_abort && p.error_flag) *p.error_flag = 1;

    if (p.argmax_partial) {
        if (tid == 0) {
            float bv = scratch[32];
            int bi = reinterpret_cast<int *>(scratch)[40];
            for (int w = 1; w < 4; w++) {
                const float ov = scratch[32 + w];
                const int oi = reinterpret_cast<int *>(scratch)[40 + w];
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            p.argmax_partial[blockIdx.x] = make_float2(bv, __int_as_float(bi));
            __threadfence();
            const unsigned ticket = atomicAdd(p.argmax_ticket, 1u);
            s_last = (ticket == gridDim.x - 1);
        }
        __syncthreads();
        if (s_last && warp == 0) {
            __threadfence();
            float bv = -3.402823466e38f;
            int bi = 0x7fffffff;
            for (int i = lane; i < G; i += 32) {
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
            if (lane == 0) {
                *p.token_out = bi;
                if (p.token_feedback) *p.token_feedback = bi;
                if (p.position_inout) {
                    const int pos = *p.position_inout;
                    if (p.token_log && pos >= 0 && pos < p.token_log_capacity) p.token_log[pos] = bi;
                    *p.position_inout = pos + 1;
                }
                *p.argmax_ticket = 0u;
            }
        }
    }
}

// ---- repack: MLX layout -> shared-memory images ----------------------------------------------------
// One thread per (row of a tile, k-block): copies the row's 64 bytes into the four 16-byte cells of the
// record and its four scale bytes into the scale block.  Rows beyond `rows` are zero weights with scale 1.
__global__ void repack_umma_kernel(const uint32_t *__restrict__ w, const uint8_t *__restrict__ s, uint8_t *__restrict__ out, int rows,
                                   int cols)
{
    const int nkb = cols >> 7;
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const size_t ntiles = (size_t(rows) + 127) >> 7;
    if (idx >= ntiles * nkb * 128) return;
    const int r = int(idx & 127);
    const size_t rec_id = idx >> 7;
    const int kb = int(rec_id % nkb);
    const size_t tile = rec_id / nkb;
    const size_t row = tile * 128 + r;
    uint8_t *rec = out + rec_id * kURec;
    uint4 q[4] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    uint32_t sc = 0x7F7F7F7Fu;
    if (row < size_t(rows)) {
        const uint4 *src = reinterpret_cast<const uint4 *>(w + row * (cols >> 3) + kb * 16);
#pragma unroll
        for (int i = 0; i < 4; i++) q[i] = src[i];
        sc = *reinterpret_cast<const uint32_t *>(s + row * (cols >> 5) + kb * 4);
    }
    // 64 bytes of the row = 2 K-steps x 2 k-cores of 16 bytes
#pragma unroll
    for (int i = 0; i < 4; i++) *reinterpret_cast<uint4 *>(rec + (i >> 1) * 4096 + (r >> 3) * 256 + (i & 1) * 128 + (r & 7) * 16) = q[i];
    *reinterpret_cast<uint32_t *>(rec + 8192 + (r & 31) * 16 + (r >> 5) * 4) = sc;
}

namespace {
// fixed launch shape (measured best; no process-wide knobs: engines and threads share this library)
constexpr int kUStages = 16, kUNacc = 8, kUPrefetch = 8;

std::mutex g_attr_mutex;
bool g_attr_done[64] = {false}; // the shared-memory opt-in is a per-device function attribute
} // namespace


int gemv_umma_launch(const insg_gemv_op *op, cudaStream_t st)
{
    if (!op || !op->in) return fail(INSG_E_ARG, "gemv: null operand");
    if (op->cols <= 0 || (op->cols & 127) || op->cols > kMaxVec * kUThreads * 4) return fail(INSG_E_SHAPE, "gemv: cols must be a multiple of 128, <= 12288");
    if (op->n_segments < 1 || op->n_segments > 4) return fail(INSG_E_SHAPE, "gemv: 1..4 segments");
    if ((op->prologue == INSG_PRO_RMSNORM || op->prologue == INSG_PRO_GATED_RMSNORM) && !op->norm_w) return fail(INSG_E_ARG, "gemv: norm weight missing");
    if (op->prologue >= INSG_PRO_GATED_RMSNORM && !op->aux) return fail(INSG_E_ARG, "gemv: prologue operand missing");
    UParams p = {};
    p.pro = ProIn{op->in, op->aux, op->norm_w, op->x_out, op->cols, op->prologue};
    p.nkb = op->cols >> 7;
    p.nseg = op->n_segments;
    int tiles = 0, nmat_all = 0;
    bool logits = false;
    for (int i = 0; i < op->n_segments; i++) {
        const insg_gemv_segment &s = op->seg[i];
        if (!s.packed || !s.out || s.rows <= 0) return fail(INSG_E_SHAPE, "gemv: bad segment");
        if (s.epilogue == INSG_EPI_SWIGLU && !s.packed2) return fail(INSG_E_ARG, "gemv: SwiGLU needs two matrices");
        if (s.epilogue == INSG_EPI_CONV_SILU && (!s.conv_state || !s.conv_w)) return fail(INSG_E_ARG, "gemv: conv operands missing");
        if (s.epilogue == INSG_EPI_DECAY && (!s.A_log || !s.dt_bias)) return fail(INSG_E_ARG, "gemv: decay operands missing");
        USeg &d = p.seg[i];
        d.packed = static_cast<const uint8_t *>(s.packed);
        d.packed2 = static_cast<const uint8_t *>(s.packed2);
        d.out = s.out; d.conv_state = s.conv_state; d.conv_w = s.conv_w; d.A_log = s.A_log; d.dt_bias = s.dt_bias;
        d.nmat = s.epilogue == INSG_EPI_SWIGLU ? 2 : 1;
        if (nmat_all && nmat_all != d.nmat) return fail(INSG_E_SHAPE, "gemv: SwiGLU segments cannot be mixed with others");
        nmat_all = d.nmat;
        d.tile_begin = tiles; d.ntiles = (s.rows + 127) >> 7; tiles += d.ntiles; d.epilogue = s.epilogue; d.rows = s.rows;
        logits |= s.epilogue == INSG_EPI_LOGITS;
    }
    p.total_tiles = tiles;
    const int grid = std::max(1, std::min(std::min(sm_count(), 256), tiles));
    if (logits) {
        if (op->n_segments != 1) return fail(INSG_E_SHAPE, "gemv: the logits epilogue takes one segment");
        if (!op->argmax_scratch || !op->token_out) return fail(INSG_E_ARG, "gemv: arg-max scratch/token missing");
        p.argmax_ticket = static_cast<unsigned *>(op->argmax_scratch);
        p.argmax_partial = reinterpret_cast<float2 *>(static_cast<uint8_t *>(op->argmax_scratch) + 64);
        p.token_out = op->token_out; p.token_feedback = op->token_feedback; p.token_log = op->token_log; p.position_inout = op->position_inout;
        p.token_log_capacity = op->token_log_capacity;
        if (op->token_log && op->token_log_capacity <= 0) return fail(INSG_E_ARG, "gemv: token_log needs its capacity");
    }
    p.error_flag = static_cast<int *>(op->error_flag);
    const size_t fixed = size_t(p.nkb) * kBImgPerKb + 512 + 64 * 4 + 1024;
    int stages = std::min(kUStages, int((size_t(220) * 1024 - fixed) / kURec));
    stages = std::max(2, std::min(stages, 24));
    p.stages = stages;
    p.nacc = kUNacc;
    p.prefetch = std::min(kUPrefetch, stages);
    const size_t smem = size_t(stages) * kURec + fixed;
    {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
        if (dev < 0 || dev >= 64) return fail(INSG_E_LIMIT, "gemv: device ordinal beyond 63");
        std::lock_guard<std::mutex> lock(g_attr_mutex);
        if (!g_attr_done[dev]) {
            e = cudaFuncSetAttribute(umma_gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
            if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(umma gemv)");
            g_attr_done[dev] = true;
        }
    }
    return launch(umma_gemv_kernel, dim3(grid), dim3(kUThreads), smem, st, op->pdl != 0, p);
}

} // namespace insg

using namespace insg;

extern "C" {

size_t insg_mxfp4_packed_umma_bytes(int rows, int cols)
{
    if (rows <= 0 || cols <= 0 || (cols & 127)) return 0;
    return size_t((rows + 127) >> 7) * (cols >> 7) * kURec;
}

int insg_mxfp4_repack_umma(const uint32_t *weight, const uint8_t *scales, void *packed, int rows, int cols, insg_stream_t stream)
{
    if (!weight || !scales || !packed) return fail(INSG_E_ARG, "repack_umma: null pointer");
    if (rows <= 0 || cols <= 0 || (cols & 127)) return fail(INSG_E_SHAPE, "repack_umma: cols % 128 must be 0");
    const size_t n = size_t((rows + 127) >> 7) * (cols >> 7) * 128;
    repack_umma_kernel<<<unsigned((n + 255) / 256), 256, 0, stream>>>(weight, scales, static_cast<uint8_t *>(packed), rows, cols);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? INSG_OK : cuda_fail(e, "repack_umma launch");
}

} // extern "C"
