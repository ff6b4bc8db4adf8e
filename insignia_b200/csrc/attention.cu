// Split-K flash-decode GQA for sm_100a: 16 query heads over 4 kv heads, head_dim 256.
//
// Math (reference: src/attention.cu:4): score_t = (q_h . K[t][h>>2]) / 16, softmax over
// the cached tokens, out_h = sum_t p_t V[t][h>>2]; cache layout [token][4][256].
//
// The reference runs one CTA per query head, keeps every score in shared memory
// (which fails past ~12K tokens) and re-reads each kv head's cache four times.
// Here a CTA owns (kv head, token range): it streams its slab of K and V exactly
// once for the four query heads that share the kv head, keeps an online softmax
// per warp, and leaves (max, denominator, weighted V) partials in scratch; the
// last CTA to finish for a kv head folds the partials in split order, so results
// do not depend on scheduling.  The fused entry also does the per-head RMSNorm,
// partial RoPE and the cache write of the current token (src/ops.cu:9,
// src/qwen_kernels.cu:15,31) so one launch replaces five.
//
// bf16 cache, long contexts: the scalar loop is bound by instruction issue (half the bytes, the same instructions),
// so from kMmaMinTokens cached rows on the warps score and accumulate on the tensor cores instead (mma.sync
// m16n8k16 bf16, fp32 accumulation): 16 cached rows per step per warp, fetched into the warp's own shared-memory tile
// by one cp.async.bulk per lane (16 key rows + 16 value rows, mbarrier completion, bounded wait); the fp32 query goes in
// as two bf16 pieces (hi + lo) in the eight N columns (4 heads x 2 pieces), the softmax weights likewise for P.V, so
// products keep ~16 bits of the fp32 operands and the cache values are exact.
#include "attention_body.cuh"
#include "host_util.h"
#include "umma_common.cuh"

#include <algorithm>
#include <mutex>

namespace insg {

constexpr int kAtThreads = 256;
constexpr int kAtWarps = 8;
constexpr int kGroup = 4;                    // tokens a warp scores at once
constexpr int kMinChunk = kAtWarps * kGroup; // tokens per split at least: one group per warp
constexpr int kMmaMinTokens = 2048;          // bf16 cache: cached rows from which the tensor-core loop is used
constexpr int kTileRow = 528;                // a staged row: 512 bytes of bf16 + 16 of padding (conflict-free ldmatrix)
constexpr int kTileBytes = 16 * kTileRow;    // 16 rows
constexpr size_t kMmaSmem = size_t(kAtWarps) * 2 * kTileBytes; // per warp: a key tile and a value tile

__device__ __forceinline__ uint32_t bf16_piece_pair(float a, float b, int piece)
{
    // piece 0: the bf16 roundings of a and b; piece 1: the bf16 roundings of what those left over
    __nv_bfloat16 ha = __float2bfloat16_rn(a), hb = __float2bfloat16_rn(b);
    if (piece) {
        ha = __float2bfloat16_rn(a - __bfloat162float(ha));
        hb = __float2bfloat16_rn(b - __bfloat162float(hb));
    }
    return uint32_t(__bfloat16_as_ushort(ha)) | (uint32_t(__bfloat16_as_ushort(hb)) << 16);
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One warp's share of a split on the tensor cores: rows t0 + 16 (warp + 8 n) .. of [t0, t1), bf16 cache.  Leaves the
// warp's (max, denominator, weighted values) in s_m_w / s_l_w / s_acc_w like the scalar loop does.
__device__ __forceinline__ void attn_mma_warp(const void *kc, const void *vc, int kvh, int t0, int t1, int warp, int lane,
                                              const float (*s_q)[256], uint8_t *tiles, uint64_t *bar, volatile int *abort_flag,
                                              float *s_m_w, float *s_l_w, float (*s_acc_w)[256])
{
    const int g = lane >> 2, t = lane & 3;
    uint8_t *tile_k = tiles + size_t(warp) * 2 * kTileBytes, *tile_v = tile_k + kTileBytes;
    if (lane == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    // the query as the B operand: column g = (head g >> 1, piece g & 1), k rows 2t, 2t+1 and 2t+8, 2t+9 of every 16 dims
    uint32_t qb[16][2];
    {
        const float *qh = s_q[g >> 1];
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int d = 16 * i + 2 * t;
            qb[i][0] = bf16_piece_pair(qh[d] * 0.0625f, qh[d + 1] * 0.0625f, g & 1);
            qb[i][1] = bf16_piece_pair(qh[d + 8] * 0.0625f, qh[d + 9] * 0.0625f, g & 1);
        }
    }
    float m_run = -3.0e38f, l_run = 0.f; // of head t (the same in the eight lanes that share t, l_run as a partial sum)
    float acc[16][4];                    // [16 dims each][dim g: (hi, lo) of head t | dim g + 8: (hi, lo)]
#pragma unroll
    for (int j = 0; j < 16; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    uint32_t phase = 0;
    const uint32_t lm_row = uint32_t(lane & 7), lm_id = uint32_t(lane >> 3);
    const uint32_t k_addr = smem_u32(tile_k) + ((lm_id & 1) * 8 + lm_row) * kTileRow + (lm_id >> 1) * 16; // + 32 i: rows of K as m, dims as k
    const uint32_t v_addr = smem_u32(tile_v) + ((lm_id >> 1) * 8 + lm_row) * kTileRow + (lm_id & 1) * 16; // + 32 j: transposed: dims as m, rows as k
    for (int tb = t0 + 16 * warp; tb < t1; tb += 16 * kAtWarps) {
        __syncwarp();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // the tile was read by ordinary loads; the copies below overwrite it
        if (lane == 0) mbar_expect_tx(bar, 32 * 512);
        __syncwarp();
        {
            const int r = lane & 15, tok = min(tb + r, t1 - 1); // rows past the split repeat its last row: masked below
            const uint8_t *src = static_cast<const uint8_t *>(lane < 16 ? kc : vc) + (size_t(tok) * 4 + kvh) * 512;
            bulk_load((lane < 16 ? tile_k : tile_v) + r * kTileRow, src, 512, bar);
        }
        if (!mbar_wait(bar, phase, abort_flag)) break;
        phase ^= 1u;
        // ---- scores: S[16 rows][8 columns] = K tile . q pieces ----
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 16; i++) {
            uint32_t a0, a1, a2, a3;
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "r"(k_addr + 32 * i));
            mma_bf16(c, a0, a1, a2, a3, qb[i][0], qb[i][1]);
        }
        const bool v0 = tb + g < t1, v1 = tb + g + 8 < t1;
        const float s0 = v0 ? c[0] + c[1] : -3.0e38f, s1 = v1 ? c[2] + c[3] : -3.0e38f; // rows tb + g and tb + g + 8, head t
        float mx = fmaxf(s0, s1);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
        const float m_new = fmaxf(m_run, mx), corr = __expf(m_run - m_new);
        const float p0 = v0 ? __expf(s0 - m_new) : 0.f, p1 = v1 ? __expf(s1 - m_new) : 0.f;
        l_run = fmaf(l_run, corr, p0 + p1);
        m_run = m_new;
#pragma unroll
        for (int j = 0; j < 16; j++) { acc[j][0] *= corr; acc[j][1] *= corr; acc[j][2] *= corr; acc[j][3] *= corr; }
        // ---- the weights as the B operand of P.V: column g = (head g >> 1, piece g & 1), k rows = cached rows ----
        const int src_a = 8 * t + (g >> 1), src_b = src_a + 4; // lanes that hold rows 2t and 2t + 1 (and + 8) of that head
        const float x0 = __shfl_sync(0xffffffffu, p0, src_a), x1 = __shfl_sync(0xffffffffu, p0, src_b);
        const float y0 = __shfl_sync(0xffffffffu, p1, src_a), y1 = __shfl_sync(0xffffffffu, p1, src_b);
        const uint32_t pb0 = bf16_piece_pair(x0, x1, g & 1), pb1 = bf16_piece_pair(y0, y1, g & 1);
#pragma unroll
        for (int j = 0; j < 16; j++) {
            uint32_t a0, a1, a2, a3;
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "r"(v_addr + 32 * j));
            mma_bf16(acc[j], a0, a1, a2, a3, pb0, pb1);
        }
    }
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 4);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 8);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 16);
    if (g == 0) { s_m_w[t] = m_run; s_l_w[t] = l_run; }
#pragma unroll
    for (int j = 0; j < 16; j++) {
        s_acc_w[t][16 * j + g] = acc[j][0] + acc[j][1];
        s_acc_w[t][16 * j + g + 8] = acc[j][2] + acc[j][3];
    }
}

template <bool BF16, bool FUSED> __global__ void __launch_bounds__(kAtThreads) attn_splitk_kernel(const __grid_constant__ AttnParams p)
{
    using Row = KvRow<BF16>;
    __shared__ __align__(16) float s_q[4][256];
    __shared__ __align__(16) float s_knew[256], s_vnew[256];
    __shared__ float s_m[kAtWarps][4], s_l[kAtWarps][4];
    __shared__ __align__(16) float s_acc[kAtWarps][4][256];
    __shared__ int s_last;
    __shared__ float s_e[64][4], s_lg[4];
    __shared__ __align__(8) uint64_t s_bar[kAtWarps];
    __shared__ int s_abort;
    extern __shared__ __align__(128) uint8_t s_tiles[]; // bf16 cache only: per warp a key tile and a value tile

    const int ns = int(gridDim.x) >> 2; // splits launched per kv head (37, or fewer when the host knows the context is short)
    const int kvh = blockIdx.x / ns, split = blockIdx.x % ns;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // token of a chunk (plain form only; a single launch has blockIdx.y == 0 and zero strides)
    const int bt = blockIdx.y;
    const float *q_in = p.q + size_t(bt) * p.q_stride;
    float *out_base = p.out + size_t(bt) * p.out_stride;
    unsigned *counters = reinterpret_cast<unsigned *>(reinterpret_cast<uint8_t *>(p.counters) + size_t(bt) * p.scratch_stride);
    float *partials = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(p.partials) + size_t(bt) * p.scratch_stride);
    void *kc = static_cast<uint8_t *>(p.kc) + size_t(bt) * p.cache_stride, *vc = static_cast<uint8_t *>(p.vc) + size_t(bt) * p.cache_stride;
    const float *k_raw = p.k_raw + size_t(bt) * p.kvin_stride, *v_new = p.v_new + size_t(bt) * p.kvin_stride;

    pdl_launch_dependents();

    // Geometry from the position as it is visible now.  Cache rows of earlier tokens never change
    // again, so the first token group of every warp is fetched while the producer of q still runs;
    // the position is read again after the wait and the fetch repeated if it moved.
    int pos = -1, tokens = p.tokens;
    if constexpr (FUSED) {
        pos = __ldcg(p.position) + p.position_offset;
        tokens = pos + 1;
    } else if (p.position) { // chunk: the rows were written by the launch before this one (plain stream order)
        tokens = __ldcg(p.position) + p.position_offset + bt + 1;
    }
    tokens = max(1, min(tokens, p.max_context)); // host checks; never index past the cache
    int chunk = max(kMinChunk, (tokens + kSplits - 1) / kSplits);
    int nsplit = (tokens + chunk - 1) / chunk;
    int t0 = split * chunk, t1 = min(tokens, t0 + chunk);
    int fresh = tokens - 1; // the row the producer (or this kernel) is still writing

    bool use_mma = BF16 && tokens >= kMmaMinTokens; // long bf16 contexts: the tensor-core loop (reads every row from the cache)
    if (tid == 0) s_abort = 0;
    GroupRaw<BF16, kGroup> ga, gb; // this warp's next two token groups, in flight while it works on earlier ones
    if (!use_mma) {
        load_group<BF16, kGroup>(kc, vc, kvh, t0 + warp * kGroup, min(t1, fresh), lane, ga);
        load_group<BF16, kGroup>(kc, vc, kvh, t0 + (warp + kAtWarps) * kGroup, min(t1, fresh), lane, gb);
    }
    uint4 norm_wv = make_uint4(0u, 0u, 0u, 0u);
    float rope_c[8], rope_s[8];
    if constexpr (FUSED) {
        if (warp < 5) {
            norm_wv = reinterpret_cast<const uint4 *>(warp < 4 ? p.q_w : p.k_w)[lane];
            if (lane < 8) rope_table(pos, lane, p.fast_trig != 0, rope_c, rope_s);
        }
    }

    pdl_wait();

    if constexpr (FUSED) {
        const int now = __ldcg(p.position) + p.position_offset;
        if (now != pos) {
            pos = now;
            tokens = max(1, min(pos + 1, p.max_context));
            chunk = max(kMinChunk, (tokens + kSplits - 1) / kSplits);
            nsplit = (tokens + chunk - 1) / chunk;
            t0 = split * chunk;
            t1 = min(tokens, t0 + chunk);
            fresh = tokens - 1;
            use_mma = BF16 && tokens >= kMmaMinTokens;
            if (!use_mma) {
                load_group<BF16, kGroup>(kc, vc, kvh, t0 + warp * kGroup, min(t1, fresh), lane, ga);
                load_group<BF16, kGroup>(kc, vc, kvh, t0 + (warp + kAtWarps) * kGroup, min(t1, fresh), lane, gb);
            }
            if (warp < 5 && lane < 8) rope_table(pos, lane, p.fast_trig != 0, rope_c, rope_s);
        }
    }
    const bool has_work = t0 < tokens;
    if (nsplit > ns && tid == 0 && p.error_flag) *p.error_flag = 1; // the host's hint was too small: rows would be left out

    if (has_work) {
        // ---- query (and current key) preparation --------------------------------
        if constexpr (FUSED) {
            if (warp < 4) {
                float v[8];
                const float4 *src = reinterpret_cast<const float4 *>(q_in + size_t(kvh * 4 + warp) * 512 + lane * 8);
                const float4 a = __ldcg(src), b = __ldcg(src + 1);
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
                norm_rope_256(v, norm_wv, lane, pos, rope_c, rope_s);
#pragma unroll
                for (int j = 0; j < 8; j++) s_q[warp][lane * 8 + j] = v[j];
            } else if (warp == 4 && pos >= t0 && pos < t1) {
                float v[8];
                const float4 *src = reinterpret_cast<const float4 *>(k_raw + kvh * 256 + lane * 8);
                const float4 a = __ldcg(src), b = __ldcg(src + 1);
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
                norm_rope_256(v, norm_wv, lane, pos, rope_c, rope_s);
                const size_t row = (size_t(pos) * 4 + kvh) * 256 + lane * 8;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    Row::store(kc, row + j, v[j]);
                    s_knew[lane * 8 + j] = Row::round(v[j]);
                }
                if (use_mma) asm volatile("fence.proxy.async;" ::: "memory"); // the tensor-core loop fetches this row by bulk copy
            } else if (warp == 5 && pos >= t0 && pos < t1) {
                const size_t row = (size_t(pos) * 4 + kvh) * 256 + lane * 8;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const float v = __ldcg(v_new + kvh * 256 + lane * 8 + j);
                    Row::store(vc, row + j, v);
                    s_vnew[lane * 8 + j] = Row::round(v);
                }
                if (use_mma) asm volatile("fence.proxy.async;" ::: "memory");
            }
        } else {
            for (int i = tid; i < 1024; i += kAtThreads) s_q[i >> 8][i & 255] = __ldcg(q_in + size_t(kvh) * 1024 + i);
        }
    }
    __syncthreads();

    bool mma_done = false;
    if constexpr (BF16) {
        if (has_work && use_mma) {
            attn_mma_warp(kc, vc, kvh, t0, t1, warp, lane, s_q, s_tiles, &s_bar[warp], &s_abort, s_m[warp], s_l[warp], s_acc[warp]);
            mma_done = true;
        }
    }
    if (has_work && !mma_done) {
        float q[4][8];
#pragma unroll
        for (int h = 0; h < 4; h++)
#pragma unroll
            for (int j = 0; j < 8; j++) q[h][j] = s_q[h][lane * 8 + j] * 0.0625f;

        float m[4], l[4], acc[4][8];
#pragma unroll
        for (int h = 0; h < 4; h++) {
            m[h] = -3.0e38f;
            l[h] = 0.f;
#pragma unroll
            for (int j = 0; j < 8; j++) acc[h][j] = 0.f;
        }
        // one token group: scores of its (up to) four tokens for the four query heads, one online-softmax update
        auto process = [&](const GroupRaw<BF16, kGroup> &grp, int tb) {
            float kk[kGroup][8];
#pragma unroll
            for (int g = 0; g < kGroup; g++) Row::unpack(grp.k[g], kk[g]);
            const bool has_fresh = fresh >= tb && fresh < tb + kGroup && fresh < t1; // warp-uniform
            typename Row::Raw vfresh = Row::zero();
            if (has_fresh) { // the newest row: from shared memory or, now that the wait is over, from the cache
#pragma unroll
                for (int g = 0; g < kGroup; g++) {
                    if (tb + g != fresh) continue;
                    if constexpr (FUSED) {
#pragma unroll
                        for (int j = 0; j < 8; j++) kk[g][j] = s_knew[lane * 8 + j];
                    } else {
                        const size_t row = (size_t(fresh) * 4 + kvh) * 256;
                        Row::unpack(Row::load_raw(kc, row, lane), kk[g]);
                        vfresh = Row::load_raw(vc, row, lane);
                    }
                }
            }
            float s[kGroup][4];
#pragma unroll
            for (int g = 0; g < kGroup; g++)
#pragma unroll
                for (int h = 0; h < 4; h++) {
                    float z = 0.f;
#pragma unroll
                    for (int j = 0; j < 8; j++) z = fmaf(q[h][j], kk[g][j], z);
                    s[g][h] = z;
                }
#pragma unroll
            for (int mk = 16; mk; mk >>= 1)
#pragma unroll
                for (int g = 0; g < kGroup; g++)
#pragma unroll
                    for (int h = 0; h < 4; h++) s[g][h] += __shfl_xor_sync(0xffffffffu, s[g][h], mk);
            float pr[kGroup][4], corr[4];
#pragma unroll
            for (int h = 0; h < 4; h++) {
                float mn = m[h];
#pragma unroll
                for (int g = 0; g < kGroup; g++)
                    if (tb + g < t1) mn = fmaxf(mn, s[g][h]);
                corr[h] = __expf(m[h] - mn);
                float psum = 0.f;
#pragma unroll
                for (int g = 0; g < kGroup; g++) {
                    pr[g][h] = tb + g < t1 ? __expf(s[g][h] - mn) : 0.f;
                    psum += pr[g][h];
                }
                m[h] = mn;
                l[h] = fmaf(l[h], corr[h], psum);
#pragma unroll
                for (int j = 0; j < 8; j++) acc[h][j] *= corr[h];
            }
#pragma unroll
            for (int g = 0; g < kGroup; g++) {
                float vv[8];
                Row::unpack(grp.v[g], vv);
                if (has_fresh && tb + g == fresh) {
                    if constexpr (FUSED) {
#pragma unroll
                        for (int j = 0; j < 8; j++) vv[j] = s_vnew[lane * 8 + j];
                    } else {
                        Row::unpack(vfresh, vv);
                    }
                }
#pragma unroll
                for (int h = 0; h < 4; h++)
#pragma unroll
                    for (int j = 0; j < 8; j++) acc[h][j] = fmaf(pr[g][h], vv[j], acc[h][j]);
            }
        };
        const int tend = min(t1, fresh);
        for (int tb = t0 + warp * kGroup; tb < t1; tb += 2 * kAtWarps * kGroup) {
            process(ga, tb);
            load_group<BF16, kGroup>(kc, vc, kvh, tb + 2 * kAtWarps * kGroup, tend, lane, ga);
            const int tb2 = tb + kAtWarps * kGroup;
            if (tb2 < t1) {
                process(gb, tb2);
                load_group<BF16, kGroup>(kc, vc, kvh, tb2 + 2 * kAtWarps * kGroup, tend, lane, gb);
            }
        }
        // ---- fold the 8 warps --------------------------------------------------------
#pragma unroll
        for (int h = 0; h < 4; h++) {
            if (lane == 0) { s_m[warp][h] = m[h]; s_l[warp][h] = l[h]; }
#pragma unroll
            for (int j = 0; j < 8; j++) s_acc[warp][h][lane * 8 + j] = acc[h][j];
        }
    }
    __syncthreads();
    float *part = partials + size_t(kvh * kSplits + split) * kPartFloats;
    if (has_work) {
        const int d = tid;
#pragma unroll
        for (int h = 0; h < 4; h++) {
            float mg = s_m[0][h];
#pragma unroll
            for (int w = 1; w < kAtWarps; w++) mg = fmaxf(mg, s_m[w][h]);
            float lg = 0.f, a = 0.f;
#pragma unroll
            for (int w = 0; w < kAtWarps; w++) {
                const float e = __expf(s_m[w][h] - mg); // warps without tokens carry m=-3e38, l=0, acc=0
                lg = fmaf(s_l[w][h], e, lg);
                a = fmaf(s_acc[w][h][d], e, a);
            }
            part[8 + h * 256 + d] = a;
            if (d == 0) { part[h] = mg; part[4 + h] = lg; }
        }
    }
    // ---- last CTA of this kv head folds the splits -----------------------------------
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned ticket = atomicAdd(counters + kvh, 1u);
        s_last = (ticket == unsigned(ns) - 1u);
    }
    __syncthreads();
    if (s_last) {
        __threadfence();
        const float *pp = partials + size_t(kvh * kSplits) * kPartFloats;
        // weights of the splits: warp h takes query head h, a lane takes splits lane and lane+32
        if (warp < 4) {
            const int h = warp, sa = lane, sb = lane + 32;
            const float ma = sa < nsplit ? __ldcg(pp + size_t(sa) * kPartFloats + h) : -3.0e38f;
            const float mb = sb < nsplit ? __ldcg(pp + size_t(sb) * kPartFloats + h) : -3.0e38f;
            const float la = sa < nsplit ? __ldcg(pp + size_t(sa) * kPartFloats + 4 + h) : 0.f;
            const float lb = sb < nsplit ? __ldcg(pp + size_t(sb) * kPartFloats + 4 + h) : 0.f;
            const float mg = warp_max(fmaxf(ma, mb));
            const float ea = sa < nsplit ? __expf(ma - mg) : 0.f, eb = sb < nsplit ? __expf(mb - mg) : 0.f;
            const float lg = warp_sum(fmaf(la, ea, lb * eb));
            s_e[sa][h] = ea;
            if (sb < kSplits) s_e[sb][h] = eb;
            if (lane == 0) s_lg[h] = lg;
        }
        __syncthreads();
        // a thread owns four output dims of one head; the loads of different splits are independent
        const int h = tid >> 6, c4 = tid & 63;
        const float4 *src = reinterpret_cast<const float4 *>(pp + 8 + h * 256) + c4;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
        for (int s = 0; s < nsplit; s++) {
            const float4 v = __ldcg(src + size_t(s) * (kPartFloats / 4));
            const float e = s_e[s][h];
            a.x = fmaf(v.x, e, a.x);
            a.y = fmaf(v.y, e, a.y);
            a.z = fmaf(v.z, e, a.z);
            a.w = fmaf(v.w, e, a.w);
        }
        const float inv = 1.0f / s_lg[h];
        reinterpret_cast<float4 *>(out_base + size_t(kvh * 4 + h) * 256)[c4] = make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
        if (tid == 0) counters[kvh] = 0u;
    }
    if (tid == 0 && s_abort && p.error_flag) *p.error_flag = 1;
}

template <bool BF16, bool FUSED> int launch_attn(const AttnParams &p, cudaStream_t st, bool pdl, int chunk_tokens = 1, int splits = kSplits)
{
    size_t smem = 0;
    if (BF16) { // the tensor-core loop's tiles: more than 48 KB of dynamic shared memory is a per-device opt-in
        static std::mutex mu;
        static bool done[64] = {false};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
        if (dev < 0 || dev >= 64) return fail(INSG_E_LIMIT, "attention: device ordinal beyond 63");
        std::lock_guard<std::mutex> lock(mu);
        if (!done[dev]) {
            e = cudaFuncSetAttribute(attn_splitk_kernel<BF16, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kMmaSmem));
            if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(attention)");
            done[dev] = true;
        }
        smem = kMmaSmem;
    }
    return launch(attn_splitk_kernel<BF16, FUSED>, dim3(4 * splits, chunk_tokens), dim3(kAtThreads), smem, st, pdl, p);
}

// A chunk of consecutive tokens, step one: per token m (one CTA each) the per-head RMSNorm + partial RoPE of the 16 query
// heads (into qn[m][16][256]) and of the 4 key heads, and the token's key and value rows written to the cache at row
// position + offset + m.  Warp tasks 0..15 = query heads, 16..19 = key heads, 20..23 = value heads.
// (reference: split_q_gate + qwen35_qk_norm_rope_gate + store_kv, src/qwen_kernels.cu:15,31 and src/ops.cu:9, once per token)
template <bool BF16> __global__ void __launch_bounds__(kAtThreads) attn_chunk_prepare_kernel(const __grid_constant__ AttnParams p, float *qn)
{
    using Row = KvRow<BF16>;
    const int m = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = __ldcg(p.position) + p.position_offset + m;
    if (pos < 0 || pos >= p.max_context) return; // host checks; never index past the cache
    float rope_c[8], rope_s[8];
    if (lane < 8) rope_table(pos, lane, p.fast_trig != 0, rope_c, rope_s);
    for (int task = warp; task < 24; task += kAtWarps) {
        if (task < 20) {
            const bool is_q = task < 16;
            const int h = is_q ? task : task - 16;
            const float *src = is_q ? p.q + size_t(m) * 8192 + size_t(h) * 512 + lane * 8 : p.k_raw + size_t(m) * 1024 + h * 256 + lane * 8;
            const float4 a = __ldcg(reinterpret_cast<const float4 *>(src)), b = __ldcg(reinterpret_cast<const float4 *>(src) + 1);
            float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            norm_rope_256(v, reinterpret_cast<const uint4 *>(is_q ? p.q_w : p.k_w)[lane], lane, pos, rope_c, rope_s);
            if (is_q) {
                float4 *dst = reinterpret_cast<float4 *>(qn + size_t(m) * 4096 + h * 256 + lane * 8);
                dst[0] = make_float4(v[0], v[1], v[2], v[3]);
                dst[1] = make_float4(v[4], v[5], v[6], v[7]);
            } else {
                const size_t row = (size_t(pos) * 4 + h) * 256 + lane * 8;
#pragma unroll
                for (int j = 0; j < 8; j++) Row::store(p.kc, row + j, v[j]);
            }
        } else {
            const int h = task - 20;
            const size_t row = (size_t(pos) * 4 + h) * 256 + lane * 8;
#pragma unroll
            for (int j = 0; j < 8; j++) Row::store(p.vc, row + j, __ldcg(p.v_new + size_t(m) * 1024 + h * 256 + lane * 8 + j));
        }
    }
}

size_t attn_scratch_bytes() { return 64 + size_t(4) * kSplits * kPartFloats * sizeof(float); }

int attn_plain_launch(const float *q, const void *kc, const void *vc, float *out, int tokens, int kv_dtype, void *scratch,
                      cudaStream_t st)
{
    AttnParams p = {};
    p.q = q; p.kc = const_cast<void *>(kc); p.vc = const_cast<void *>(vc); p.out = out;
    p.tokens = tokens; p.max_context = tokens;
    p.counters = static_cast<unsigned *>(scratch);
    p.partials = reinterpret_cast<float *>(static_cast<uint8_t *>(scratch) + 64);
    return kv_dtype == INSG_KV_BF16 ? launch_attn<true, false>(p, st, false) : launch_attn<false, false>(p, st, false);
}

// ---- allocation-free variant -----------------------------------------------------
// Scratch for insg_gqa_decode_noalloc: lives in the library image, one copy per GPU that loads it
// (about 600 KB, held until the process exits).  In host code the symbol name is only a handle, so
// the device address is looked up once per device with cudaGetSymbolAddress and handed to the kernel.
constexpr int kNoAllocMaxTokens = 262144; // the model's longest context
constexpr size_t kNoAllocScratchBytes = 64 + size_t(4) * kSplits * kPartFloats * sizeof(float);
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// Device address of the static scratch on the current device.  Looked up on every call: the lookup allocates nothing,
// and an address cached across calls would dangle after the application resets the device or its primary context.
static int noalloc_scratch(void **out)
{
    void *p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static attention scratch)");
    *out = p;
    return INSG_OK;
}

} // namespace insg

using namespace insg;

extern "C" {

int insg_gqa_decode_noalloc(const float *q, const void *k_cache, const void *v_cache, float *out, int tokens, int kv_dtype,
                            insg_stream_t stream)
{
    if (tokens <= 0) return INSG_OK;
    if (tokens > kNoAllocMaxTokens) return fail(INSG_E_LIMIT, "gqa_decode_noalloc: more than 262144 cached tokens");
    if (!q || !k_cache || !v_cache || !out) return fail(INSG_E_ARG, "gqa_decode_noalloc: null pointer");
    if (kv_dtype != INSG_KV_F32 && kv_dtype != INSG_KV_BF16) return fail(INSG_E_ARG, "gqa_decode_noalloc: bad kv dtype");
    void *scratch = nullptr;
    const int rc = noalloc_scratch(&scratch);
    if (rc != INSG_OK) return rc;
    // the per-kv-head arrival counters must start at zero; an earlier call that was cut short could have left them set
    cudaError_t e = cudaMemsetAsync(scratch, 0, 64, stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(static attention scratch)");
    return attn_plain_launch(q, k_cache, v_cache, out, tokens, kv_dtype, scratch, stream);
}

size_t insg_gqa_scratch_bytes(int tokens)
{
    (void)tokens; // the split count is fixed, so the scratch does not grow with the context
    return attn_scratch_bytes();
}

int insg_gqa_decode(const float *q, const void *k_cache, const void *v_cache, float *out, int tokens, int kv_dtype,
                    void *scratch, size_t scratch_bytes, insg_stream_t stream)
{
    if (tokens <= 0) return INSG_OK; // src/attention.cu:5 returns silently
    if (!q || !k_cache || !v_cache || !out || !scratch) return fail(INSG_E_ARG, "gqa_decode: null pointer");
    if (kv_dtype != INSG_KV_F32 && kv_dtype != INSG_KV_BF16) return fail(INSG_E_ARG, "gqa_decode: bad kv dtype");
    if (scratch_bytes < attn_scratch_bytes()) return fail(INSG_E_SHAPE, "gqa_decode: scratch too small");
    return attn_plain_launch(q, k_cache, v_cache, out, tokens, kv_dtype, scratch, stream);
}

int insg_attention_chunk(const insg_attn_op *op, int tokens, float *q_scratch, int rows_hint, insg_stream_t stream)
{
    if (!op || !op->qraw || !op->k_raw || !op->v || !op->q_norm_w || !op->k_norm_w || !op->k_cache || !op->v_cache ||
        !op->out || !op->position || !op->scratch || !q_scratch)
        return fail(INSG_E_ARG, "attention_chunk: null pointer");
    if (tokens < 1 || tokens > 65535) return fail(INSG_E_SHAPE, "attention_chunk: 1 <= tokens <= 65535");
    if (op->scratch_bytes < size_t(tokens) * attn_scratch_bytes()) return fail(INSG_E_SHAPE, "attention_chunk: scratch too small");
    if (op->max_context <= 0) return fail(INSG_E_SHAPE, "attention_chunk: max_context");
    AttnParams p = {};
    p.q = op->qraw; p.k_raw = op->k_raw; p.v_new = op->v; p.q_w = op->q_norm_w; p.k_w = op->k_norm_w;
    p.kc = op->k_cache; p.vc = op->v_cache; p.out = op->out;
    p.position = op->position; p.position_offset = op->position_offset;
    p.max_context = op->max_context; p.fast_trig = op->fast_trig; p.error_flag = op->error_flag;
    const bool bf16 = op->kv_dtype == INSG_KV_BF16;
    int rc = bf16 ? launch(attn_chunk_prepare_kernel<true>, dim3(tokens), dim3(kAtThreads), 0, stream, false, p, q_scratch)
                  : launch(attn_chunk_prepare_kernel<false>, dim3(tokens), dim3(kAtThreads), 0, stream, false, p, q_scratch);
    if (rc != INSG_OK) return rc;
    // step two: every (kv head, split, token) CTA is the plain split-K decode of its token over the rows up to its own
    p.q = q_scratch; p.q_stride = 4096; p.out_stride = 4096; p.scratch_stride = attn_scratch_bytes();
    p.counters = static_cast<unsigned *>(op->scratch);
    p.partials = reinterpret_cast<float *>(static_cast<uint8_t *>(op->scratch) + 64);
    // the splits a context of rows_hint rows needs (the kernel's own geometry); fewer CTAs to start and to count in
    int splits = kSplits;
    if (rows_hint > 0) {
        const int chunk = std::max(kMinChunk, (rows_hint + kSplits - 1) / kSplits);
        splits = std::max(1, std::min(kSplits, (rows_hint + chunk - 1) / chunk));
    }
    return bf16 ? launch_attn<true, false>(p, stream, false, tokens, splits) : launch_attn<false, false>(p, stream, false, tokens, splits);
}

int insg_attention_batch(const insg_attn_op *op, int sequences, size_t cache_stride_bytes, insg_stream_t stream)
{
    if (!op || !op->qraw || !op->k_raw || !op->v || !op->q_norm_w || !op->k_norm_w || !op->k_cache || !op->v_cache ||
        !op->out || !op->position || !op->scratch)
        return fail(INSG_E_ARG, "attention_batch: null pointer");
    if (sequences < 1 || sequences > 65535) return fail(INSG_E_SHAPE, "attention_batch: 1 <= sequences <= 65535");
    if (op->scratch_bytes < size_t(sequences) * attn_scratch_bytes()) return fail(INSG_E_SHAPE, "attention_batch: scratch too small");
    if (op->max_context <= 0) return fail(INSG_E_SHAPE, "attention_batch: max_context");
    if (sequences > 1 && (cache_stride_bytes == 0 || (cache_stride_bytes & 15))) return fail(INSG_E_ARG, "attention_batch: cache stride must be a positive multiple of 16 bytes");
    AttnParams p = {};
    p.q = op->qraw; p.k_raw = op->k_raw; p.v_new = op->v; p.q_w = op->q_norm_w; p.k_w = op->k_norm_w;
    p.kc = op->k_cache; p.vc = op->v_cache; p.out = op->out;
    p.position = op->position; p.position_offset = op->position_offset;
    p.max_context = op->max_context; p.fast_trig = op->fast_trig; p.error_flag = op->error_flag;
    p.counters = static_cast<unsigned *>(op->scratch);
    p.partials = reinterpret_cast<float *>(static_cast<uint8_t *>(op->scratch) + 64);
    p.q_stride = 8192; p.out_stride = 4096; p.kvin_stride = 1024; p.scratch_stride = attn_scratch_bytes(); p.cache_stride = cache_stride_bytes;
    const bool pdl = op->pdl != 0;
    return op->kv_dtype == INSG_KV_BF16 ? launch_attn<true, true>(p, stream, pdl, sequences) : launch_attn<false, true>(p, stream, pdl, sequences);
}

int insg_attention_step(const insg_attn_op *op, insg_stream_t stream)
{
    if (!op || !op->qraw || !op->k_raw || !op->v || !op->q_norm_w || !op->k_norm_w || !op->k_cache || !op->v_cache ||
        !op->out || !op->position || !op->scratch)
        return fail(INSG_E_ARG, "attention_step: null pointer");
    if (op->scratch_bytes < attn_scratch_bytes()) return fail(INSG_E_SHAPE, "attention_step: scratch too small");
    if (op->max_context <= 0) return fail(INSG_E_SHAPE, "attention_step: max_context");
    AttnParams p = {};
    p.q = op->qraw; p.k_raw = op->k_raw; p.v_new = op->v; p.q_w = op->q_norm_w; p.k_w = op->k_norm_w;
    p.kc = op->k_cache; p.vc = op->v_cache; p.out = op->out;
    p.position = op->position; p.position_offset = op->position_offset;
    p.max_context = op->max_context; p.fast_trig = op->fast_trig; p.error_flag = op->error_flag;
    p.counters = static_cast<unsigned *>(op->scratch);
    p.partials = reinterpret_cast<float *>(static_cast<uint8_t *>(op->scratch) + 64);
    const bool pdl = op->pdl != 0;
    return op->kv_dtype == INSG_KV_BF16 ? launch_attn<true, true>(p, stream, pdl) : launch_attn<false, true>(p, stream, pdl);
}

} // extern "C"
