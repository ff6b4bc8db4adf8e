// Persistent token kernel for sm_100a: one cooperative launch walks a whole token step (or several).
//
// The reference issues ~580 launches per token (src/decode.cu:14-23) and the graph path of this library 162, every one
// of them strictly dependent on the one before: most of a token is then launch turn-around, not weight streaming.
// Here a *program* -- the same sequence of fused operations, recorded instead of launched -- is run by one grid of
// one CTA per SM that stays resident for the whole token:
//   * each operation becomes a *phase*; phases are separated by a grid-wide barrier (an arrival counter in global
//     memory, release/acquire, with a bounded wait that raises an error flag and makes every CTA leave);
//   * the fused GEMV phases run the stages of gemv_body.cuh unchanged (same split of the records over CTAs and
//     warps, same summation order, hence bit-identical results to the stand-alone kernel); the first weight chunks of
//     the NEXT GEMV phase are issued into registers before the current phase is closed, so they are in flight across
//     the epilogue, the barrier and any DeltaNet / attention phase in between;
//   * weights do not depend on activations, so every warp also runs an L2 prefetch cursor a fixed number of records
//     ahead of its own consumption along its token-long record sequence (cp.async.bulk.prefetch.L2, across phase
//     boundaries): HBM keeps streaming while the SMs sit in barriers, prologues and the small recurrent phases;
//   * the DeltaNet step, the split-K attention step and the embedding lookup are phases of the same kernel;
//   * for device-fed generation the kernel loops over tokens itself (the head phase feeds its arg-max back).
// Activations that another CTA wrote in an earlier phase are always read past L1 (ld.global.cg / cp.async.cg): no kernel
// boundary invalidates L1 inside a persistent launch.
#include "attention_body.cuh"
#include "gemv_body.cuh"
#include "host_util.h"

#include <algorithm>
#include <mutex>
#include <vector>

namespace insg {

// Records per register prefetch chunk in the phases: one fewer than the stand-alone kernel's, which sits exactly at the
// register ceiling; the loop here also carries the phase bookkeeping and would spill.  The chunk depth does not change
// the order of any sum.
constexpr int kPersistUnr = 2;

enum { PH_GEMV = 0, PH_DELTANET = 1, PH_ATTENTION = 2, PH_EMBED = 3 };

struct DnParams {
    float *state;
    const float *q16, *k16, *v32, *g32, *beta32;
    float *out32;
};

struct EmbedParams {
    const uint32_t *w;
    const uint8_t *s;
    float *out;
    const int *row_ptr;
    int rows, cols;
};

struct AttnPhase {
    AttnParams p;
    int bf16;
};

struct alignas(16) Phase {
    int type;
    int next_gemv; // index of the next GEMV phase after this one, or -1
    int grid;      // GEMV: CTAs that take part (the stand-alone kernel's grid for the same operation)
    int pad;
    union {
        GemvParams g;
        DnParams d;
        AttnPhase a;
        EmbedParams e;
    };
};

// Barrier state in device memory, zero at creation.  `count` only grows: barrier k of a launch is passed when it
// reaches base + (k + 1) * arrivals; the launch leaves base advanced for the next one.
struct SyncState {
    unsigned count;
    unsigned base;
    int error;
    int pad;
};

struct RunArgs {
    const Phase *phases;
    int nphases, first_gemv;
    SyncState *sync;
    int n_tokens;
    int set_token, set_position; // >= 0: written to *d_token / *d_position before the first phase
    int *d_token, *d_position;
    int *error_flag;             // raised (with sync->error) when a barrier wait runs out
    unsigned long long timeout_ns;
    int arrivals;                // CTAs a barrier waits for (the grid size; a self-test passes more)
    int pf_records;              // per-warp L2 prefetch distance in records, 0 = off
    int work_offset;             // bytes of dynamic shared memory taken by the program copy; the phases' buffers follow
    unsigned long long *times;   // development builds (INSG_PHASE_TIMES): [step][CTA][4] nanosecond stamps, or null
};

// Development aid, compiled in only with -DINSG_PHASE_TIMES: every CTA stamps the clock at four points of every phase.
#ifdef INSG_PHASE_TIMES
#define INSG_STAMP(slot)                                                                                              \
    do {                                                                                                              \
        if (a.times && threadIdx.x == 0) a.times[(size_t(step) * gridDim.x + blockIdx.x) * 4 + (slot)] = globaltimer_ns(); \
    } while (0)
#else
#define INSG_STAMP(slot) \
    do {                 \
    } while (0)
#endif

__device__ __forceinline__ unsigned long long globaltimer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ unsigned ld_acquire(const unsigned *p)
{
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Grid-wide barrier.  Returns false when it gave up (error raised): the caller must leave the kernel.
__device__ __forceinline__ bool grid_barrier(const RunArgs &a, unsigned target, int *s_ok)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        int ok = 1;
        __threadfence();
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(&a.sync->count) : "memory");
        if (int(ld_acquire(&a.sync->count) - target) < 0) {
            const unsigned long long t0 = globaltimer_ns();
            unsigned polls = 0;
            while (int(ld_acquire(&a.sync->count) - target) < 0) {
                if ((++polls & 63u) == 0u) {
                    if (*reinterpret_cast<volatile int *>(&a.sync->error) != 0) { ok = 0; break; }
                    if (globaltimer_ns() - t0 > a.timeout_ns) {
                        *reinterpret_cast<volatile int *>(&a.sync->error) = 1;
                        if (a.error_flag) *reinterpret_cast<volatile int *>(a.error_flag) = 1;
                        __threadfence();
                        ok = 0;
                        break;
                    }
                }
            }
        }
        *s_ok = ok;
    }
    __syncthreads();
    return *s_ok != 0;
}

// ---- L2 prefetch cursor -------------------------------------------------------------------------------------------
// One cursor per CTA, run by its last warp: it walks the CTA's records of the GEMV phases in program order (wrapping to
// the next token while tokens remain) and stays a fixed number of records ahead of the phase being consumed.  Records
// of one (tile, matrix) run are contiguous in memory, and so are consecutive runs of one matrix: a lane takes one run
// and issues ONE bulk prefetch for the part of it inside the range (the copy engine is slow on many small requests).
struct PfCursor {
    int ph;       // phase the cursor is in, -1 = finished
    int u, end;   // next record and end of this CTA's share in that phase
    int wraps;    // token wraps still allowed
    int ahead;    // records between the end of the share being consumed and the cursor
};

__device__ __forceinline__ GemvRange phase_range(const Phase &P, int c, int warp)
{
    if (c >= P.grid) return GemvRange{0, 0, 0, 0, 0};
    return gemv_range(P.g, P.grid, c, warp);
}

__device__ __forceinline__ void pf_enter(const Phase *prog, PfCursor &pf, int ph, int c)
{
    pf.ph = ph;
    if (ph < 0) return;
    const GemvRange r = phase_range(prog[ph], c, 0);
    pf.u = r.a;
    pf.end = r.b;
}

__device__ __forceinline__ void pf_next_phase(const RunArgs &a, const Phase *prog, PfCursor &pf, int c)
{
    int nx = prog[pf.ph].next_gemv;
    if (nx < 0) {
        if (pf.wraps > 0) { pf.wraps--; nx = a.first_gemv; }
    }
    pf_enter(prog, pf, nx, c);
}

// Called by one warp when the CTA starts consuming GEMV phase `ph` (its share is [ra, rb)): the cursor is moved past
// that share if it is still inside it, then advanced until it is `distance` records ahead of the share's end.
__device__ __forceinline__ void pf_advance(const RunArgs &a, const Phase *prog, PfCursor &pf, int ph, int ra, int rb, int c, int lane)
{
    const int distance = a.pf_records * kWarps;
    if (pf.ph < 0) return;
    pf.ahead -= rb - ra;
    if (pf.ahead < 0) { // the cursor is still inside the share being consumed now: move it to the phase after
        pf.ahead = 0;
        pf.ph = ph;
        pf_next_phase(a, prog, pf, c);
    }
    int guard = 0;
    while (pf.ph >= 0 && pf.ahead < distance && ++guard < 64) {
        const GemvParams &q = prog[pf.ph].g;
        const int n = min(distance - pf.ahead, pf.end - pf.u);
        if (n > 0) {
            const int nkb = q.nkb, u0 = pf.u, u1 = pf.u + n;
            for (int tm = u0 / nkb + lane; tm * nkb < u1; tm += 32) { // one run per lane
                const int lo = max(tm * nkb, u0), hi = min((tm + 1) * nkb, u1);
                const uint8_t *ptr = run_base(q, tm) + size_t(lo - tm * nkb) * kRec;
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(ptr), "r"((hi - lo) * kRec) : "memory");
            }
        }
        pf.u += n;
        pf.ahead += n;
        if (pf.u >= pf.end) pf_next_phase(a, prog, pf, c);
    }
}

// ---- DeltaNet step as a phase (reference: src/deltanet.cu:4-13) -----------------------------------------------------
// 128 CTAs = 32 value heads x 4 slices of 32 columns; 512 threads: thread (kr = tid >> 3, vq = tid & 7) holds rows kr and
// kr + 64 of its float4 column group.  Same recurrence and the same reduction shape as deltanet_step_kernel.
__device__ __noinline__ void deltanet_phase(const DnParams &d, uint8_t *smem, int c)
{
    constexpr int kSlices = 4;
    if (c >= 32 * kSlices) return;
    float(*s_qk)[2][128] = reinterpret_cast<float(*)[2][128]>(smem);                            // [16 warps][q|k][128]
    float(*s_part)[kWarps][32] = reinterpret_cast<float(*)[kWarps][32]>(smem + kWarps * 2 * 128 * 4); // [2][16][32]
    const int head = c / kSlices, slice = c % kSlices, kh = head >> 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int vq = tid & 7, kr = tid >> 3;
    const int v0 = slice * 32 + vq * 4;
    float *S = d.state + size_t(head) * 128 * 128;
    float4 cell[2];
#pragma unroll
    for (int j = 0; j < 2; j++) cell[j] = __ldcg(reinterpret_cast<const float4 *>(S + size_t(kr + 64 * j) * 128 + v0));
    const float4 q4 = __ldcg(reinterpret_cast<const float4 *>(d.q16 + kh * 128) + lane);
    const float4 k4 = __ldcg(reinterpret_cast<const float4 *>(d.k16 + kh * 128) + lane);
    const float4 v4 = __ldcg(reinterpret_cast<const float4 *>(d.v32 + head * 128 + slice * 32) + vq);
    const float g_in = __ldcg(d.g32 + head), beta = __ldcg(d.beta32 + head);
    const float qn = warp_sum(fmaf(q4.x, q4.x, fmaf(q4.y, q4.y, fmaf(q4.z, q4.z, q4.w * q4.w))));
    const float kn = warp_sum(fmaf(k4.x, k4.x, fmaf(k4.y, k4.y, fmaf(k4.z, k4.z, k4.w * k4.w))));
    const float qs = rsqrtf(qn + 1e-6f) * 0.08838834764831845f, ks = rsqrtf(kn + 1e-6f);
    reinterpret_cast<float4 *>(s_qk[warp][0])[lane] = make_float4(q4.x * qs, q4.y * qs, q4.z * qs, q4.w * qs);
    reinterpret_cast<float4 *>(s_qk[warp][1])[lane] = make_float4(k4.x * ks, k4.y * ks, k4.z * ks, k4.w * ks);
    __syncwarp();
    float qq[2], kk[2];
#pragma unroll
    for (int j = 0; j < 2; j++) {
        qq[j] = s_qk[warp][0][kr + 64 * j];
        kk[j] = s_qk[warp][1][kr + 64 * j];
    }
    const float decay = expf(g_in);
    float4 pm = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 2; j++) {
        pm.x = fmaf(cell[j].x * decay, kk[j], pm.x);
        pm.y = fmaf(cell[j].y * decay, kk[j], pm.y);
        pm.z = fmaf(cell[j].z * decay, kk[j], pm.z);
        pm.w = fmaf(cell[j].w * decay, kk[j], pm.w);
    }
#pragma unroll
    for (int m = 8; m <= 16; m <<= 1) {
        pm.x += __shfl_xor_sync(0xffffffffu, pm.x, m);
        pm.y += __shfl_xor_sync(0xffffffffu, pm.y, m);
        pm.z += __shfl_xor_sync(0xffffffffu, pm.z, m);
        pm.w += __shfl_xor_sync(0xffffffffu, pm.w, m);
    }
    if (lane < 8) *reinterpret_cast<float4 *>(&s_part[0][warp][lane * 4]) = pm;
    __syncthreads();
    float4 mem = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < kWarps; w++) {
        const float4 t = *reinterpret_cast<const float4 *>(&s_part[0][w][vq * 4]);
        mem.x += t.x; mem.y += t.y; mem.z += t.z; mem.w += t.w;
    }
    const float4 dl = make_float4((v4.x - mem.x) * beta, (v4.y - mem.y) * beta, (v4.z - mem.z) * beta, (v4.w - mem.w) * beta);
    float4 po = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 2; j++) {
        cell[j].x = fmaf(cell[j].x, decay, kk[j] * dl.x);
        cell[j].y = fmaf(cell[j].y, decay, kk[j] * dl.y);
        cell[j].z = fmaf(cell[j].z, decay, kk[j] * dl.z);
        cell[j].w = fmaf(cell[j].w, decay, kk[j] * dl.w);
        po.x = fmaf(cell[j].x, qq[j], po.x);
        po.y = fmaf(cell[j].y, qq[j], po.y);
        po.z = fmaf(cell[j].z, qq[j], po.z);
        po.w = fmaf(cell[j].w, qq[j], po.w);
        *reinterpret_cast<float4 *>(S + size_t(kr + 64 * j) * 128 + v0) = cell[j];
    }
#pragma unroll
    for (int m = 8; m <= 16; m <<= 1) {
        po.x += __shfl_xor_sync(0xffffffffu, po.x, m);
        po.y += __shfl_xor_sync(0xffffffffu, po.y, m);
        po.z += __shfl_xor_sync(0xffffffffu, po.z, m);
        po.w += __shfl_xor_sync(0xffffffffu, po.w, m);
    }
    if (lane < 8) *reinterpret_cast<float4 *>(&s_part[1][warp][lane * 4]) = po;
    __syncthreads();
    if (tid < 32) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; w++) o += s_part[1][w][tid];
        d.out32[head * 128 + slice * 32 + tid] = o;
    }
}

// ---- fused attention step as a phase (reference: src/ops.cu:9, src/qwen_kernels.cu:15,31, src/attention.cu:4) -------
// Job (kv head, split) = a range of cached tokens for the four query heads of one kv head; 16 warps, each scoring two
// tokens at a time with an online softmax; partials to scratch; the last job of a kv head folds its splits.
template <bool BF16> __device__ __noinline__ void attention_phase(const AttnParams &p, uint8_t *smem, int G, int c)
{
    using Row = KvRow<BF16>;
    constexpr int KG = 2;
    constexpr int kMinChunk = kWarps * KG;
    float(*s_q)[256] = reinterpret_cast<float(*)[256]>(smem);                   // [4][256], pre-scaled by 1/16
    float *s_knew = reinterpret_cast<float *>(smem + 4096), *s_vnew = s_knew + 256;
    float(*s_m)[4] = reinterpret_cast<float(*)[4]>(smem + 4096 + 2048);          // [16][4]
    float(*s_l)[4] = s_m + kWarps;
    float(*s_e)[4] = s_l + kWarps;                                               // [64][4]
    float *s_lg = reinterpret_cast<float *>(s_e + 64);                           // [4]
    int *s_last = reinterpret_cast<int *>(s_lg + 4);
    float(*s_acc)[4][256] = reinterpret_cast<float(*)[4][256]>(smem + 8192);     // [16][4][256] = 64 KB
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    const int pos = __ldcg(p.position) + p.position_offset;
    const int tokens = max(1, min(pos + 1, p.max_context));
    const int chunk = max(kMinChunk, (tokens + kSplits - 1) / kSplits);
    const int nsplit = (tokens + chunk - 1) / chunk;
    const int fresh = tokens - 1; // the row this phase writes

    for (int job = c; job < 4 * nsplit; job += G) {
        const int kvh = job / nsplit, split = job % nsplit;
        const int t0 = split * chunk, t1 = min(tokens, t0 + chunk);
        const int tend = min(t1, fresh);
        GroupRaw<BF16, KG> ga;
        load_group<BF16, KG>(p.kc, p.vc, kvh, t0 + warp * KG, tend, lane, ga);
        // ---- query (and current key / value) preparation ----
        if (warp < 5) {
            const uint4 norm_wv = reinterpret_cast<const uint4 *>(warp < 4 ? p.q_w : p.k_w)[lane];
            float rope_c[8], rope_s[8];
            if (lane < 8) rope_table(pos, lane, p.fast_trig != 0, rope_c, rope_s);
            if (warp < 4) {
                float v[8];
                const float4 *src = reinterpret_cast<const float4 *>(p.q + size_t(kvh * 4 + warp) * 512 + lane * 8);
                const float4 a = __ldcg(src), b = __ldcg(src + 1);
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
                norm_rope_256(v, norm_wv, lane, pos, rope_c, rope_s);
#pragma unroll
                for (int j = 0; j < 8; j++) s_q[warp][lane * 8 + j] = v[j] * 0.0625f;
            } else if (pos >= t0 && pos < t1) {
                float v[8];
                const float4 *src = reinterpret_cast<const float4 *>(p.k_raw + kvh * 256 + lane * 8);
                const float4 a = __ldcg(src), b = __ldcg(src + 1);
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
                norm_rope_256(v, norm_wv, lane, pos, rope_c, rope_s);
                const size_t row = (size_t(pos) * 4 + kvh) * 256 + lane * 8;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    Row::store(p.kc, row + j, v[j]);
                    s_knew[lane * 8 + j] = Row::round(v[j]);
                }
            }
        } else if (warp == 5 && pos >= t0 && pos < t1) {
            const size_t row = (size_t(pos) * 4 + kvh) * 256 + lane * 8;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float v = __ldcg(p.v_new + kvh * 256 + lane * 8 + j);
                Row::store(p.vc, row + j, v);
                s_vnew[lane * 8 + j] = Row::round(v);
            }
        }
        __syncthreads();

        float m[4], l[4], acc[4][8];
#pragma unroll
        for (int h = 0; h < 4; h++) {
            m[h] = -3.0e38f;
            l[h] = 0.f;
#pragma unroll
            for (int j = 0; j < 8; j++) acc[h][j] = 0.f;
        }
        // cached rows [t0, tend): one online-softmax update per group of KG tokens
        for (int tb = t0 + warp * KG; tb < tend; tb += kWarps * KG) {
            float kk[KG][8];
#pragma unroll
            for (int g = 0; g < KG; g++) Row::unpack(ga.k[g], kk[g]);
            float s[KG][4];
#pragma unroll
            for (int h = 0; h < 4; h++) {
                const float4 qa = *reinterpret_cast<const float4 *>(&s_q[h][lane * 8]);
                const float4 qb = *reinterpret_cast<const float4 *>(&s_q[h][lane * 8 + 4]);
#pragma unroll
                for (int g = 0; g < KG; g++) {
                    float z = qa.x * kk[g][0];
                    z = fmaf(qa.y, kk[g][1], z); z = fmaf(qa.z, kk[g][2], z); z = fmaf(qa.w, kk[g][3], z);
                    z = fmaf(qb.x, kk[g][4], z); z = fmaf(qb.y, kk[g][5], z); z = fmaf(qb.z, kk[g][6], z); z = fmaf(qb.w, kk[g][7], z);
                    s[g][h] = z;
                }
            }
#pragma unroll
            for (int mk = 16; mk; mk >>= 1)
#pragma unroll
                for (int g = 0; g < KG; g++)
#pragma unroll
                    for (int h = 0; h < 4; h++) s[g][h] += __shfl_xor_sync(0xffffffffu, s[g][h], mk);
            float pr[KG][4];
#pragma unroll
            for (int h = 0; h < 4; h++) {
                float mn = m[h];
#pragma unroll
                for (int g = 0; g < KG; g++)
                    if (tb + g < tend) mn = fmaxf(mn, s[g][h]);
                const float corr = __expf(m[h] - mn);
                float psum = 0.f;
#pragma unroll
                for (int g = 0; g < KG; g++) {
                    pr[g][h] = tb + g < tend ? __expf(s[g][h] - mn) : 0.f;
                    psum += pr[g][h];
                }
                m[h] = mn;
                l[h] = fmaf(l[h], corr, psum);
#pragma unroll
                for (int j = 0; j < 8; j++) acc[h][j] *= corr;
            }
#pragma unroll
            for (int g = 0; g < KG; g++) {
                float vv[8];
                Row::unpack(ga.v[g], vv);
#pragma unroll
                for (int h = 0; h < 4; h++)
#pragma unroll
                    for (int j = 0; j < 8; j++) acc[h][j] = fmaf(pr[g][h], vv[j], acc[h][j]);
            }
            load_group<BF16, KG>(p.kc, p.vc, kvh, tb + kWarps * KG, tend, lane, ga);
        }
        // the row this phase wrote (the current token), from shared memory: one more update, by the last warp
        if (warp == kWarps - 1 && fresh >= t0 && fresh < t1) {
#pragma unroll
            for (int h = 0; h < 4; h++) {
                float z = 0.f;
#pragma unroll
                for (int j = 0; j < 8; j++) z = fmaf(s_q[h][lane * 8 + j], s_knew[lane * 8 + j], z);
                z = warp_sum(z);
                const float mn = fmaxf(m[h], z);
                const float corr = __expf(m[h] - mn), pe = __expf(z - mn);
                m[h] = mn;
                l[h] = fmaf(l[h], corr, pe);
#pragma unroll
                for (int j = 0; j < 8; j++) acc[h][j] = fmaf(pe, s_vnew[lane * 8 + j], acc[h][j] * corr);
            }
        }
        // ---- fold the 16 warps ----
#pragma unroll
        for (int h = 0; h < 4; h++) {
            if (lane == 0) { s_m[warp][h] = m[h]; s_l[warp][h] = l[h]; }
#pragma unroll
            for (int j = 0; j < 8; j++) s_acc[warp][h][lane * 8 + j] = acc[h][j];
        }
        __syncthreads();
        float *part = p.partials + size_t(kvh * kSplits + split) * kPartFloats;
        for (int o = tid; o < 1024; o += kThreads) {
            const int h = o >> 8, d = o & 255;
            float mg = s_m[0][h];
#pragma unroll
            for (int w = 1; w < kWarps; w++) mg = fmaxf(mg, s_m[w][h]);
            float lg = 0.f, av = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; w++) {
                const float e = __expf(s_m[w][h] - mg); // warps without tokens carry m=-3e38, l=0, acc=0
                lg = fmaf(s_l[w][h], e, lg);
                av = fmaf(s_acc[w][h][d], e, av);
            }
            part[8 + h * 256 + d] = av;
            if (d == 0) { part[h] = mg; part[4 + h] = lg; }
        }
        // ---- the last job of this kv head folds the splits ----
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned ticket = atomicAdd(p.counters + kvh, 1u);
            *s_last = (ticket == unsigned(nsplit) - 1u);
        }
        __syncthreads();
        if (*s_last) {
            __threadfence();
            const float *pp = p.partials + size_t(kvh * kSplits) * kPartFloats;
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
            if (tid < 256) {
                const int h = tid >> 6, c4 = tid & 63;
                const float4 *src = reinterpret_cast<const float4 *>(pp + 8 + h * 256) + c4;
                float4 av = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
                for (int s = 0; s < nsplit; s++) {
                    const float4 v = __ldcg(src + size_t(s) * (kPartFloats / 4));
                    const float e = s_e[s][h];
                    av.x = fmaf(v.x, e, av.x);
                    av.y = fmaf(v.y, e, av.y);
                    av.z = fmaf(v.z, e, av.z);
                    av.w = fmaf(v.w, e, av.w);
                }
                const float inv = 1.0f / s_lg[h];
                reinterpret_cast<float4 *>(p.out + size_t(kvh * 4 + h) * 256)[c4] = make_float4(av.x * inv, av.y * inv, av.z * inv, av.w * inv);
            }
            if (tid == 0) p.counters[kvh] = 0u;
        }
        __syncthreads(); // shared buffers are reused by the next job
    }
}

// ---- embedding row as a phase (reference: src/qwen35.cu:9, src/mxfp4.cu:132-133) --------------------------------------
__device__ __noinline__ void embed_phase(const EmbedParams &e, int c)
{
    if (c != 0) return;
    const int row = __ldcg(e.row_ptr);
    const bool ok = row >= 0 && row < e.rows;
    for (int wi = threadIdx.x; wi < (e.cols >> 3); wi += kThreads) {
        float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
        if (ok) {
            const uint32_t word = e.w[size_t(row) * (e.cols >> 3) + wi];
            const float sc = e8m0_to_float(e.s[size_t(row) * (e.cols >> 5) + (wi >> 2)]);
            lo = make_float4(e2m1_to_float(word) * sc, e2m1_to_float(word >> 4) * sc, e2m1_to_float(word >> 8) * sc,
                             e2m1_to_float(word >> 12) * sc);
            hi = make_float4(e2m1_to_float(word >> 16) * sc, e2m1_to_float(word >> 20) * sc, e2m1_to_float(word >> 24) * sc,
                             e2m1_to_float(word >> 28) * sc);
        }
        reinterpret_cast<float4 *>(e.out)[wi * 2] = lo;
        reinterpret_cast<float4 *>(e.out)[wi * 2 + 1] = hi;
    }
}

// ---- the kernel -------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, 1) persistent_token_kernel(const __grid_constant__ RunArgs a)
{
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __shared__ GemvShared sh;
    __shared__ int s_ok;
    __shared__ unsigned s_base;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = int(gridDim.x), c = int(blockIdx.x);

    // The program is copied into shared memory once: every descriptor read of every phase (the current one, the next one
    // whose first chunks are issued early, the ones the prefetch cursor walks) is then an on-chip read.  From global
    // memory each of them would be an L2 round trip, several of them dependent on one another, after every barrier
    // (the barrier's acquire drops the SM's L1 contents).
    Phase *prog = reinterpret_cast<Phase *>(smem_raw);
    uint8_t *work = smem_raw + a.work_offset;
    {
        const uint4 *src = reinterpret_cast<const uint4 *>(a.phases);
        uint4 *dst = reinterpret_cast<uint4 *>(prog);
        const int n16 = int(size_t(a.nphases) * sizeof(Phase) / 16);
        for (int i = tid; i < n16; i += kThreads) dst[i] = src[i];
    }
    if (tid == 0) {
        s_base = ld_acquire(&a.sync->base);
        if (c == 0) {
            if (a.set_token >= 0 && a.d_token) *a.d_token = a.set_token;
            if (a.set_position >= 0 && a.d_position) *a.d_position = a.set_position;
        }
    }
    __syncthreads();
    unsigned target = s_base;
    // The scalars CTA 0 has just stored are read by every CTA of a first phase that is not CTA 0's alone (an attention
    // phase reads the position): one barrier orders the store before those reads.  Once per launch, not per token.
    if ((a.set_token >= 0 && a.d_token) || (a.set_position >= 0 && a.d_position)) {
        target += unsigned(a.arrivals);
        if (!grid_barrier(a, target, &s_ok)) return;
    }

    // the prefetch cursors live in shared memory between phases: they must not cost registers in the record loop
    __shared__ PfCursor s_pf;
    if (warp == kWarps - 1) {
        PfCursor pf;
        pf.wraps = a.n_tokens - 1;
        pf.ahead = 0;
        pf_enter(prog, pf, a.first_gemv, c);
        if (lane == 0) s_pf = pf;
        __syncwarp();
    }

    const int total = a.n_tokens * a.nphases;
    int step = 0, ph = 0;
    while (step < total) {
        if (prog[ph].type == PH_GEMV) {
            // A run of consecutive GEMV phases.  The chunk registers live only inside this scope, so the recurrent phases
            // below have the whole register file; inside the run the next phase's first chunks are issued before the
            // current phase is closed and stay in flight across its epilogue and the barrier.
            // Every CTA runs every stage, CTAs beyond the phase's grid with an empty range: the weight loads must not sit
            // inside a branch (the compiler then waits for them where the branch rejoins, and a phase that keeps its loads
            // in flight across stages streams at two thirds of the rate).
            Chunk<kPersistUnr> A, B;
            UnitIt lit;
            GemvRange r = phase_range(prog[ph], c, warp);
            gemv_issue_first<kPersistUnr>(prog[ph].g, r, A, B, lit, lane);
            for (;;) {
                const Phase &P = prog[ph];
                const GemvParams &p = P.g;
                INSG_STAMP(0);
                if (a.pf_records > 0 && warp == kWarps - 1) {
                    PfCursor pf = s_pf;
                    pf_advance(a, prog, pf, ph, r.a, r.b, c, lane);
                    __syncwarp();
                    if (lane == 0) s_pf = pf;
                    __syncwarp();
                }
                const int nph = ph + 1 < a.nphases ? ph + 1 : 0;
                const bool more = step + 1 < total;
                const bool chain = more && prog[nph].type == PH_GEMV;
                const int xstride = p.cols + 8;
                __half *xs = reinterpret_cast<__half *>(work);
                float *rec = reinterpret_cast<float *>(work + size_t(2) * xstride * sizeof(__half));
                float *scratch = rec + size_t(kWarps) * p.slots * 16;
                gemv_publish_range(r, sh, lane, warp);
                uint2 wpre[kPreVec];
                preload_norm_weights(ProIn{p.in, p.aux, p.norm_w, p.x_out, p.cols, p.prologue}, wpre);
                float inv_alpha[1];
                gemv_activation<1>(p, xs, xstride, scratch, wpre, inv_alpha);
                INSG_STAMP(1);
                gemv_stream<kPersistUnr, 1>(p, r, A, B, lit, xs, xstride, rec + size_t(warp) * p.slots * 16, inv_alpha, lane);
                // the next phase's first chunks go out now and stay in flight across this phase's closing and the barrier
                const Phase &N = prog[chain ? nph : ph];
                const GemvRange rn = chain ? phase_range(N, c, warp) : GemvRange{0, 0, 0, 0, 0};
                gemv_issue_first<kPersistUnr>(N.g, rn, A, B, lit, lane);
                __syncthreads();
                INSG_STAMP(2);
                gemv_finish<1>(p, r, P.grid, c, rec, scratch, sh);
                INSG_STAMP(3);
                if (more) {
                    target += unsigned(a.arrivals);
                    if (!grid_barrier(a, target, &s_ok)) return;
                }
                step++;
                ph = nph;
                if (!chain) break;
                r = rn;
            }
        } else {
            const Phase &P = prog[ph];
            INSG_STAMP(0);
            if (P.type == PH_DELTANET) {
                deltanet_phase(P.d, work, c);
            } else if (P.type == PH_ATTENTION) {
                if (P.a.bf16) attention_phase<true>(P.a.p, work, G, c);
                else attention_phase<false>(P.a.p, work, G, c);
            } else if (P.type == PH_EMBED) {
                embed_phase(P.e, c);
            }
            INSG_STAMP(3);
            if (step + 1 < total) {
                target += unsigned(a.arrivals);
                if (!grid_barrier(a, target, &s_ok)) return;
            }
            step++;
            ph = ph + 1 < a.nphases ? ph + 1 : 0;
        }
    }
    // every CTA read `base` before its first arrival, and CTA 0 is past every barrier only after all arrived
    if (c == 0 && tid == 0) a.sync->base = target;
}

// ---- host side --------------------------------------------------------------------------------------------------------
int gemv_build_params(const insg_gemv_op *op, int M, int max_grid, GemvParams *out, int *grid_out, size_t *smem_out);
size_t attn_scratch_bytes();

} // namespace insg

using namespace insg;

struct insg_program {
    std::vector<Phase> phases;
    Phase *d_phases = nullptr;
    SyncState *d_sync = nullptr;
    size_t smem = 0;      // largest working area of any phase
    size_t prog_bytes = 0; // the program copy in front of it
    int grid = 0;
    int device = 0;
    bool final = false;
    int pf_records = 24;
    unsigned long long timeout_ns = 2000000000ull;
    uint64_t weight_bytes = 0;
    unsigned long long *times = nullptr;
};

namespace {
constexpr size_t kDnSmem = size_t(kWarps) * 2 * 128 * 4 + size_t(2) * kWarps * 32 * 4;
constexpr size_t kAtSmem = 8192 + size_t(kWarps) * 4 * 256 * 4;

int program_check(insg_program *g, bool want_final)
{
    if (!g) return fail(INSG_E_ARG, "program: null handle");
    if (g->final != want_final) return fail(INSG_E_ARG, want_final ? "program: not finalised" : "program: already finalised");
    return INSG_OK;
}
} // namespace

extern "C" {

insg_program *insg_program_create(void)
{
    insg_program *g = new insg_program();
    if (cudaGetDevice(&g->device) != cudaSuccess) g->device = 0;
    int sms = sm_count();
    g->grid = std::min(sms, kMaxGrid);
    return g;
}

void insg_program_destroy(insg_program *g)
{
    if (!g) return;
    if (g->d_phases) cudaFree(g->d_phases);
    if (g->d_sync) cudaFree(g->d_sync);
    delete g;
}

int insg_program_add_gemv(insg_program *g, const insg_gemv_op *op)
{
    int rc = program_check(g, false);
    if (rc) return rc;
    if (op && op->layout != 0) return fail(INSG_E_ARG, "program: the tcgen05 weight layout has no phase form");
    if (op && op->tokens > 1) return fail(INSG_E_SHAPE, "program: one token per phase");
    Phase P = {};
    P.type = PH_GEMV;
    size_t smem = 0;
    rc = gemv_build_params(op, 1, g->grid, &P.g, &P.grid, &smem);
    if (rc) return rc;
    g->smem = std::max(g->smem, smem);
    for (int i = 0; i < op->n_segments; i++)
        g->weight_bytes += uint64_t(op->seg[i].rows) * op->cols * 17 / 32 * (op->seg[i].epilogue == INSG_EPI_SWIGLU ? 2 : 1);
    g->phases.push_back(P);
    return INSG_OK;
}

int insg_program_add_deltanet(insg_program *g, float *state, const float *q16, const float *k16, const float *v32, const float *g32,
                              const float *beta32, float *out32)
{
    int rc = program_check(g, false);
    if (rc) return rc;
    if (!state || !q16 || !k16 || !v32 || !g32 || !beta32 || !out32) return fail(INSG_E_ARG, "program: deltanet null pointer");
    if (g->grid < 128) return fail(INSG_E_LIMIT, "program: the DeltaNet phase needs 128 CTAs");
    Phase P = {};
    P.type = PH_DELTANET;
    P.d = DnParams{state, q16, k16, v32, g32, beta32, out32};
    g->smem = std::max(g->smem, kDnSmem);
    g->phases.push_back(P);
    return INSG_OK;
}

int insg_program_add_attention(insg_program *g, const insg_attn_op *op)
{
    int rc = program_check(g, false);
    if (rc) return rc;
    if (!op || !op->qraw || !op->k_raw || !op->v || !op->q_norm_w || !op->k_norm_w || !op->k_cache || !op->v_cache || !op->out ||
        !op->position || !op->scratch)
        return fail(INSG_E_ARG, "program: attention null pointer");
    if (op->scratch_bytes < attn_scratch_bytes()) return fail(INSG_E_SHAPE, "program: attention scratch too small");
    if (op->max_context <= 0) return fail(INSG_E_SHAPE, "program: max_context");
    Phase P = {};
    P.type = PH_ATTENTION;
    AttnParams &p = P.a.p;
    p.q = op->qraw; p.k_raw = op->k_raw; p.v_new = op->v; p.q_w = op->q_norm_w; p.k_w = op->k_norm_w;
    p.kc = op->k_cache; p.vc = op->v_cache; p.out = op->out;
    p.position = op->position; p.position_offset = op->position_offset;
    p.max_context = op->max_context; p.fast_trig = op->fast_trig;
    p.counters = static_cast<unsigned *>(op->scratch);
    p.partials = reinterpret_cast<float *>(static_cast<uint8_t *>(op->scratch) + 64);
    P.a.bf16 = op->kv_dtype == INSG_KV_BF16;
    g->smem = std::max(g->smem, kAtSmem);
    g->phases.push_back(P);
    return INSG_OK;
}

int insg_program_add_embed(insg_program *g, const uint32_t *weight, const uint8_t *scales, float *out, const int *device_row, int rows,
                           int cols)
{
    int rc = program_check(g, false);
    if (rc) return rc;
    if (!weight || !scales || !out || !device_row) return fail(INSG_E_ARG, "program: embed null pointer");
    if (rows <= 0 || cols <= 0 || (cols & 31)) return fail(INSG_E_SHAPE, "program: embed rows/cols");
    Phase P = {};
    P.type = PH_EMBED;
    P.e = EmbedParams{weight, scales, out, device_row, rows, cols};
    g->phases.push_back(P);
    return INSG_OK;
}

int insg_program_finalize(insg_program *g)
{
    int rc = program_check(g, false);
    if (rc) return rc;
    if (g->phases.empty()) return fail(INSG_E_ARG, "program: no phases");
    int next = -1;
    for (int i = int(g->phases.size()) - 1; i >= 0; i--) {
        g->phases[i].next_gemv = next;
        if (g->phases[i].type == PH_GEMV) next = i;
    }
    cudaError_t e = cudaFuncSetAttribute(persistent_token_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(persistent)");
    g->smem = std::max<size_t>(g->smem, 1024);
    g->prog_bytes = (g->phases.size() * sizeof(Phase) + 127) / 128 * 128;
    if (g->prog_bytes + g->smem > 220 * 1024)
        return fail(INSG_E_LIMIT, "program: too many operations for the shared-memory copy of the program (about 180 with full-size GEMVs)");
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, persistent_token_kernel, kThreads, g->prog_bytes + g->smem);
    if (e != cudaSuccess) return cuda_fail(e, "occupancy query");
    if (per_sm < 1) return fail(INSG_E_LIMIT, "program: the kernel does not fit an SM");
    e = cudaMalloc(&g->d_phases, g->phases.size() * sizeof(Phase));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(program)");
    e = cudaMalloc(&g->d_sync, sizeof(SyncState));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(program)");
    e = cudaMemcpy(g->d_phases, g->phases.data(), g->phases.size() * sizeof(Phase), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy(program)");
    e = cudaMemset(g->d_sync, 0, sizeof(SyncState));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemset(program)");
    g->final = true;
    return INSG_OK;
}

int insg_program_set_option(insg_program *g, const char *key, long long value)
{
    if (!g || !key) return fail(INSG_E_ARG, "program: null argument");
    const std::string k = key;
    if (k == "prefetch_records") g->pf_records = int(std::max(0ll, std::min(value, 4096ll)));
    else if (k == "timeout_ns") g->timeout_ns = (unsigned long long)std::max(1000ll, value);
#ifdef INSG_PHASE_TIMES
    else if (k == "phase_times") g->times = reinterpret_cast<unsigned long long *>(value);
#endif
    else return fail(INSG_E_ARG, "program: unknown option");
    return INSG_OK;
}

static int program_launch(insg_program *g, int n_tokens, int token, int position, int *d_token, int *d_position, int *error_flag,
                          int arrivals, cudaStream_t stream)
{
    RunArgs a = {};
    a.phases = g->d_phases;
    a.nphases = int(g->phases.size());
    a.first_gemv = -1;
    for (int i = 0; i < a.nphases; i++)
        if (g->phases[i].type == PH_GEMV) { a.first_gemv = i; break; }
    a.sync = g->d_sync;
    a.n_tokens = n_tokens;
    a.set_token = token;
    a.set_position = position;
    a.d_token = d_token;
    a.d_position = d_position;
    a.error_flag = error_flag;
    a.timeout_ns = g->timeout_ns;
    a.arrivals = arrivals;
    a.pf_records = g->pf_records;
    a.work_offset = int(g->prog_bytes);
    a.times = g->times;
    void *args[] = {&a};
    const cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void *>(persistent_token_kernel), dim3(g->grid), dim3(kThreads), args,
                                                      g->prog_bytes + g->smem, stream);
    if (e != cudaSuccess) return cuda_fail(e, "cooperative launch");
    return INSG_OK;
}

int insg_program_run(insg_program *g, int n_tokens, int token, int position, int *device_token, int *device_position, int *error_flag,
                     insg_stream_t stream)
{
    int rc = program_check(g, true);
    if (rc) return rc;
    if (n_tokens < 1) return fail(INSG_E_SHAPE, "program: n_tokens >= 1");
    if ((token >= 0 && !device_token) || (position >= 0 && !device_position)) return fail(INSG_E_ARG, "program: scalar pointer missing");
    return program_launch(g, n_tokens, token, position, device_token, device_position, error_flag, g->grid, stream);
}

int insg_program_recover(insg_program *g, insg_stream_t stream)
{
    int rc = program_check(g, true);
    if (rc) return rc;
    const cudaError_t e = cudaMemsetAsync(g->d_sync, 0, sizeof(SyncState), stream);
    return e == cudaSuccess ? INSG_OK : cuda_fail(e, "cudaMemsetAsync(program)");
}

int insg_program_selftest_barrier_timeout(insg_program *g, unsigned long long timeout_ns, int *error_flag, insg_stream_t stream)
{
    int rc = program_check(g, true);
    if (rc) return rc;
    if (!error_flag) return fail(INSG_E_ARG, "program: error flag missing");
    const unsigned long long keep = g->timeout_ns;
    g->timeout_ns = std::max(1000ull, std::min(timeout_ns, 100000000ull));
    // every barrier waits for one arrival more than there are CTAs: the first wait runs out, every CTA leaves
    rc = program_launch(g, 1, -1, -1, nullptr, nullptr, error_flag, g->grid + 1, stream);
    g->timeout_ns = keep;
    return rc;
}

int insg_program_phase_count(const insg_program *g) { return g ? int(g->phases.size()) : 0; }
uint64_t insg_program_weight_bytes(const insg_program *g) { return g ? g->weight_bytes : 0; }

} // extern "C"
