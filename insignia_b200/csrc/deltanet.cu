// Gated DeltaNet single-token step for sm_100a.
//
// Recurrence (reference: src/deltanet.cu:4-13), per value head h with key head kh = h>>1:
//   qh = q * rsqrt(sum q^2 + 1e-6) / sqrt(128),  kh_ = k * rsqrt(sum k^2 + 1e-6),  d = exp(g_h)
//   mem_v  = sum_i S[i][v] * d * kh_[i]
//   dl_v   = (v_v - mem_v) * beta_h
//   S[i][v] = S[i][v] * d + kh_[i] * dl_v
//   out_v  = sum_i S[i][v] * qh[i]
// State layout fp32 [head][k=128][v=128], v contiguous.
//
// The reference reads the 64 KiB head state twice and writes it once from global
// memory with 32 CTAs.  Columns v are independent, so here each head is cut into
// 4 slices of 32 columns (128 CTAs); a CTA pulls its 16 KiB slice into registers
// once (coalesced 128-byte row segments, issued before the dependent-launch wait
// because the state was last written a whole token ago), does both reductions
// over k on chip, and writes the slice back once: 2 x 2 MiB of traffic per layer.
// The step is a latency chain, so it is kept short: all inputs are requested
// together, every warp normalises q and k for itself, and only the two sums over
// the eight warps cross a CTA barrier.
#include "common.cuh"
#include "host_util.h"

namespace insg {

constexpr int kDnThreads = 256;
constexpr int kSlices = 4; // 32 columns each

// `tokens` consecutive steps of the sequence in one launch: the slice stays in registers from step to step and is
// written back once; q/k/v of step m are at + m * qkv_stride, g/beta at + m * 32, the output at + m * 4096.
__global__ void __launch_bounds__(kDnThreads) deltanet_step_kernel(float *__restrict__ state, const float *__restrict__ q16,
                                                                   const float *__restrict__ k16, const float *__restrict__ v32,
                                                                   const float *__restrict__ g32, const float *__restrict__ beta32,
                                                                   float *__restrict__ out32, int tokens, int qkv_stride, long long state_stride,
                                                                   float *__restrict__ state_first, float *__restrict__ state_last)
{
    __shared__ __align__(16) float s_qk[8][2][128]; // per warp: its own copy of the normalised q and k (no block barrier)
    __shared__ __align__(16) float s_part[2][8][32]; // per-warp partial sums over k: [0] memory read-out, [1] output

    const int head = blockIdx.x / kSlices, slice = blockIdx.x % kSlices, kh = head >> 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int vq = tid & 7, kr = tid >> 3; // float4 column group, k row (rows kr, kr+32, kr+64, kr+96)
    const int v0 = slice * 32 + vq * 4;

    pdl_launch_dependents();

    // blockIdx.y: independent sequence of a decode batch (its own state, its own inputs and outputs)
    const int seq = blockIdx.y;
    q16 += size_t(seq) * qkv_stride; k16 += size_t(seq) * qkv_stride; v32 += size_t(seq) * qkv_stride;
    g32 += seq * 32; beta32 += seq * 32; out32 += size_t(seq) * 4096;
    float *S = state + size_t(seq) * state_stride + size_t(head) * 128 * 128;
    float4 cell[4];
#pragma unroll
    for (int j = 0; j < 4; j++) cell[j] = __ldcg(reinterpret_cast<const float4 *>(S + size_t(kr + 32 * j) * 128 + v0));

    pdl_wait();

    // Every dependent input of a step is requested at once; with several steps the next step's inputs are requested
    // before this step's arithmetic (they do not depend on it), so only the first step waits for a load.
    // Each warp reads the whole q and k of the key head (four values per lane) and normalises them itself: L2 norms
    // over 128 with eps added to the sum, as the reference.
    float4 nq4 = __ldcg(reinterpret_cast<const float4 *>(q16 + kh * 128) + lane);
    float4 nk4 = __ldcg(reinterpret_cast<const float4 *>(k16 + kh * 128) + lane);
    float4 nv4 = __ldcg(reinterpret_cast<const float4 *>(v32 + head * 128 + slice * 32) + vq); // this thread's columns
    float ng = __ldcg(g32 + head), nbeta = __ldcg(beta32 + head);
    for (int step = 0; step < tokens; step++, q16 += qkv_stride, k16 += qkv_stride, v32 += qkv_stride, g32 += 32, beta32 += 32, out32 += 4096) {
        __syncwarp(); // the previous step's reads of this warp's q/k copy are done
        const float4 q4 = nq4, k4 = nk4, v4 = nv4;
        const float g_in = ng, beta = nbeta;
        if (step + 1 < tokens) {
            nq4 = __ldcg(reinterpret_cast<const float4 *>(q16 + qkv_stride + kh * 128) + lane);
            nk4 = __ldcg(reinterpret_cast<const float4 *>(k16 + qkv_stride + kh * 128) + lane);
            nv4 = __ldcg(reinterpret_cast<const float4 *>(v32 + qkv_stride + head * 128 + slice * 32) + vq);
            ng = __ldcg(g32 + 32 + head);
            nbeta = __ldcg(beta32 + 32 + head);
        }
        const float qn = warp_sum(fmaf(q4.x, q4.x, fmaf(q4.y, q4.y, fmaf(q4.z, q4.z, q4.w * q4.w))));
        const float kn = warp_sum(fmaf(k4.x, k4.x, fmaf(k4.y, k4.y, fmaf(k4.z, k4.z, k4.w * k4.w))));
        const float qs = rsqrtf(qn + 1e-6f) * 0.08838834764831845f, ks = rsqrtf(kn + 1e-6f);
        reinterpret_cast<float4 *>(s_qk[warp][0])[lane] = make_float4(q4.x * qs, q4.y * qs, q4.z * qs, q4.w * qs);
        reinterpret_cast<float4 *>(s_qk[warp][1])[lane] = make_float4(k4.x * ks, k4.y * ks, k4.z * ks, k4.w * ks);
        __syncwarp();
        float qq[4], kk[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            qq[j] = s_qk[warp][0][kr + 32 * j];
            kk[j] = s_qk[warp][1][kr + 32 * j];
        }
        const float decay = expf(g_in);

        // mem_v = sum_i (S*d) * k
        float4 pm = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            pm.x = fmaf(cell[j].x * decay, kk[j], pm.x);
            pm.y = fmaf(cell[j].y * decay, kk[j], pm.y);
            pm.z = fmaf(cell[j].z * decay, kk[j], pm.z);
            pm.w = fmaf(cell[j].w * decay, kk[j], pm.w);
        }
        // a warp holds 4 k-rows (lane>>3) x 8 column groups: fold the rows, then every thread folds the 8 warps itself
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
        for (int w = 0; w < 8; w++) {
            const float4 t = *reinterpret_cast<const float4 *>(&s_part[0][w][vq * 4]);
            mem.x += t.x; mem.y += t.y; mem.z += t.z; mem.w += t.w;
        }
        const float4 dl = make_float4((v4.x - mem.x) * beta, (v4.y - mem.y) * beta, (v4.z - mem.z) * beta, (v4.w - mem.w) * beta);

        // S = S*d + k*delta ; out_v = sum_i S * q
        float4 po = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            cell[j].x = fmaf(cell[j].x, decay, kk[j] * dl.x);
            cell[j].y = fmaf(cell[j].y, decay, kk[j] * dl.y);
            cell[j].z = fmaf(cell[j].z, decay, kk[j] * dl.z);
            cell[j].w = fmaf(cell[j].w, decay, kk[j] * dl.w);
            po.x = fmaf(cell[j].x, qq[j], po.x);
            po.y = fmaf(cell[j].y, qq[j], po.y);
            po.z = fmaf(cell[j].z, qq[j], po.z);
            po.w = fmaf(cell[j].w, qq[j], po.w);
            // the state after the last step goes to state_last (default: in place); a speculative verify pass also keeps the
            // state after its first step (state_first), which is the one to continue from when the second token is rejected
            if (step == tokens - 1) *reinterpret_cast<float4 *>((state_last ? state_last + size_t(head) * 128 * 128 : S) + size_t(kr + 32 * j) * 128 + v0) = cell[j];
            else if (step == 0 && state_first) *reinterpret_cast<float4 *>(state_first + size_t(head) * 128 * 128 + size_t(kr + 32 * j) * 128 + v0) = cell[j];
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
            for (int w = 0; w < 8; w++) o += s_part[1][w][tid];
            out32[head * 128 + slice * 32 + tid] = o;
        }
    }
}


// The recurrence over many consecutive steps (a prompt pass): the same arithmetic in the same order as
// deltanet_step_kernel, so the state and the outputs are bit-identical to single steps, with everything that does not
// depend on the state taken off the serial chain.  Per block of 32 steps the eight warps normalise q and k (four steps
// each, all loads in flight), fetch v, beta and exp(g) into shared memory; a step then is: products with the slice,
// fold over k (shuffles + one CTA barrier), update, products with q.  The partial sums are double-buffered by step
// parity, so one barrier per step is enough, and the output of step t is folded by warp 0 while step t+1 runs.
constexpr int kDnBlock = 32;

__global__ void __launch_bounds__(kDnThreads) deltanet_steps_kernel(float *__restrict__ state, const float *__restrict__ q16,
                                                                    const float *__restrict__ k16, const float *__restrict__ v32,
                                                                    const float *__restrict__ g32, const float *__restrict__ beta32,
                                                                    float *__restrict__ out32, int tokens, int qkv_stride)
{
    __shared__ __align__(16) float s_q[kDnBlock][128];
    __shared__ __align__(16) float s_k[kDnBlock][128];
    __shared__ __align__(16) float s_v[kDnBlock][32];
    __shared__ float s_decay[kDnBlock], s_beta[kDnBlock];
    __shared__ __align__(16) float s_mem[2][8][32];
    __shared__ __align__(16) float s_out[2][8][32];

    const int head = blockIdx.x / kSlices, slice = blockIdx.x % kSlices, kh = head >> 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int vq = tid & 7, kr = tid >> 3;
    const int v0 = slice * 32 + vq * 4;

    pdl_launch_dependents();
    float *S = state + size_t(head) * 128 * 128;
    float4 cell[4];
#pragma unroll
    for (int j = 0; j < 4; j++) cell[j] = __ldcg(reinterpret_cast<const float4 *>(S + size_t(kr + 32 * j) * 128 + v0));
    pdl_wait();

    for (int base = 0; base < tokens; base += kDnBlock) {
        const int nb = min(kDnBlock, tokens - base);
        // ---- inputs of the block's steps: warp w takes steps w, w+8, w+16, w+24 (every read of the previous block's rows
        // lies before the barrier of its last step, which every warp has passed) ----
        {
            float4 q4[4], k4[4], x4[4];
            float gs[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int s = warp + 8 * i;
                q4[i] = k4[i] = x4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                gs[i] = 0.f;
                if (s < nb) {
                    const size_t off = size_t(base + s) * qkv_stride;
                    q4[i] = __ldcg(reinterpret_cast<const float4 *>(q16 + off + kh * 128) + lane);
                    k4[i] = __ldcg(reinterpret_cast<const float4 *>(k16 + off + kh * 128) + lane);
                    if (lane < 8) x4[i] = __ldcg(reinterpret_cast<const float4 *>(v32 + off + head * 128 + slice * 32) + lane);
                    else if (lane == 8) gs[i] = __ldcg(g32 + size_t(base + s) * 32 + head);
                    else if (lane == 9) gs[i] = __ldcg(beta32 + size_t(base + s) * 32 + head);
                }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int s = warp + 8 * i;
                if (s < nb) { // warp-uniform
                    const float qn = warp_sum(fmaf(q4[i].x, q4[i].x, fmaf(q4[i].y, q4[i].y, fmaf(q4[i].z, q4[i].z, q4[i].w * q4[i].w))));
                    const float kn = warp_sum(fmaf(k4[i].x, k4[i].x, fmaf(k4[i].y, k4[i].y, fmaf(k4[i].z, k4[i].z, k4[i].w * k4[i].w))));
                    const float qs = rsqrtf(qn + 1e-6f) * 0.08838834764831845f, ks = rsqrtf(kn + 1e-6f);
                    reinterpret_cast<float4 *>(s_q[s])[lane] = make_float4(q4[i].x * qs, q4[i].y * qs, q4[i].z * qs, q4[i].w * qs);
                    reinterpret_cast<float4 *>(s_k[s])[lane] = make_float4(k4[i].x * ks, k4[i].y * ks, k4[i].z * ks, k4[i].w * ks);
                    if (lane < 8) reinterpret_cast<float4 *>(s_v[s])[lane] = x4[i];
                    else if (lane == 8) s_decay[s] = expf(gs[i]);
                    else if (lane == 9) s_beta[s] = gs[i];
                }
            }
        }
        __syncthreads();

        for (int s = 0; s < nb; s++) {
            const int t = base + s, par = t & 1;
            float qq[4], kk[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                qq[j] = s_q[s][kr + 32 * j];
                kk[j] = s_k[s][kr + 32 * j];
            }
            const float decay = s_decay[s], beta = s_beta[s];
            const float4 v4 = *reinterpret_cast<const float4 *>(&s_v[s][vq * 4]);

            float4 pm = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 4; j++) {
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
            if (lane < 8) *reinterpret_cast<float4 *>(&s_mem[par][warp][lane * 4]) = pm;
            __syncthreads();
            if (t > 0 && tid < 32) { // the previous step's output, off the chain
                float o = 0.f;
#pragma unroll
                for (int w = 0; w < 8; w++) o += s_out[par ^ 1][w][tid];
                out32[size_t(t - 1) * 4096 + head * 128 + slice * 32 + tid] = o;
            }
            float4 mem = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < 8; w++) {
                const float4 u = *reinterpret_cast<const float4 *>(&s_mem[par][w][vq * 4]);
                mem.x += u.x; mem.y += u.y; mem.z += u.z; mem.w += u.w;
            }
            const float4 dl = make_float4((v4.x - mem.x) * beta, (v4.y - mem.y) * beta, (v4.z - mem.z) * beta, (v4.w - mem.w) * beta);
            float4 po = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                cell[j].x = fmaf(cell[j].x, decay, kk[j] * dl.x);
                cell[j].y = fmaf(cell[j].y, decay, kk[j] * dl.y);
                cell[j].z = fmaf(cell[j].z, decay, kk[j] * dl.z);
                cell[j].w = fmaf(cell[j].w, decay, kk[j] * dl.w);
                po.x = fmaf(cell[j].x, qq[j], po.x);
                po.y = fmaf(cell[j].y, qq[j], po.y);
                po.z = fmaf(cell[j].z, qq[j], po.z);
                po.w = fmaf(cell[j].w, qq[j], po.w);
            }
#pragma unroll
            for (int m = 8; m <= 16; m <<= 1) {
                po.x += __shfl_xor_sync(0xffffffffu, po.x, m);
                po.y += __shfl_xor_sync(0xffffffffu, po.y, m);
                po.z += __shfl_xor_sync(0xffffffffu, po.z, m);
                po.w += __shfl_xor_sync(0xffffffffu, po.w, m);
            }
            if (lane < 8) *reinterpret_cast<float4 *>(&s_out[par][warp][lane * 4]) = po;
        }
    }
#pragma unroll
    for (int j = 0; j < 4; j++) *reinterpret_cast<float4 *>(S + size_t(kr + 32 * j) * 128 + v0) = cell[j];
    __syncthreads();
    if (tid < 32) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) o += s_out[(tokens - 1) & 1][w][tid];
        out32[size_t(tokens - 1) * 4096 + head * 128 + slice * 32 + tid] = o;
    }
}

} // namespace insg

using namespace insg;

extern "C" int insg_deltanet_decode(float *state, const float *q16, const float *k16, const float *v32, const float *g32,
                                    const float *beta32, float *out32, int pdl, insg_stream_t stream)
{
    if (!state || !q16 || !k16 || !v32 || !g32 || !beta32 || !out32) return fail(INSG_E_ARG, "deltanet: null pointer");
    return launch(deltanet_step_kernel, dim3(32 * kSlices), dim3(kDnThreads), 0, stream, pdl != 0, state, q16, k16, v32, g32,
                  beta32, out32, 1, 0, 0ll, nullptr, nullptr);
}

extern "C" int insg_deltanet_decode_tokens(float *state, const float *q16, const float *k16, const float *v32, const float *g32,
                                           const float *beta32, float *out32, int tokens, int qkv_stride, int pdl,
                                           insg_stream_t stream)
{
    if (!state || !q16 || !k16 || !v32 || !g32 || !beta32 || !out32) return fail(INSG_E_ARG, "deltanet: null pointer");
    if (tokens < 1 || tokens > 1024 || qkv_stride < 0) return fail(INSG_E_SHAPE, "deltanet: 1..1024 tokens per launch");
    if (tokens == 1)
        return launch(deltanet_step_kernel, dim3(32 * kSlices), dim3(kDnThreads), 0, stream, pdl != 0, state, q16, k16, v32, g32, beta32,
                      out32, 1, qkv_stride, 0ll, nullptr, nullptr);
    return launch(deltanet_steps_kernel, dim3(32 * kSlices), dim3(kDnThreads), 0, stream, pdl != 0, state, q16, k16, v32, g32, beta32,
                  out32, tokens, qkv_stride);
}

extern "C" int insg_deltanet_decode_verify(const float *state, float *state_first, float *state_second, const float *q16, const float *k16,
                                           const float *v32, const float *g32, const float *beta32, float *out32, int qkv_stride, int pdl,
                                           insg_stream_t stream)
{
    if (!state || !state_first || !state_second || !q16 || !k16 || !v32 || !g32 || !beta32 || !out32) return fail(INSG_E_ARG, "deltanet: null pointer");
    if (qkv_stride < 0 || state_second == state) return fail(INSG_E_SHAPE, "deltanet: the second state needs a buffer of its own");
    return launch(deltanet_step_kernel, dim3(32 * kSlices), dim3(kDnThreads), 0, stream, pdl != 0, const_cast<float *>(state), q16, k16, v32, g32,
                  beta32, out32, 2, qkv_stride, 0ll, state_first, state_second);
}

extern "C" int insg_deltanet_decode_batch(float *state, long long state_stride, const float *q16, const float *k16, const float *v32,
                                          const float *g32, const float *beta32, float *out32, int sequences, int qkv_stride, int pdl,
                                          insg_stream_t stream)
{
    if (!state || !q16 || !k16 || !v32 || !g32 || !beta32 || !out32) return fail(INSG_E_ARG, "deltanet: null pointer");
    if (sequences < 1 || sequences > 64 || qkv_stride < 0 || state_stride < 32 * 128 * 128) return fail(INSG_E_SHAPE, "deltanet: 1..64 sequences");
    return launch(deltanet_step_kernel, dim3(32 * kSlices, sequences), dim3(kDnThreads), 0, stream, pdl != 0, state, q16, k16, v32, g32,
                  beta32, out32, 1, qkv_stride, state_stride, nullptr, nullptr);
}
