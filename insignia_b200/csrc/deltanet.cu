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
#include "common.cuh"
#include "host_util.h"

namespace insg {

constexpr int kDnThreads = 256;
constexpr int kSlices = 4; // 32 columns each

__global__ void __launch_bounds__(kDnThreads) deltanet_step_kernel(float *__restrict__ state, const float *__restrict__ q16,
                                                                   const float *__restrict__ k16, const float *__restrict__ v32,
                                                                   const float *__restrict__ g32, const float *__restrict__ beta32,
                                                                   float *__restrict__ out32)
{
    __shared__ float s_q[128], s_k[128];
    __shared__ float s_part[8][32];
    __shared__ float s_red[16];
    __shared__ float s_delta[32];

    const int head = blockIdx.x / kSlices, slice = blockIdx.x % kSlices, kh = head >> 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int vq = tid & 7, kr = tid >> 3; // float4 column group, k row (rows kr, kr+32, kr+64, kr+96)
    const int v0 = slice * 32 + vq * 4;

    pdl_launch_dependents();

    float *S = state + size_t(head) * 128 * 128;
    float4 cell[4];
#pragma unroll
    for (int j = 0; j < 4; j++) cell[j] = __ldcg(reinterpret_cast<const float4 *>(S + size_t(kr + 32 * j) * 128 + v0));

    pdl_wait();

    // L2 norms of q and k over 128 (eps added to the sum, as the reference)
    float qv = 0.f, kv = 0.f;
    if (tid < 128) {
        qv = __ldcg(q16 + kh * 128 + tid);
        kv = __ldcg(k16 + kh * 128 + tid);
    }
    // every dependent input is requested now, so the later stages do not each pay a trip to L2
    const float g_in = __ldcg(g32 + head), beta = __ldcg(beta32 + head);
    const float v_in = tid < 32 ? __ldcg(v32 + head * 128 + slice * 32 + tid) : 0.f;
    float qn = warp_sum(qv * qv), kn = warp_sum(kv * kv);
    if (lane == 0) { s_red[warp] = qn; s_red[8 + warp] = kn; }
    __syncthreads();
    const float qa = s_red[0] + s_red[1] + s_red[2] + s_red[3];
    const float ka = s_red[8] + s_red[9] + s_red[10] + s_red[11];
    const float qs = rsqrtf(qa + 1e-6f) * 0.08838834764831845f, ks = rsqrtf(ka + 1e-6f);
    if (tid < 128) { s_q[tid] = qv * qs; s_k[tid] = kv * ks; }
    __syncthreads();

    const float decay = expf(g_in);

    // mem_v = sum_i (S*d) * k
    float4 pm = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float kk = s_k[kr + 32 * j];
        pm.x = fmaf(cell[j].x * decay, kk, pm.x);
        pm.y = fmaf(cell[j].y * decay, kk, pm.y);
        pm.z = fmaf(cell[j].z * decay, kk, pm.z);
        pm.w = fmaf(cell[j].w * decay, kk, pm.w);
    }
    // a warp holds 4 k-rows (lane>>3) x 8 column groups: fold the rows, then the 8 warps
#pragma unroll
    for (int m = 8; m <= 16; m <<= 1) {
        pm.x += __shfl_xor_sync(0xffffffffu, pm.x, m);
        pm.y += __shfl_xor_sync(0xffffffffu, pm.y, m);
        pm.z += __shfl_xor_sync(0xffffffffu, pm.z, m);
        pm.w += __shfl_xor_sync(0xffffffffu, pm.w, m);
    }
    if (lane < 8) *reinterpret_cast<float4 *>(&s_part[warp][lane * 4]) = pm;
    __syncthreads();
    if (tid < 32) {
        float mem = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) mem += s_part[w][tid];
        s_delta[tid] = (v_in - mem) * beta;
    }
    __syncthreads();
    const float4 dl = *reinterpret_cast<const float4 *>(&s_delta[vq * 4]);

    // S = S*d + k*delta ; out_v = sum_i S * q
    float4 po = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float kk = s_k[kr + 32 * j], qq = s_q[kr + 32 * j];
        cell[j].x = fmaf(cell[j].x, decay, kk * dl.x);
        cell[j].y = fmaf(cell[j].y, decay, kk * dl.y);
        cell[j].z = fmaf(cell[j].z, decay, kk * dl.z);
        cell[j].w = fmaf(cell[j].w, decay, kk * dl.w);
        po.x = fmaf(cell[j].x, qq, po.x);
        po.y = fmaf(cell[j].y, qq, po.y);
        po.z = fmaf(cell[j].z, qq, po.z);
        po.w = fmaf(cell[j].w, qq, po.w);
        *reinterpret_cast<float4 *>(S + size_t(kr + 32 * j) * 128 + v0) = cell[j];
    }
#pragma unroll
    for (int m = 8; m <= 16; m <<= 1) {
        po.x += __shfl_xor_sync(0xffffffffu, po.x, m);
        po.y += __shfl_xor_sync(0xffffffffu, po.y, m);
        po.z += __shfl_xor_sync(0xffffffffu, po.z, m);
        po.w += __shfl_xor_sync(0xffffffffu, po.w, m);
    }
    __syncthreads(); // s_part is reused
    if (lane < 8) *reinterpret_cast<float4 *>(&s_part[warp][lane * 4]) = po;
    __syncthreads();
    if (tid < 32) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) o += s_part[w][tid];
        out32[head * 128 + slice * 32 + tid] = o;
    }
}

} // namespace insg

using namespace insg;

extern "C" int insg_deltanet_decode(float *state, const float *q16, const float *k16, const float *v32, const float *g32,
                                    const float *beta32, float *out32, int pdl, insg_stream_t stream)
{
    if (!state || !q16 || !k16 || !v32 || !g32 || !beta32 || !out32) return fail(INSG_E_ARG, "deltanet: null pointer");
    return launch(deltanet_step_kernel, dim3(32 * kSlices), dim3(kDnThreads), 0, stream, pdl != 0, state, q16, k16, v32, g32,
                  beta32, out32);
}
