// Activation prologue shared by the fused GEMV kernels: loads the fp32 input vector once, applies the fused
// transform (RMSNorm, gated RMSNorm, sigmoid gates) and leaves the result in registers with its maximum magnitude.
#pragma once
#include "common.cuh"
#include "insignia_b200.h"

namespace insg {

constexpr int kProThreads = 512; // threads per CTA the prologue is written for
constexpr int kProWarps = kProThreads / 32;
constexpr int kMaxVec = 6;       // float4 per thread held in registers (cols <= 12288)

struct ProIn {
    const float *in, *aux;
    const uint16_t *norm_w;
    float *x_out;
    int cols, prologue;
};

__device__ __forceinline__ float block_max16(float v, float *scratch)
{
    v = warp_max(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = scratch[0];
#pragma unroll
    for (int i = 1; i < kProWarps; i++) t = fmaxf(t, scratch[i]);
    return t;
}

// Vectors per thread whose norm weights are fetched early (covers 4096 columns).
constexpr int kPreVec = 2;

// Norm weights are parameters, not activations: they can be fetched before the programmatic-dependent-launch wait.
__device__ __forceinline__ void preload_norm_weights(const ProIn &p, uint2 (&wv)[kPreVec])
{
    const int tid = threadIdx.x, nvec = p.cols >> 2;
#pragma unroll
    for (int j = 0; j < kPreVec; j++) {
        const int i = tid + j * kProThreads;
        wv[j] = make_uint2(0u, 0u);
        if (p.prologue == INSG_PRO_RMSNORM && i < nvec) wv[j] = reinterpret_cast<const uint2 *>(p.norm_w)[i];
        if (p.prologue == INSG_PRO_GATED_RMSNORM) wv[j] = reinterpret_cast<const uint2 *>(p.norm_w)[tid & 31];
    }
}

// Requests elements 4*(tid + 512 j) .. +3 of token m's input vector.  Reads go through L2 (ld.global.cg): under
// programmatic dependent launch this CTA may have been resident, and its L1 filled, before the producer wrote the inputs.
__device__ __forceinline__ void load_activation(const ProIn &p, int m, float4 (&v)[kMaxVec])
{
    const float *in = p.in + size_t(m) * p.cols;
    const int nvec = p.cols >> 2, tid = threadIdx.x;
#pragma unroll
    for (int j = 0; j < kMaxVec; j++) {
        const int i = tid + j * kProThreads;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < nvec) v[j] = __ldcg(reinterpret_cast<const float4 *>(in) + i);
    }
}

// Applies the fused transform to the vector load_activation fetched and returns max |x| over it.  `scratch` needs 32 floats.
__device__ __forceinline__ float transform_activation(const ProIn &p, int m, float4 (&v)[kMaxVec], const uint2 (&wpre)[kPreVec], float *scratch)
{
    const int cols = p.cols, tid = threadIdx.x, lane = tid & 31;
    const int nvec = cols >> 2;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxVec; j++) ss = fmaf(v[j].x, v[j].x, fmaf(v[j].y, v[j].y, fmaf(v[j].z, v[j].z, fmaf(v[j].w, v[j].w, ss))));
    float inv_rms = 1.f;
    float amax = 0.f;
    if (p.prologue == INSG_PRO_RMSNORM) {
        // one reduction round for both the sum of squares and max|x*w| (the maximum after scaling is that times inv_rms)
        float pre = 0.f;
#pragma unroll
        for (int j = 0; j < kMaxVec; j++) {
            const int i = tid + j * kProThreads;
            if (i < nvec) {
                const uint2 wv = j < kPreVec ? wpre[j < kPreVec ? j : 0] : reinterpret_cast<const uint2 *>(p.norm_w)[p.prologue == INSG_PRO_GATED_RMSNORM ? lane : i];
                pre = fmaxf(pre, fmaxf(fmaxf(fabsf(v[j].x * bf16_bits_to_float(wv.x & 0xffff)), fabsf(v[j].y * bf16_bits_to_float(wv.x >> 16))),
                                       fmaxf(fabsf(v[j].z * bf16_bits_to_float(wv.y & 0xffff)), fabsf(v[j].w * bf16_bits_to_float(wv.y >> 16)))));
            }
        }
        ss = warp_sum(ss);
        pre = warp_max(pre);
        __syncthreads();
        if (lane == 0) { scratch[tid >> 5] = ss; scratch[16 + (tid >> 5)] = pre; }
        __syncthreads();
        float tot = 0.f, mx = 0.f;
#pragma unroll
        for (int i = 0; i < kProWarps; i++) { tot += scratch[i]; mx = fmaxf(mx, scratch[16 + i]); }
        inv_rms = rsqrtf(tot / float(cols) + 1e-6f);
        amax = mx * inv_rms;
    }
#pragma unroll
    for (int j = 0; j < kMaxVec; j++) {
        const int i = tid + j * kProThreads;
        if (i < nvec) { // warp-uniform: nvec is a multiple of 32
            float4 x = v[j];
            const int k = i << 2;
            switch (p.prologue) {
            case INSG_PRO_RMSNORM: {
                const uint2 wv = j < kPreVec ? wpre[j < kPreVec ? j : 0] : reinterpret_cast<const uint2 *>(p.norm_w)[p.prologue == INSG_PRO_GATED_RMSNORM ? lane : i];
                x.x = x.x * inv_rms * bf16_bits_to_float(wv.x & 0xffff);
                x.y = x.y * inv_rms * bf16_bits_to_float(wv.x >> 16);
                x.z = x.z * inv_rms * bf16_bits_to_float(wv.y & 0xffff);
                x.w = x.w * inv_rms * bf16_bits_to_float(wv.y >> 16);
                break;
            }
            case INSG_PRO_GATED_RMSNORM: {
                // a warp covers one 128-wide head per j (32 lanes x float4)
                const float hs = warp_sum(fmaf(x.x, x.x, fmaf(x.y, x.y, fmaf(x.z, x.z, x.w * x.w))));
                const float inv = rsqrtf(hs / 128.f + 1e-6f);
                const uint2 wv = j < kPreVec ? wpre[j < kPreVec ? j : 0] : reinterpret_cast<const uint2 *>(p.norm_w)[p.prologue == INSG_PRO_GATED_RMSNORM ? lane : i];
                const float4 z = __ldcg(reinterpret_cast<const float4 *>(p.aux + size_t(m) * cols) + i);
                x.x = x.x * inv * bf16_bits_to_float(wv.x & 0xffff) * fast_silu(z.x);
                x.y = x.y * inv * bf16_bits_to_float(wv.x >> 16) * fast_silu(z.y);
                x.z = x.z * inv * bf16_bits_to_float(wv.y & 0xffff) * fast_silu(z.z);
                x.w = x.w * inv * bf16_bits_to_float(wv.y >> 16) * fast_silu(z.w);
                break;
            }
            case INSG_PRO_SIGMOID_GATE: {
                const float4 g = __ldcg(reinterpret_cast<const float4 *>(p.aux + size_t(m) * cols) + i);
                x.x *= fast_sigmoid(g.x); x.y *= fast_sigmoid(g.y); x.z *= fast_sigmoid(g.z); x.w *= fast_sigmoid(g.w);
                break;
            }
            case INSG_PRO_SIGMOID_GATE_HEAD0: {
                const float g = fast_sigmoid(__ldcg(p.aux + size_t(m) * 2 * cols + (k >> 8) * 512 + 256));
                x.x *= g; x.y *= g; x.z *= g; x.w *= g;
                break;
            }
            case INSG_PRO_SIGMOID_GATE_QPROJ: {
                const float4 g =
                    __ldcg(reinterpret_cast<const float4 *>(p.aux + size_t(m) * 2 * cols + (k >> 8) * 512 + 256 + (k & 255)));
                x.x *= fast_sigmoid(g.x); x.y *= fast_sigmoid(g.y); x.z *= fast_sigmoid(g.z); x.w *= fast_sigmoid(g.w);
                break;
            }
            default: break;
            }
            v[j] = x;
            if (p.prologue != INSG_PRO_RMSNORM) amax = fmaxf(amax, fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))));
            if (p.x_out && blockIdx.x == 0) reinterpret_cast<float4 *>(p.x_out + size_t(m) * cols)[i] = x;
        }
    }
    return p.prologue == INSG_PRO_RMSNORM ? amax : block_max16(amax, scratch);
}

} // namespace insg
