// Shared device helpers for the sm_100a decode kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace insg {

constexpr int kSMsFallback = 148;

// Programmatic dependent launch: let the next kernel in the stream start its
// independent preamble (weight / state prefetch) now, and block until the
// previous kernel's writes are visible before touching activations.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float bf16_bits_to_float(uint16_t h) { return __uint_as_float(uint32_t(h) << 16); }

// E2M1 code -> fp32, exact (reference table: include/insignia_layout.cuh:20-26).
// For magnitude codes m >= 2 the fp32 pattern is (m + 252) << 22 (exponent
// (m>>1)+126, mantissa msb m&1); m == 1 is 0.5 and m == 0 is 0.
__device__ __forceinline__ float e2m1_to_float(uint32_t code)
{
    const uint32_t m = code & 7u;
    const uint32_t mag = m >= 2u ? (m + 252u) << 22 : (m ? 0x3F000000u : 0u);
    return __uint_as_float(mag | ((code & 8u) << 28));
}

// E8M0 byte straight into the exponent field (0 -> 0.0, 255 -> +Inf), as the
// reference's MLX kernels do (src/mxfp4.cu:52).
__device__ __forceinline__ float e8m0_to_float(uint32_t byte) { return __uint_as_float(byte << 23); }

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int m = 16; m; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}
__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int m = 16; m; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
    return v;
}

// Block-wide sum for blockDim.x == 32*NW; `scratch` needs NW floats.  Every
// thread receives the result.  Contains two __syncthreads().
template <int NW> __device__ __forceinline__ float block_sum(float v, float *scratch)
{
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < NW; i++) t += scratch[i];
    return t;
}
template <int NW> __device__ __forceinline__ float block_max(float v, float *scratch)
{
    v = warp_max(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = scratch[0];
#pragma unroll
    for (int i = 1; i < NW; i++) t = fmaxf(t, scratch[i]);
    return t;
}

__device__ __forceinline__ float fast_sigmoid(float v) { return 1.0f / (1.0f + __expf(-v)); }
__device__ __forceinline__ float fast_silu(float v) { return v / (1.0f + __expf(-v)); }

// 128-bit streaming load that does not allocate in L1 (weights are read once per token).
__device__ __forceinline__ uint4 ldg_stream(const void *p)
{
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}
__device__ __forceinline__ uint32_t ldg_stream_u16(const void *p)
{
    uint16_t r;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(r) : "l"(p));
    return r;
}

} // namespace insg
