// Helpers shared by the tcgen05 kernels (umma_gemv.cu: one token, activation image resident in shared memory;
// umma_gemm.cu: eight tokens per MMA, activation image streamed): shared-memory descriptors, mbarrier waits with a
// bound, bulk copies, and the split of an fp32 activation into exact E2M1 digits.
#pragma once
#include "common.cuh"

namespace insg {

constexpr int kURec = 8704;          // bytes per (128-row tile, 128-k block) weight record: 8192 of codes + 512 of scales
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// shared-memory matrix descriptor: no swizzle, version 1 (sm_100); offsets in bytes
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo)
{
    return uint64_t((saddr >> 4) & 0x3FFF) | (uint64_t((lbo >> 4) & 0x3FFF) << 16) | (uint64_t((sbo >> 4) & 0x3FFF) << 32) | (uint64_t(1) << 46);
}

__device__ __forceinline__ void mbar_init(uint64_t *b, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *b)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *b, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
// Bounded wait on a phase parity; false when the limit ran out or another role raised the abort flag.
__device__ __forceinline__ bool mbar_wait(uint64_t *b, uint32_t parity, volatile int *abort_flag)
{
    for (uint32_t it = 0; it < kSpinLimit; it++) {
        uint32_t done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(smem_u32(b)), "r"(parity) : "memory");
        if (done) return true;
        if ((it & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Twelve base-4 digits of |v| (24 bits) as E2M1 codes, one per nibble: digits 0..7 in lo, 8..11 in hi; sign in bit 3.
__device__ __forceinline__ void digit_codes(float x, float alpha, uint32_t &lo, uint32_t &hi)
{
    const float sc = fabsf(x) * alpha;                      // < 2^24
    const uint32_t v = min(__float2uint_rn(sc), 0xFFFFFFu);
    const uint32_t sgn = (__float_as_uint(x) >> 31) * 0x88888888u;
    uint32_t t = v & 0xFFFFu;                               // 16 bits -> eight 2-bit digits, one per nibble
    t = (t | (t << 8)) & 0x00FF00FFu;
    t = (t | (t << 4)) & 0x0F0F0F0Fu;
    t = (t | (t << 2)) & 0x33333333u;
    uint32_t u = v >> 16;                                   // 8 bits -> four digits
    u = (u | (u << 4)) & 0x0F0F0F0Fu;
    u = (u | (u << 2)) & 0x33333333u;
    // digit d -> E2M1 code of the value d: 0,1,2,3 -> 0,2,4,5 = 2d - (d == 3)
    lo = ((t << 1) - ((t >> 1) & t & 0x11111111u)) | sgn;
    hi = ((u << 1) - ((u >> 1) & u & 0x11111111u)) | (sgn & 0x0000FFFFu);
}

} // namespace insg
