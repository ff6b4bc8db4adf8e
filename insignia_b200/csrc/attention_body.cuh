// Pieces of the split-K GQA decode shared by the stand-alone kernel (attention.cu) and by the attention phase of the
// persistent token kernel (persistent.cu): cache-row loads, the per-head RMSNorm + partial RoPE, the parameter block.
//
// Math (reference: src/attention.cu:4): score_t = (q_h . K[t][h>>2]) / 16, softmax over the cached tokens,
// out_h = sum_t p_t V[t][h>>2]; cache layout [token][4][256].
#pragma once
#include "common.cuh"

namespace insg {

constexpr int kSplits = 37;              // 4 kv heads x 37 = 148 CTAs
constexpr int kPartFloats = 8 + 4 * 256; // m[4], l[4], acc[4][256]

struct AttnParams {
    const float *q;        // plain: [16][256] normalised; fused: interleaved q_proj output [16][512]
    const float *k_raw;    // fused only
    const float *v_new;    // fused only
    const uint16_t *q_w, *k_w;
    void *kc, *vc;
    float *out;
    const int *position;   // fused: device scalar
    int position_offset;
    int tokens;            // plain
    int max_context;
    int fast_trig;
    unsigned *counters;    // [4] at the head of scratch
    float *partials;       // [4][kSplits][kPartFloats]
    // a chunk of consecutive tokens in one launch (blockIdx.y = token; all zero for a single token): token m uses
    // q + m * q_stride, out + m * out_stride, scratch + m * scratch_stride bytes, and sees position + offset + m + 1 rows
    int q_stride, out_stride;
    size_t scratch_stride;
    // independent sequences in one launch of the fused form (blockIdx.y = sequence, all at the same position): sequence s
    // also takes k_raw + s * kvin_stride, v_new + s * kvin_stride and the caches at + s * cache_stride bytes
    int kvin_stride;
    size_t cache_stride;
    int *error_flag;       // set to 1 when a bounded wait inside the kernel ran out (bf16 tensor-core path), or null
};

// A lane's 8 dims of one cache row, as loaded (converted only when used, so that two token groups can be in flight).
template <bool BF16> struct KvRow;
template <> struct KvRow<false> {
    struct Raw { float4 a, b; };
    static __device__ __forceinline__ Raw load_raw(const void *base, size_t row_elems, int lane)
    {
        const float4 *p = reinterpret_cast<const float4 *>(static_cast<const float *>(base) + row_elems) + lane * 2;
        return Raw{__ldcg(p), __ldcg(p + 1)};
    }
    static __device__ __forceinline__ Raw zero() { return Raw{make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)}; }
    static __device__ __forceinline__ void unpack(const Raw &r, float (&o)[8])
    {
        o[0] = r.a.x; o[1] = r.a.y; o[2] = r.a.z; o[3] = r.a.w; o[4] = r.b.x; o[5] = r.b.y; o[6] = r.b.z; o[7] = r.b.w;
    }
    static __device__ __forceinline__ float round(float v) { return v; }
    static __device__ __forceinline__ void store(void *base, size_t idx, float v) { static_cast<float *>(base)[idx] = v; }
};
template <> struct KvRow<true> {
    struct Raw { uint4 r; };
    static __device__ __forceinline__ Raw load_raw(const void *base, size_t row_elems, int lane)
    {
        return Raw{__ldcg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(base) + row_elems) + lane)};
    }
    static __device__ __forceinline__ Raw zero() { return Raw{make_uint4(0u, 0u, 0u, 0u)}; }
    static __device__ __forceinline__ void unpack(const Raw &w, float (&o)[8])
    {
        const uint4 r = w.r;
        o[0] = __uint_as_float(r.x << 16); o[1] = __uint_as_float(r.x & 0xffff0000u);
        o[2] = __uint_as_float(r.y << 16); o[3] = __uint_as_float(r.y & 0xffff0000u);
        o[4] = __uint_as_float(r.z << 16); o[5] = __uint_as_float(r.z & 0xffff0000u);
        o[6] = __uint_as_float(r.w << 16); o[7] = __uint_as_float(r.w & 0xffff0000u);
    }
    static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
    static __device__ __forceinline__ void store(void *base, size_t idx, float v)
    {
        static_cast<__nv_bfloat16 *>(base)[idx] = __float2bfloat16_rn(v);
    }
};

template <bool BF16, int KG> struct GroupRaw {
    typename KvRow<BF16>::Raw k[KG], v[KG];
};

// Rows tb..tb+KG-1 of one kv head (those below `tend`; the rest read as zero).
template <bool BF16, int KG>
__device__ __forceinline__ void load_group(const void *kc, const void *vc, int kvh, int tb, int tend, int lane, GroupRaw<BF16, KG> &g)
{
#pragma unroll
    for (int i = 0; i < KG; i++) {
        const int t = tb + i;
        if (t < tend) {
            const size_t row = (size_t(t) * 4 + kvh) * 256;
            g.k[i] = KvRow<BF16>::load_raw(kc, row, lane);
            g.v[i] = KvRow<BF16>::load_raw(vc, row, lane);
        } else {
            g.k[i] = KvRow<BF16>::zero();
            g.v[i] = KvRow<BF16>::zero();
        }
    }
}

// cos/sin of the rotate-half RoPE for the 8 dims a lane owns (only lanes 0..7 rotate: dims 0..63).
__device__ __forceinline__ void rope_table(int pos, int lane, bool fast, float (&c)[8], float (&s)[8])
{
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int half = (lane * 8 + j) & 31;
        if (fast) {
            const float a = float(pos) * __powf(10000000.0f, -float(2 * half) / 64.0f);
            c[j] = __cosf(a);
            s[j] = __sinf(a);
        } else {
            const float a = float(pos) * powf(10000000.0f, -float(2 * half) / 64.0f);
            sincosf(a, &s[j], &c[j]);
        }
    }
}

// RMSNorm over 256 (one warp, 8 values per lane, dims lane*8..+7) then rotate-half
// RoPE on dims 0..63 (lanes 0..7; the partner dim i+-32 lives 4 lanes away).
__device__ __forceinline__ void norm_rope_256(float (&v)[8], const uint4 wv, int lane, int pos, const float (&c)[8],
                                              const float (&s)[8])
{
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) ss = fmaf(v[j], v[j], ss);
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / 256.f + 1e-6f);
    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const float wf = bf16_bits_to_float((j & 1) ? (ww[j >> 1] >> 16) : (ww[j >> 1] & 0xffff));
        v[j] *= inv * wf;
    }
    if (pos != 0) {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float other = __shfl_xor_sync(0xffffffffu, v[j], 4);
            if (lane < 8) v[j] = v[j] * c[j] + (lane < 4 ? -other : other) * s[j];
        }
    }
}

} // namespace insg
