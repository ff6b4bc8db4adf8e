// Single-token grouped-query attention over a cache of `tokens` rows.
//
// Drop-in for the reference header of the same name (include/insignia_attention.cuh:4, behaviour src/attention.cu:4-5):
// 16 query heads of 256 over 4 kv heads, fp32 cache [token][4][256], out [16][256]; nothing happens for tokens <= 0.
// The reference's signature has no scratch argument, so this forwards to the entry point whose split-K scratch
// lives inside the library (at most 262144 tokens, one call at a time per GPU).
#pragma once
#include "insignia_b200.h"

#include <cuda_runtime.h>

namespace insignia {

inline void gqa_decode(const float *q, const float *k_cache, const float *v_cache, float *out, int tokens,
                       cudaStream_t stream = nullptr)
{
    (void)insg_gqa_decode_noalloc(q, k_cache, v_cache, out, tokens, INSG_KV_F32, stream);
}

} // namespace insignia
