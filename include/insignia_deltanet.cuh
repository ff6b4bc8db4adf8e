// One gated DeltaNet step for 32 value heads (16 key heads) of width 128.
//
// Drop-in for the reference header of the same name (include/insignia_deltanet.cuh:5, behaviour src/deltanet.cu:4-14):
// state fp32 [32][128 k][128 v] updated in place, q16/k16 [16][128], v32 [32][128], g32/beta32 [32], out32 [32][128].
#pragma once
#include "insignia_b200.h"

#include <cuda_runtime.h>

namespace insignia {

inline void deltanet_decode(float *state, const float *q16, const float *k16, const float *v32, const float *g32,
                            const float *beta32, float *out32, cudaStream_t stream = nullptr)
{
    (void)insg_deltanet_decode(state, q16, k16, v32, g32, beta32, out32, /*pdl*/ 0, stream);
}

} // namespace insignia
