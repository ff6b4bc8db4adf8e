// MXFP4 storage helpers and GEMV launchers.
//
// Drop-in for the reference header of the same name (include/insignia_layout.cuh:1-52): the 17-byte block type,
// the scalar decode helpers its tests use on the host, and the launchers, which here forward to the C ABI
// (insignia_b200.h).  Like the reference's launchers they return nothing and do nothing on a bad shape
// (src/mxfp4.cu:33,69); the reason stays available from insg_last_error().
#pragma once
#include "insignia_b200.h"

#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>

namespace insignia {

constexpr int MXFP4_BLOCK_VALUES = 32;
constexpr int MXFP4_BLOCK_BYTES = 17;

// One scale byte and 32 four-bit codes; element i < 16 is the low nibble of q[i], element 16 + i the high nibble.
#pragma pack(push, 1)
struct MxFp4Block {
    uint8_t scale;
    uint8_t q[16];
};
#pragma pack(pop)
static_assert(sizeof(MxFp4Block) == MXFP4_BLOCK_BYTES && alignof(MxFp4Block) == 1, "blocks are packed back to back");

// E2M1: sign, two exponent bits, one mantissa bit -> {0, .5, 1, 1.5, 2, 3, 4, 6} and their negatives (code 8 is -0).
__host__ __device__ __forceinline__ float fp4_e2m1(uint8_t x)
{
    const int e = (x >> 1) & 3, m = x & 1;
    const float mag = e == 0 ? 0.5f * float(m) : float(1 << (e - 1)) * (1.0f + 0.5f * float(m));
    return (x & 8) ? -mag : mag;
}

// E8M0: 2^(x - 127) built by placing x in the exponent field (so 0 gives +0); 255 is the format's NaN.
__host__ __device__ __forceinline__ float e8m0(uint8_t x)
{
    const uint32_t bits = x == 0xff ? 0x7fffffffu : uint32_t(x) << 23;
    float f;
    memcpy(&f, &bits, sizeof f);
    return f;
}

__host__ __device__ __forceinline__ uint8_t mxfp4_code(const MxFp4Block &block, int lane)
{
    const uint8_t byte = block.q[lane & 15];
    return lane < 16 ? uint8_t(byte & 15) : uint8_t(byte >> 4);
}

__host__ __device__ __forceinline__ float mxfp4_value(const MxFp4Block &block, int lane)
{
    return e8m0(block.scale) * fp4_e2m1(mxfp4_code(block, lane));
}

inline void mxfp4_gemv(const MxFp4Block *weights, const float *x, float *y, int rows, int cols, cudaStream_t stream = nullptr)
{
    (void)insg_mxfp4_gemv_blocks(weights, x, y, rows, cols, stream);
}

// MLX checkpoint layout: eight codes per U32, one scale byte per 32 columns.  warps_per_row tuned the reference's
// kernel and has no meaning here.
inline void mxfp4_gemv_mlx(const uint32_t *weights, const uint8_t *scales, const float *x, float *y, int rows, int cols,
                           int warps_per_row = 4, cudaStream_t stream = nullptr)
{
    (void)warps_per_row;
    (void)insg_mxfp4_gemv_mlx(weights, scales, x, y, rows, cols, stream);
}

inline void mxfp4_get_row_mlx(const uint32_t *weights, const uint8_t *scales, float *out, int row, int cols,
                              cudaStream_t stream = nullptr)
{
    (void)insg_mxfp4_get_row_mlx(weights, scales, out, row, cols, stream);
}

inline void quantize_q8_groups(const float *x, int8_t *qx, float *qscale, int cols, cudaStream_t stream = nullptr)
{
    (void)insg_quantize_q8_groups(x, qx, qscale, cols, stream);
}

inline void mxfp4_gemv_dp4a(const uint32_t *weights, const uint8_t *scales, const int8_t *qx, const float *qscale, float *y,
                            int rows, int cols, int warps_per_row = 4, cudaStream_t stream = nullptr)
{
    (void)warps_per_row;
    (void)insg_mxfp4_gemv_dp4a(weights, scales, qx, qscale, y, rows, cols, stream);
}

} // namespace insignia
