// Launchers the reference declares next to its MLX-layout GEMV but does not use in the token loop:
// the GEMV over 17-byte {scale, 16 code bytes} blocks (include/insignia_layout.cuh:11-15,45 and
// src/mxfp4.cu:5-35 in the reference), and the int8 activation path of its microbenchmark
// (src/mxfp4.cu:83-127: per-32 absmax quantisation of x, then integer dot products against the E2M1
// codes doubled to integers).  They exist here so that the reference's kernel-level drivers link and
// give the same answers; the decode engine never calls them.
#include "common.cuh"
#include "host_util.h"

namespace insg {

constexpr int kCompatWarps = 4;

// ---- block layout: row r, block b at byte (r * blocks + b) * 17; byte 0 = E8M0 scale, byte 1+i holds
// element i in its low nibble and element 16+i in its high nibble.
__global__ void __launch_bounds__(kCompatWarps * 32) gemv_blocks_kernel(const uint8_t *__restrict__ w, const float *__restrict__ x,
                                                                       float *__restrict__ y, int rows, int blocks)
{
    const int lane = threadIdx.x & 31, row = blockIdx.x * kCompatWarps + (threadIdx.x >> 5);
    if (row >= rows) return;
    const uint8_t *base = w + size_t(row) * blocks * 17;
    float acc = 0.f;
    for (int b = 0; b < blocks; b++) {
        const uint8_t *blk = base + size_t(b) * 17;
        const uint8_t sc = blk[0], byte = blk[1 + (lane & 15)];
        const uint32_t code = lane < 16 ? (byte & 15u) : (byte >> 4);
        // the reference's helper maps scale byte 255 to a NaN (bits 0x7fffffff), every other byte to 2^(byte-127)
        const float s = sc == 0xff ? __uint_as_float(0x7fffffffu) : __uint_as_float(uint32_t(sc) << 23);
        acc = fmaf(s * e2m1_to_float(code), x[b * 32 + lane], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) y[row] = acc;
}

// ---- activations to int8: one warp per group of 32, scale = max|x| / 127 (1 when the group is all zero)
__global__ void __launch_bounds__(kCompatWarps * 32) quantize_q8_kernel(const float *__restrict__ x, int8_t *__restrict__ q,
                                                                       float *__restrict__ scale, int groups)
{
    const int lane = threadIdx.x & 31, grp = blockIdx.x * kCompatWarps + (threadIdx.x >> 5);
    if (grp >= groups) return;
    const float v = x[grp * 32 + lane];
    const float amax = warp_max(fabsf(v));
    const float s = amax > 0.f ? amax * (1.0f / 127.0f) : 1.0f;
    if (lane == 0) scale[grp] = s;
    q[grp * 32 + lane] = static_cast<int8_t>(__float2int_rn(v / s));
}

// ---- MLX-layout weights against int8 activations.  Twice an E2M1 value is an integer (0,1,2,3,4,6,8,12),
// so a group of 32 is eight 4-way integer dot products; the group's sum is scaled by
// 2^(scale-127) * activation scale / 2 and added in fp32.  A warp owns a row; lane l takes groups l, l+32, ...
__device__ __forceinline__ int e2m1_twice(uint32_t code)
{
    const int mag = int(code & 7u);
    const int v = mag < 4 ? mag : (mag == 4 ? 4 : (mag == 5 ? 6 : (mag == 6 ? 8 : 12)));
    return (code & 8u) ? -v : v;
}

__global__ void __launch_bounds__(kCompatWarps * 32) gemv_dp4a_kernel(const uint32_t *__restrict__ w, const uint8_t *__restrict__ sc,
                                                                     const int8_t *__restrict__ qx, const float *__restrict__ qs,
                                                                     float *__restrict__ y, int rows, int groups)
{
    const int lane = threadIdx.x & 31, row = blockIdx.x * kCompatWarps + (threadIdx.x >> 5);
    if (row >= rows) return;
    const uint4 *wr = reinterpret_cast<const uint4 *>(w + size_t(row) * groups * 4);
    const uint8_t *sr = sc + size_t(row) * groups;
    float acc = 0.f;
    for (int g = lane; g < groups; g += 32) {
        const uint4 pk = wr[g];
        const uint32_t words[4] = {pk.x, pk.y, pk.z, pk.w};
        const int *xa = reinterpret_cast<const int *>(qx + g * 32);
        int dot = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
#pragma unroll
            for (int half = 0; half < 2; half++) {
                int packed = 0;
#pragma unroll
                for (int j = 0; j < 4; j++)
                    packed |= (e2m1_twice((words[i] >> ((half * 4 + j) * 4)) & 15u) & 0xff) << (8 * j);
                dot = __dp4a(packed, xa[i * 2 + half], dot);
            }
        }
        acc = fmaf(float(dot), __uint_as_float(uint32_t(sr[g]) << 23) * qs[g] * 0.5f, acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) y[row] = acc;
}

} // namespace insg

using namespace insg;

extern "C" {

int insg_mxfp4_gemv_blocks(const void *blocks, const float *x, float *y, int rows, int cols, insg_stream_t stream)
{
    if (rows <= 0 || cols <= 0 || (cols & 31)) return fail(INSG_E_SHAPE, "mxfp4_gemv_blocks: rows, cols > 0 and cols % 32 == 0");
    if (!blocks || !x || !y) return fail(INSG_E_ARG, "mxfp4_gemv_blocks: null pointer");
    return launch(gemv_blocks_kernel, dim3((rows + kCompatWarps - 1) / kCompatWarps), dim3(kCompatWarps * 32), 0, stream, false,
                  static_cast<const uint8_t *>(blocks), x, y, rows, cols >> 5);
}

int insg_quantize_q8_groups(const float *x, int8_t *qx, float *qscale, int cols, insg_stream_t stream)
{
    if (cols <= 0 || (cols & 31)) return fail(INSG_E_SHAPE, "quantize_q8_groups: cols > 0 and cols % 32 == 0");
    if (!x || !qx || !qscale) return fail(INSG_E_ARG, "quantize_q8_groups: null pointer");
    const int groups = cols >> 5;
    return launch(quantize_q8_kernel, dim3((groups + kCompatWarps - 1) / kCompatWarps), dim3(kCompatWarps * 32), 0, stream, false, x, qx,
                  qscale, groups);
}

int insg_mxfp4_gemv_dp4a(const uint32_t *weight, const uint8_t *scales, const int8_t *qx, const float *qscale, float *y, int rows,
                         int cols, insg_stream_t stream)
{
    if (rows <= 0 || cols <= 0 || (cols & 31)) return fail(INSG_E_SHAPE, "mxfp4_gemv_dp4a: rows, cols > 0 and cols % 32 == 0");
    if (!weight || !scales || !qx || !qscale || !y) return fail(INSG_E_ARG, "mxfp4_gemv_dp4a: null pointer");
    return launch(gemv_dp4a_kernel, dim3((rows + kCompatWarps - 1) / kCompatWarps), dim3(kCompatWarps * 32), 0, stream, false, weight,
                  scales, qx, qscale, y, rows, cols >> 5);
}

} // extern "C"
