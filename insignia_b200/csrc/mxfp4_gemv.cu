// MXFP4 codec kernels for sm_100a: repack into the streaming layout, plain GEMV on the MLX layout,
// row dequantisation (embedding), full dequantisation.  The fused streaming GEMV is in gemv_fused.cu.
//
// Layouts (reference: include/insignia_layout.cuh:47-48, src/mxfp4.cu:50-52): MLX checkpoint layout is
// U32[rows][cols/8] (nibble j of word i = element 8i+j) + U8[rows][cols/32]; the packed layout groups
// rows in tiles of 16 and K in blocks of 128, one 1088-byte record per (tile, block): lane L = (g, t)
// of a warp owns bytes [16L, 16L+16) = scale group t of row g, bytes [512+16L, ...) = the same group of
// row g+8, and scale bytes [1024+2L, 1024+2L+2) = the two rows' E8M0 scales for that group.
#include "common.cuh"
#include "host_util.h"

namespace insg {

constexpr int kRec = 1088;

// ---- repack: MLX layout -> tile-interleaved records ---------------------------
__global__ void repack_kernel(const uint32_t *__restrict__ w, const uint8_t *__restrict__ s, uint8_t *__restrict__ out,
                              int rows, int cols)
{
    const int nkb = cols >> 7;
    const size_t rec_id = size_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const size_t nrec = size_t(rows >> 4) * nkb;
    if (rec_id >= nrec) return;
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int tile = int(rec_id / nkb), kb = int(rec_id % nkb);
    uint8_t *rec = out + rec_id * kRec;
    const int words_per_row = cols >> 3, groups_per_row = cols >> 5;
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const size_t row = size_t(tile) * 16 + g + half * 8;
        const uint4 v = *reinterpret_cast<const uint4 *>(w + row * words_per_row + kb * 16 + t * 4);
        *reinterpret_cast<uint4 *>(rec + half * 512 + lane * 16) = v;
        rec[1024 + lane * 2 + half] = s[row * groups_per_row + kb * 4 + t];
    }
}

// ---- plain SIMT kernel on the MLX layout (stand-alone API, any rows) ----------
// One warp per row; lane L owns scale groups L, L+32, ... (a 16-byte load is one
// whole group), fp32 fmaf, shuffle tree.
__global__ void __launch_bounds__(256) gemv_mlx_kernel(const uint32_t *__restrict__ w, const uint8_t *__restrict__ s,
                                                       const float *__restrict__ x, float *__restrict__ y, int rows,
                                                       int cols)
{
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int groups = cols >> 5;
    const uint4 *rw = reinterpret_cast<const uint4 *>(w + size_t(row) * groups * 4);
    const uint8_t *rs = s + size_t(row) * groups;
    float sum = 0.f;
    for (int gi = lane; gi < groups; gi += 32) {
        const uint4 q = ldg_stream(rw + gi);
        const float sc = e8m0_to_float(rs[gi]);
        const uint32_t qq[4] = {q.x, q.y, q.z, q.w};
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
#pragma unroll
            for (int j = 0; j < 8; j++) part = fmaf(e2m1_to_float(qq[i] >> (4 * j)), x[gi * 32 + i * 8 + j], part);
        }
        sum = fmaf(part, sc, sum);
    }
    sum = warp_sum(sum);
    if (lane == 0) y[row] = sum;
}

__global__ void get_row_kernel(const uint32_t *__restrict__ w, const uint8_t *__restrict__ s, float *__restrict__ out,
                               size_t row, int cols)
{
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= cols) return;
    const uint32_t word = w[row * (cols >> 3) + (k >> 3)];
    out[k] = e2m1_to_float(word >> ((k & 7) * 4)) * e8m0_to_float(s[row * (cols >> 5) + (k >> 5)]);
}

__global__ void embed_kernel(const uint32_t *__restrict__ w, const uint8_t *__restrict__ s, float *__restrict__ out,
                             const int *__restrict__ row_ptr, int rows, int cols)
{
    pdl_launch_dependents();
    pdl_wait();
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= cols) return;
    // blockIdx.y: token of a prompt pass (its own row index, its own output row)
    const int row = __ldcg(row_ptr + blockIdx.y);
    out += size_t(blockIdx.y) * cols;
    if (row < 0 || row >= rows) {
        out[k] = 0.f;
        return;
    }
    const uint32_t word = w[size_t(row) * (cols >> 3) + (k >> 3)];
    out[k] = e2m1_to_float(word >> ((k & 7) * 4)) * e8m0_to_float(s[size_t(row) * (cols >> 5) + (k >> 5)]);
}

__global__ void set_scalars_kernel(int *tok, int token, int *pos, int position)
{
    if (tok) *tok = token;
    if (pos) *pos = position;
}

__global__ void dequant_kernel(const uint32_t *__restrict__ w, const uint8_t *__restrict__ s, float *__restrict__ out,
                               size_t total_words, int cols)
{
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total_words) return;
    const uint32_t word = w[i];
    const float sc = e8m0_to_float(s[i >> 2]); // 4 words per group, rows are whole groups
    float4 a, b;
    a.x = e2m1_to_float(word) * sc; a.y = e2m1_to_float(word >> 4) * sc;
    a.z = e2m1_to_float(word >> 8) * sc; a.w = e2m1_to_float(word >> 12) * sc;
    b.x = e2m1_to_float(word >> 16) * sc; b.y = e2m1_to_float(word >> 20) * sc;
    b.z = e2m1_to_float(word >> 24) * sc; b.w = e2m1_to_float(word >> 28) * sc;
    reinterpret_cast<float4 *>(out)[i * 2] = a;
    reinterpret_cast<float4 *>(out)[i * 2 + 1] = b;
    (void)cols;
}

} // namespace insg

using namespace insg;

extern "C" {

size_t insg_mxfp4_packed_bytes(int rows, int cols)
{
    if (rows <= 0 || cols <= 0 || (rows & 15) || (cols & 127)) return 0;
    return size_t(rows >> 4) * (cols >> 7) * kRec;
}

int insg_mxfp4_repack(const uint32_t *weight, const uint8_t *scales, void *packed, int rows, int cols, insg_stream_t stream)
{
    if (!weight || !scales || !packed) return fail(INSG_E_ARG, "repack: null pointer");
    if (rows <= 0 || cols <= 0 || (rows & 15) || (cols & 127)) return fail(INSG_E_SHAPE, "repack: rows % 16 and cols % 128 must be 0");
    const size_t nrec = size_t(rows >> 4) * (cols >> 7);
    const unsigned blocks = unsigned((nrec + 7) / 8);
    repack_kernel<<<blocks, 256, 0, stream>>>(weight, scales, static_cast<uint8_t *>(packed), rows, cols);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? INSG_OK : cuda_fail(e, "repack launch");
}

int insg_mxfp4_gemv_mlx(const uint32_t *weight, const uint8_t *scales, const float *x, float *y, int rows, int cols,
                        insg_stream_t stream)
{
    if (rows <= 0 || cols <= 0 || (cols & 31)) return fail(INSG_E_SHAPE, "gemv_mlx: cols must be a positive multiple of 32");
    if (!weight || !scales || !x || !y) return fail(INSG_E_ARG, "gemv_mlx: null pointer");
    gemv_mlx_kernel<<<(rows + 7) / 8, 256, 0, stream>>>(weight, scales, x, y, rows, cols);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? INSG_OK : cuda_fail(e, "gemv_mlx launch");
}

int insg_mxfp4_get_row_mlx(const uint32_t *weight, const uint8_t *scales, float *out, int row, int cols, insg_stream_t stream)
{
    if (row < 0 || cols <= 0 || (cols & 31)) return fail(INSG_E_SHAPE, "get_row: bad row/cols");
    if (!weight || !scales || !out) return fail(INSG_E_ARG, "get_row: null pointer");
    get_row_kernel<<<(cols + 255) / 256, 256, 0, stream>>>(weight, scales, out, size_t(row), cols);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? INSG_OK : cuda_fail(e, "get_row launch");
}

int insg_mxfp4_embed(const uint32_t *weight, const uint8_t *scales, float *out, const int *device_row, int rows, int cols,
                     int pdl, insg_stream_t stream)
{
    if (!weight || !scales || !out || !device_row) return fail(INSG_E_ARG, "embed: null pointer");
    if (rows <= 0 || cols <= 0 || (cols & 31)) return fail(INSG_E_SHAPE, "embed: bad rows/cols");
    return launch(embed_kernel, dim3((cols + 255) / 256), dim3(256), 0, stream, pdl != 0, weight, scales, out, device_row, rows, cols);
}

int insg_mxfp4_embed_tokens(const uint32_t *weight, const uint8_t *scales, float *out, const int *device_rows, int count, int rows,
                            int cols, int pdl, insg_stream_t stream)
{
    if (!weight || !scales || !out || !device_rows) return fail(INSG_E_ARG, "embed: null pointer");
    if (rows <= 0 || cols <= 0 || (cols & 31) || count < 1 || count > 65535) return fail(INSG_E_SHAPE, "embed: bad rows/cols/count");
    return launch(embed_kernel, dim3((cols + 255) / 256, count), dim3(256), 0, stream, pdl != 0, weight, scales, out, device_rows, rows,
                  cols);
}

int insg_set_scalars(int *device_token, int token, int *device_position, int position, insg_stream_t stream)
{
    set_scalars_kernel<<<1, 1, 0, stream>>>(device_token, token, device_position, position);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? INSG_OK : cuda_fail(e, "set_scalars launch");
}

int insg_mxfp4_dequant_mlx(const uint32_t *weight, const uint8_t *scales, float *out, int rows, int cols, insg_stream_t stream)
{
    if (rows <= 0 || cols <= 0 || (cols & 31)) return fail(INSG_E_SHAPE, "dequant: cols must be a positive multiple of 32");
    if (!weight || !scales || !out) return fail(INSG_E_ARG, "dequant: null pointer");
    const size_t words = size_t(rows) * (cols >> 3);
    dequant_kernel<<<unsigned((words + 255) / 256), 256, 0, stream>>>(weight, scales, out, words, cols);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? INSG_OK : cuda_fail(e, "dequant launch");
}

} // extern "C"
