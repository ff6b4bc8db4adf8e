// Weight facade for the Qwen3.5-style hybrid: shape constants, MXFP4 matrix lookup, embedding.
//
// Drop-in for the reference header of the same name (include/insignia_qwen35.hpp:7-19,
// behaviour: src/qwen35.cu:5-9).  Additive: packed(), which hands the decode
// kernels a tile-interleaved copy of a matrix built once on first use.
#pragma once
#include "insignia_model.hpp"
#include "insignia_storage.hpp"

#include <cuda_runtime.h>

#include <memory>
#include <string>
#include <unordered_map>

namespace insignia {

struct Qwen35Shape {
    static constexpr int hidden = 4096, intermediate = 12288, layers = 32, vocab = 248320;
    static constexpr bool full_attention(int i) { return (i & 3) == 3; }
};

// MLX-layout matrix: weight U32[rows][cols/8], scales U8[rows][cols/32]; pinned until release().
struct QuantMatrix {
    DeviceView weight, scales;
    int rows{}, cols{};
};

// Tile-interleaved copy (see insg_mxfp4_repack); owned by Qwen35Weights, lives until it is destroyed; its bytes are
// charged to the storage budget (TieredStorage::reserve).
struct PackedMatrix {
    const void *data{};
    int rows{}, cols{};
    uint64_t bytes{};
    int layout{}; // 0: 16-row records (insg_mxfp4_repack), 1: 128-row tcgen05 images (insg_mxfp4_repack_umma)
};

class INSIGNIA_API Qwen35Weights final {
public:
    Qwen35Weights(const ModelFile &model, uint64_t device_budget_bytes, cudaStream_t stream = nullptr);
    ~Qwen35Weights();
    // Dequantises row `token` of embed_tokens into device_hidden[4096]; throws "token out of range".
    void embed(int token, float *device_hidden);
    // Acquires base+".weight"/".scales"; throws "not an MXFP4 matrix: ..." / "MXFP4 scale shape mismatch: ...".
    QuantMatrix matrix(const std::string &base);
    void release(const std::string &base) noexcept;
    TieredStorage &storage() noexcept { return storage_; }

    // Additive: packed copy of matrix `base` for the fused GEMV kernels (built on first call).
    PackedMatrix packed(const std::string &base, int layout = 0);
    uint64_t packed_bytes() const noexcept { return packed_bytes_; }
    // Additive: starts the upload of a matrix' checkpoint-layout tensors in the background (see TieredStorage::prefetch).
    void prefetch(const std::string &base);

private:
    TieredStorage storage_;
    cudaStream_t stream_{};
    std::unordered_map<std::string, PackedMatrix> packed_;
    uint64_t packed_bytes_{};
};

} // namespace insignia
