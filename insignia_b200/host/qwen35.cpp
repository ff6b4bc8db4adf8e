// insignia::Qwen35Weights (interface: include/insignia_qwen35.hpp; reference behaviour: src/qwen35.cu:5-9).
#include "insignia_qwen35.hpp"

#include "insignia_b200.h"

#include <stdexcept>

namespace insignia {

Qwen35Weights::Qwen35Weights(const ModelFile &model, uint64_t device_budget_bytes, cudaStream_t stream)
    : storage_(model, device_budget_bytes, stream), stream_(stream)
{
}

Qwen35Weights::~Qwen35Weights()
{
    cudaStreamSynchronize(stream_);
    for (auto &kv : packed_) {
        cudaFree(const_cast<void *>(kv.second.data));
        storage_.unreserve(kv.second.bytes);
    }
}

QuantMatrix Qwen35Weights::matrix(const std::string &base)
{
    DeviceView w = storage_.acquire(base + ".weight");
    DeviceView s;
    try {
        s = storage_.acquire(base + ".scales");
    } catch (...) {
        storage_.release(base + ".weight");
        throw;
    }
    auto bad = [&](const std::string &msg) {
        release(base);
        throw std::runtime_error(msg + base);
    };
    if (w.dtype != DType::u32 || s.dtype != DType::u8 || !w.shape || w.shape->size() != 2) bad("not an MXFP4 matrix: ");
    const int rows = int((*w.shape)[0]), cols = int((*w.shape)[1]) * 8;
    if (s.bytes != uint64_t(rows) * uint64_t(cols / 32)) bad("MXFP4 scale shape mismatch: ");
    return QuantMatrix{w, s, rows, cols};
}

void Qwen35Weights::release(const std::string &base) noexcept
{
    storage_.release(base + ".weight");
    storage_.release(base + ".scales");
}

void Qwen35Weights::embed(int token, float *device_hidden)
{
    if (token < 0 || token >= Qwen35Shape::vocab) throw std::runtime_error("token out of range");
    const std::string base = "language_model.model.embed_tokens";
    QuantMatrix m = matrix(base);
    const int rc = insg_mxfp4_get_row_mlx(static_cast<const uint32_t *>(m.weight.data), static_cast<const uint8_t *>(m.scales.data),
                                          device_hidden, token, Qwen35Shape::hidden, stream_);
    release(base);
    if (rc != INSG_OK) throw std::runtime_error(insg_last_error());
}

void Qwen35Weights::prefetch(const std::string &base)
{
    if (packed_.count(base + "#rec") || packed_.count(base + "#umma")) return; // the checkpoint-layout copy is not needed again
    storage_.prefetch(base + ".weight");
    storage_.prefetch(base + ".scales");
}

PackedMatrix Qwen35Weights::packed(const std::string &base, int layout)
{
    const std::string key = base + (layout ? "#umma" : "#rec");
    if (auto it = packed_.find(key); it != packed_.end()) return it->second;
    QuantMatrix m = matrix(base);
    PackedMatrix p;
    p.rows = m.rows;
    p.cols = m.cols;
    p.layout = layout;
    p.bytes = layout ? insg_mxfp4_packed_umma_bytes(m.rows, m.cols) : insg_mxfp4_packed_bytes(m.rows, m.cols);
    if (p.bytes == 0) {
        release(base);
        throw std::runtime_error("matrix shape not packable (rows % 16, cols % 128): " + base);
    }
    // The packed copy is weight memory like any other: it is charged to the storage budget (unpinned checkpoint-layout
    // copies are evicted to make room; the budget errors are the storage's).
    try {
        storage_.reserve(p.bytes);
    } catch (...) {
        release(base);
        throw;
    }
    void *d = nullptr;
    cudaError_t e = cudaMalloc(&d, p.bytes);
    if (e != cudaSuccess) {
        storage_.unreserve(p.bytes);
        release(base);
        throw std::runtime_error(std::string("cudaMalloc packed matrix: ") + cudaGetErrorString(e));
    }
    const auto *wp = static_cast<const uint32_t *>(m.weight.data);
    const auto *sp = static_cast<const uint8_t *>(m.scales.data);
    const int rc = layout ? insg_mxfp4_repack_umma(wp, sp, d, m.rows, m.cols, stream_) : insg_mxfp4_repack(wp, sp, d, m.rows, m.cols, stream_);
    e = cudaStreamSynchronize(stream_);
    release(base); // the MLX copy becomes evictable again
    if (rc != INSG_OK || e != cudaSuccess) {
        cudaFree(d);
        storage_.unreserve(p.bytes);
        throw std::runtime_error(rc != INSG_OK ? insg_last_error() : cudaGetErrorString(e));
    }
    p.data = d;
    packed_bytes_ += p.bytes;
    packed_.emplace(key, p);
    return p;
}

} // namespace insignia
