// Budgeted device residency for checkpoint tensors: pin counts + LRU eviction.
//
// Drop-in for the reference header of the same name (include/insignia_storage.hpp:11-31,
// behaviour: src/storage.cu:5-11).  acquire() uploads a tensor from the mapped
// file on first use (evicting least-recently-used unpinned tensors until it fits
// the byte budget), pins it and returns a non-owning view; release() unpins.
// Error strings are the reference's.
#pragma once
#include "insignia_model.hpp"

#include <cuda_runtime.h>

#include <cstdint>
#include <string>
#include <string_view>
#include <unordered_map>

namespace insignia {

// Declared by the reference and unused there too (include/insignia_storage.hpp:11).
enum class MemoryTier : uint8_t { nvme_mapped, host_pinned, device };

struct DeviceView {
    void *data{};
    uint64_t bytes{};
    DType dtype{};
    const std::vector<uint64_t> *shape{};
    explicit operator bool() const noexcept { return data != nullptr; }
};

class INSIGNIA_API TieredStorage final {
public:
    TieredStorage(const ModelFile &model, uint64_t device_budget_bytes, cudaStream_t stream = nullptr);
    ~TieredStorage();
    TieredStorage(const TieredStorage &) = delete;
    TieredStorage &operator=(const TieredStorage &) = delete;

    DeviceView acquire(std::string_view name);
    void release(std::string_view name) noexcept;
    void clear();
    uint64_t device_bytes() const noexcept { return used_; }
    uint64_t budget_bytes() const noexcept { return budget_; }
    // Additive: the file the storage reads from.
    const ModelFile &model() const noexcept { return model_; }

private:
    struct Entry {
        void *device{};
        uint64_t bytes{};
        uint32_t pins{};
        uint64_t tick{};
        const TensorView *host{};
    };
    void make_room(uint64_t bytes);
    const ModelFile &model_;
    uint64_t budget_{}, used_{}, tick_{};
    cudaStream_t stream_{};
    std::unordered_map<std::string, Entry> entries_;
};

} // namespace insignia
