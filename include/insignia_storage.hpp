// Budgeted residency of checkpoint tensors across three tiers: the mapped file, pinned host memory, device memory.
//
// Drop-in for the reference header of the same name (include/insignia_storage.hpp:11-31, behaviour:
// src/storage.cu:5-11): same public class, methods and error strings.  acquire() makes a tensor resident on the device
// (evicting least-recently-used unpinned tensors until it fits the byte budget), pins it and returns a non-owning view;
// release() unpins.  What is behind that interface is this library's own:
//   * one slot per tensor of the file, in the file's (name-sorted) order, so a lookup is the model's binary search and
//     nothing is hashed or copied per call; unpinned resident slots form an intrusive least-recently-used list;
//   * uploads go file mapping -> pinned staging buffers -> device in chunks on a copy stream of the store's own, the
//     host copy of chunk k+1 overlapping the DMA of chunk k; the consumer stream is made to wait on an event, the host
//     is not;
//   * prefetch() queues a tensor for a background uploader thread, so that the upload overlaps whatever the caller
//     does next (the repack kernel of the previous matrix, for instance); a later acquire() only joins it;
//   * an optional pinned-host cache tier keeps the bytes of uploaded tensors, so a tensor evicted under a budget
//     smaller than the model comes back by DMA alone;
//   * reserve() charges device memory that other parts of the engine allocate for weights (the repacked copies) to
//     the same budget.
// MemoryTier (declared and unused by the reference, include/insignia_storage.hpp:11) is what tier() reports.
#pragma once
#include "insignia_model.hpp"

#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <string>
#include <string_view>
#include <vector>

namespace insignia {

enum class MemoryTier : uint8_t { nvme_mapped, host_pinned, device };

struct DeviceView {
    void *data{};
    uint64_t bytes{};
    DType dtype{};
    const std::vector<uint64_t> *shape{};
    explicit operator bool() const noexcept { return data != nullptr; }
};

// Additive: where device memory comes from.  The default talks to the CUDA runtime; a host-memory stand-in exists so
// that the residency logic (budget, eviction order, errors, prefetch) can be exercised on a machine without a GPU.
struct StorageBackend {
    virtual ~StorageBackend() = default;
    virtual void *device_alloc(uint64_t bytes) = 0;             // throws std::runtime_error
    virtual void device_free(void *p) noexcept = 0;
    virtual void *pinned_alloc(uint64_t bytes) = 0;             // throws std::runtime_error
    virtual void pinned_free(void *p) noexcept = 0;
    // copy `bytes` from pinned host memory to the device on the store's copy stream; returns after queueing
    virtual void copy_to_device(void *dst, const void *pinned_src, uint64_t bytes) = 0;
    virtual uint64_t record() = 0;                              // marks the copy stream; returns a ticket
    virtual void host_wait(uint64_t ticket) = 0;                // host blocks until the ticket's point is reached
    virtual void consumer_wait(uint64_t ticket, cudaStream_t consumer) = 0; // the consumer stream waits for it
    virtual void sync_consumer(cudaStream_t consumer) = 0;      // before memory the consumer may still read is freed
};
INSIGNIA_API std::unique_ptr<StorageBackend> make_cuda_backend();
INSIGNIA_API std::unique_ptr<StorageBackend> make_host_backend(); // "device" = malloc: for tests without a GPU

struct StorageStats {
    uint64_t uploads{}, upload_bytes{}, evictions{}, hits{}, pinned_cache_hits{}, prefetches{};
};

class INSIGNIA_API TieredStorage final {
public:
    TieredStorage(const ModelFile &model, uint64_t device_budget_bytes, cudaStream_t stream = nullptr);
    // Additive: explicit backend.
    TieredStorage(const ModelFile &model, uint64_t device_budget_bytes, cudaStream_t stream, std::unique_ptr<StorageBackend> backend);
    ~TieredStorage();
    TieredStorage(const TieredStorage &) = delete;
    TieredStorage &operator=(const TieredStorage &) = delete;

    DeviceView acquire(std::string_view name);
    void release(std::string_view name) noexcept;
    void clear();
    uint64_t device_bytes() const noexcept;
    uint64_t budget_bytes() const noexcept { return budget_; }

    // Additive.
    const ModelFile &model() const noexcept { return model_; }
    // Starts the upload of a tensor in the background (no pin); false when it is absent from the file.  A tensor that
    // does not fit right now (everything else pinned) is simply not prefetched.
    bool prefetch(std::string_view name);
    MemoryTier tier(std::string_view name) const;
    // Charges / returns device bytes allocated elsewhere for weights; evicts unpinned tensors to make room and throws
    // the budget errors of acquire() when it cannot.
    void reserve(uint64_t bytes);
    void unreserve(uint64_t bytes) noexcept;
    uint64_t reserved_bytes() const noexcept;
    // Pinned-host cache tier: bytes of uploaded tensors kept in pinned memory (0 = off, the default).
    void set_host_cache_bytes(uint64_t bytes);
    StorageStats stats() const;

private:
    struct Impl;
    const ModelFile &model_;
    uint64_t budget_{};
    std::unique_ptr<Impl> impl_;
};

} // namespace insignia
