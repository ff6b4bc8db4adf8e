// insignia::TieredStorage: byte-budgeted device residency with pin counts and LRU eviction
// (interface: include/insignia_storage.hpp; reference behaviour: src/storage.cu:5-11).
#include "insignia_storage.hpp"

#include <stdexcept>

namespace insignia {
namespace {
void check(cudaError_t e, const char *what)
{
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
} // namespace

TieredStorage::TieredStorage(const ModelFile &model, uint64_t device_budget_bytes, cudaStream_t stream)
    : model_(model), budget_(device_budget_bytes), stream_(stream)
{
}

TieredStorage::~TieredStorage()
{
    try {
        clear();
    } catch (...) {
    }
}

// Evicts unpinned tensors, least recently used first, until `bytes` more fit.
void TieredStorage::make_room(uint64_t bytes)
{
    if (bytes > budget_) throw std::runtime_error("tensor exceeds device budget");
    while (used_ + bytes > budget_) {
        auto victim = entries_.end();
        for (auto it = entries_.begin(); it != entries_.end(); ++it) {
            const Entry &e = it->second;
            if (!e.device || e.pins != 0) continue;
            if (victim == entries_.end() || e.tick < victim->second.tick) victim = it;
        }
        if (victim == entries_.end()) throw std::runtime_error("device budget exhausted by pinned tensors");
        check(cudaStreamSynchronize(stream_), "synchronize before eviction");
        check(cudaFree(victim->second.device), "cudaFree");
        used_ -= victim->second.bytes;
        entries_.erase(victim);
    }
}

DeviceView TieredStorage::acquire(std::string_view name)
{
    std::string key(name);
    if (auto it = entries_.find(key); it != entries_.end()) {
        Entry &e = it->second;
        e.pins++;
        e.tick = ++tick_;
        return DeviceView{e.device, e.bytes, e.host->dtype, &e.host->shape};
    }
    const TensorView *t = model_.find(name);
    if (!t) throw std::runtime_error("tensor not found: " + key);
    make_room(t->bytes);
    void *d = nullptr;
    check(cudaMalloc(&d, size_t(t->bytes ? t->bytes : 1)), "cudaMalloc tensor");
    try {
        check(cudaMemcpyAsync(d, t->data, size_t(t->bytes), cudaMemcpyHostToDevice, stream_), "upload tensor");
        check(cudaStreamSynchronize(stream_), "finish tensor upload");
    } catch (...) {
        cudaFree(d);
        throw;
    }
    used_ += t->bytes;
    entries_.emplace(std::move(key), Entry{d, t->bytes, 1, ++tick_, t});
    return DeviceView{d, t->bytes, t->dtype, &t->shape};
}

void TieredStorage::release(std::string_view name) noexcept
{
    auto it = entries_.find(std::string(name));
    if (it != entries_.end() && it->second.pins) it->second.pins--;
}

void TieredStorage::clear()
{
    check(cudaStreamSynchronize(stream_), "synchronize clear");
    for (auto &kv : entries_)
        if (kv.second.device) check(cudaFree(kv.second.device), "cudaFree clear");
    entries_.clear();
    used_ = 0;
}

} // namespace insignia
