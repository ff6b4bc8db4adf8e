// insignia::TieredStorage: three-tier residency of checkpoint tensors (interface and design notes:
// include/insignia_storage.hpp; reference contract: src/storage.cu:5-11 -- budget, pins, least-recently-used eviction,
// error strings).
#include "insignia_storage.hpp"

#include <algorithm>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <mutex>
#include <stdexcept>
#include <thread>

namespace insignia {
namespace {

constexpr uint64_t kStageBytes = uint64_t(32) << 20; // one pinned staging buffer
constexpr int kStages = 2;

[[noreturn]] void cuda_throw(cudaError_t e, const char *what) { throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e)); }
void cuda_ok(cudaError_t e, const char *what)
{
    if (e != cudaSuccess) cuda_throw(e, what);
}

class CudaBackend final : public StorageBackend {
public:
    CudaBackend()
    {
        cuda_ok(cudaGetDevice(&device_), "cudaGetDevice");
        cuda_ok(cudaStreamCreateWithFlags(&copy_, cudaStreamNonBlocking), "create copy stream");
    }
    ~CudaBackend() override
    {
        for (cudaEvent_t e : events_) cudaEventDestroy(e);
        cudaStreamDestroy(copy_);
    }
    void *device_alloc(uint64_t bytes) override
    {
        bind();
        void *p = nullptr;
        cuda_ok(cudaMalloc(&p, size_t(bytes ? bytes : 1)), "cudaMalloc tensor");
        return p;
    }
    void device_free(void *p) noexcept override
    {
        bind();
        cudaFree(p);
    }
    void *pinned_alloc(uint64_t bytes) override
    {
        bind();
        void *p = nullptr;
        cuda_ok(cudaHostAlloc(&p, size_t(bytes ? bytes : 1), cudaHostAllocDefault), "cudaHostAlloc");
        return p;
    }
    void pinned_free(void *p) noexcept override { cudaFreeHost(p); }
    void copy_to_device(void *dst, const void *src, uint64_t bytes) override
    {
        bind();
        cuda_ok(cudaMemcpyAsync(dst, src, size_t(bytes), cudaMemcpyHostToDevice, copy_), "upload tensor");
    }
    uint64_t record() override
    {
        bind();
        std::lock_guard<std::mutex> lock(mu_);
        const uint64_t ticket = next_++;
        const size_t slot = size_t(ticket % kRing);
        if (events_.size() <= slot) {
            cudaEvent_t e;
            cuda_ok(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "create event");
            events_.push_back(e);
        }
        cuda_ok(cudaEventRecord(events_[slot], copy_), "record event");
        return ticket;
    }
    void host_wait(uint64_t ticket) override
    {
        cudaEvent_t e = event_of(ticket);
        if (e) cuda_ok(cudaEventSynchronize(e), "finish tensor upload");
        else cuda_ok(cudaStreamSynchronize(copy_), "finish tensor upload"); // the event was reused: everything older is done once the stream is
    }
    void consumer_wait(uint64_t ticket, cudaStream_t consumer) override
    {
        cudaEvent_t e = event_of(ticket);
        if (e) cuda_ok(cudaStreamWaitEvent(consumer, e, 0), "wait for tensor upload");
        else cuda_ok(cudaStreamSynchronize(copy_), "finish tensor upload");
    }
    void sync_consumer(cudaStream_t consumer) override { cuda_ok(cudaStreamSynchronize(consumer), "synchronize before eviction"); }

private:
    static constexpr uint64_t kRing = 64;
    void bind() { cudaSetDevice(device_); } // the uploader thread starts without a current device
    cudaEvent_t event_of(uint64_t ticket)
    {
        std::lock_guard<std::mutex> lock(mu_);
        if (ticket + kRing < next_) return nullptr; // its ring entry has been recorded again since
        return events_[size_t(ticket % kRing)];
    }
    int device_ = 0;
    cudaStream_t copy_{};
    std::mutex mu_;
    std::vector<cudaEvent_t> events_;
    uint64_t next_ = 0;
};

// Host memory in place of device memory; copies complete at once.  For exercising the store without a GPU.
class HostBackend final : public StorageBackend {
public:
    void *device_alloc(uint64_t bytes) override
    {
        void *p = std::malloc(size_t(bytes ? bytes : 1));
        if (!p) throw std::runtime_error("cudaMalloc tensor: out of memory");
        return p;
    }
    void device_free(void *p) noexcept override { std::free(p); }
    void *pinned_alloc(uint64_t bytes) override { return device_alloc(bytes); }
    void pinned_free(void *p) noexcept override { std::free(p); }
    void copy_to_device(void *dst, const void *src, uint64_t bytes) override { std::memcpy(dst, src, size_t(bytes)); }
    uint64_t record() override { return 0; }
    void host_wait(uint64_t) override {}
    void consumer_wait(uint64_t, cudaStream_t) override {}
    void sync_consumer(cudaStream_t) override {}
};

} // namespace

std::unique_ptr<StorageBackend> make_cuda_backend() { return std::make_unique<CudaBackend>(); }
std::unique_ptr<StorageBackend> make_host_backend() { return std::make_unique<HostBackend>(); }

// ------------------------------------------------------------------------------------------------- implementation
struct TieredStorage::Impl {
    enum State : uint8_t { Absent, Loading, Resident };
    struct Slot {
        void *device = nullptr;
        void *pinned = nullptr;    // copy in the pinned-host cache tier, or null
        uint32_t pins = 0;
        State state = Absent;
        bool in_lru = false, queued = false;
        int prev = -1, next = -1;  // least-recently-used list of unpinned resident slots
        int cprev = -1, cnext = -1; // least-recently-used list of the pinned-host cache
        uint64_t ready = 0;        // ticket after which the device copy is complete
        bool ready_valid = false;
    };

    const ModelFile &model;
    uint64_t &budget;
    cudaStream_t consumer;
    std::unique_ptr<StorageBackend> be;
    mutable std::mutex mu;           // slots, lists, counters
    std::condition_variable cv;      // a Loading slot became Resident (or Absent again)
    std::vector<Slot> slots;
    int lru_head = -1, lru_tail = -1; // head = least recently used
    int cache_head = -1, cache_tail = -1;
    uint64_t used = 0, reserved = 0, cache_used = 0, cache_budget = 0;
    StorageStats st;
    // staging pipeline (one upload at a time)
    std::mutex upload_mu;
    void *stage[kStages] = {nullptr, nullptr};
    uint64_t stage_ticket[kStages] = {0, 0};
    bool stage_busy[kStages] = {false, false};
    // background uploader
    std::thread worker;
    std::deque<int> queue;
    std::condition_variable qcv;
    bool stop = false;

    Impl(const ModelFile &m, uint64_t &b, cudaStream_t s, std::unique_ptr<StorageBackend> backend)
        : model(m), budget(b), consumer(s), be(std::move(backend)), slots(m.tensors().size())
    {
    }

    int index_of(std::string_view name) const
    {
        const TensorView *t = model.find(name);
        return t ? int(t - model.tensors().data()) : -1;
    }
    const TensorView &tensor(int i) const { return model.tensors()[size_t(i)]; }

    // ---- intrusive lists ----
    void lru_push(int i)
    {
        Slot &s = slots[size_t(i)];
        s.prev = lru_tail;
        s.next = -1;
        if (lru_tail >= 0) slots[size_t(lru_tail)].next = i;
        else lru_head = i;
        lru_tail = i;
        s.in_lru = true;
    }
    void lru_remove(int i)
    {
        Slot &s = slots[size_t(i)];
        if (!s.in_lru) return;
        if (s.prev >= 0) slots[size_t(s.prev)].next = s.next;
        else lru_head = s.next;
        if (s.next >= 0) slots[size_t(s.next)].prev = s.prev;
        else lru_tail = s.prev;
        s.prev = s.next = -1;
        s.in_lru = false;
    }
    void cache_push(int i)
    {
        Slot &s = slots[size_t(i)];
        s.cprev = cache_tail;
        s.cnext = -1;
        if (cache_tail >= 0) slots[size_t(cache_tail)].cnext = i;
        else cache_head = i;
        cache_tail = i;
    }
    void cache_remove(int i)
    {
        Slot &s = slots[size_t(i)];
        if (s.cprev >= 0) slots[size_t(s.cprev)].cnext = s.cnext;
        else if (cache_head == i) cache_head = s.cnext;
        if (s.cnext >= 0) slots[size_t(s.cnext)].cprev = s.cprev;
        else if (cache_tail == i) cache_tail = s.cprev;
        s.cprev = s.cnext = -1;
    }

    // Frees unpinned resident tensors, oldest use first, until `bytes` more fit.  Caller holds mu.
    void make_room(uint64_t bytes, bool quiet)
    {
        if (bytes > budget) throw std::runtime_error("tensor exceeds device budget");
        bool synced = false;
        while (used + reserved + bytes > budget) {
            const int victim = lru_head;
            if (victim < 0) {
                if (quiet) throw std::runtime_error("");
                throw std::runtime_error("device budget exhausted by pinned tensors");
            }
            if (!synced) { // kernels already queued on the consumer stream may still read the victim
                be->sync_consumer(consumer);
                synced = true;
            }
            Slot &s = slots[size_t(victim)];
            lru_remove(victim);
            be->device_free(s.device);
            s.device = nullptr;
            s.state = Absent;
            s.ready_valid = false;
            used -= tensor(victim).bytes;
            st.evictions++;
        }
    }

    // The pinned-host cache keeps the most recently uploaded tensors within its own budget.  Caller holds mu.
    void *cache_take(int i, uint64_t bytes)
    {
        if (cache_budget == 0 || bytes > cache_budget) return nullptr;
        while (cache_used + bytes > cache_budget && cache_head >= 0) {
            const int v = cache_head;
            cache_remove(v);
            be->pinned_free(slots[size_t(v)].pinned);
            slots[size_t(v)].pinned = nullptr;
            cache_used -= tensor(v).bytes;
        }
        if (cache_used + bytes > cache_budget) return nullptr;
        void *p = be->pinned_alloc(bytes);
        cache_used += bytes;
        cache_push(i);
        return p;
    }

    // Moves the tensor's bytes to `dst`.  From the pinned cache: one DMA.  From the mapping: through the staging
    // buffers, the host copy of a chunk overlapping the DMA of the chunk before.  Caller holds upload_mu, not mu.
    uint64_t transfer(int i, void *dst, void *pinned_copy, bool fill_cache)
    {
        const TensorView &t = tensor(i);
        if (pinned_copy && !fill_cache) {
            be->copy_to_device(dst, pinned_copy, t.bytes);
            return be->record();
        }
        uint64_t ticket = 0;
        bool have = false;
        int k = 0;
        for (uint64_t off = 0; off < t.bytes; off += kStageBytes, k ^= 1) {
            const uint64_t n = std::min(kStageBytes, t.bytes - off);
            const void *src;
            if (pinned_copy) { // filling the cache: its pinned buffer is the staging area
                std::memcpy(static_cast<uint8_t *>(pinned_copy) + off, t.data + off, size_t(n));
                src = static_cast<uint8_t *>(pinned_copy) + off;
            } else {
                if (!stage[k]) stage[k] = be->pinned_alloc(kStageBytes);
                if (stage_busy[k]) be->host_wait(stage_ticket[k]); // its last DMA must have drained
                std::memcpy(stage[k], t.data + off, size_t(n));
                src = stage[k];
            }
            be->copy_to_device(static_cast<uint8_t *>(dst) + off, src, n);
            ticket = be->record();
            have = true;
            if (!pinned_copy) {
                stage_ticket[k] = ticket;
                stage_busy[k] = true;
            }
        }
        if (!have) ticket = be->record();
        return ticket;
    }

    // Makes slot i resident (state Absent on entry, caller holds `lock` on mu).  Returns with mu held.
    void load(int i, std::unique_lock<std::mutex> &lock, bool quiet)
    {
        const TensorView &t = tensor(i);
        Slot &s = slots[size_t(i)];
        make_room(t.bytes, quiet);
        void *d = be->device_alloc(t.bytes);
        used += t.bytes;
        s.device = d;
        s.state = Loading;
        void *pinned = s.pinned;
        bool fill = false;
        if (!pinned) {
            pinned = cache_take(i, t.bytes);
            fill = pinned != nullptr;
            s.pinned = pinned;
        } else {
            st.pinned_cache_hits++;
            cache_remove(i);
            cache_push(i);
        }
        lock.unlock();
        uint64_t ticket = 0;
        try {
            std::lock_guard<std::mutex> up(upload_mu);
            ticket = transfer(i, d, pinned, fill);
        } catch (...) {
            lock.lock();
            be->device_free(d);
            used -= t.bytes;
            s.device = nullptr;
            s.state = Absent;
            cv.notify_all();
            throw;
        }
        lock.lock();
        s.ready = ticket;
        s.ready_valid = true;
        s.state = Resident;
        st.uploads++;
        st.upload_bytes += t.bytes;
        cv.notify_all();
    }

    void worker_main()
    {
        std::unique_lock<std::mutex> lock(mu);
        for (;;) {
            qcv.wait(lock, [&] { return stop || !queue.empty(); });
            if (stop) return;
            const int i = queue.front();
            queue.pop_front();
            Slot &s = slots[size_t(i)];
            s.queued = false;
            if (s.state != Absent) continue;
            try {
                load(i, lock, true);
                if (s.pins == 0 && !s.in_lru) lru_push(i);
            } catch (...) {
                // a prefetch that does not fit or fails is dropped; acquire() will report the error if it matters
            }
        }
    }
};

TieredStorage::TieredStorage(const ModelFile &model, uint64_t device_budget_bytes, cudaStream_t stream)
    : TieredStorage(model, device_budget_bytes, stream, nullptr)
{
}

TieredStorage::TieredStorage(const ModelFile &model, uint64_t device_budget_bytes, cudaStream_t stream, std::unique_ptr<StorageBackend> backend)
    : model_(model), budget_(device_budget_bytes)
{
    // the CUDA backend is created on first use, so that constructing a store needs no device (as in the reference)
    impl_ = std::make_unique<Impl>(model, budget_, stream, std::move(backend));
}

TieredStorage::~TieredStorage()
{
    try {
        clear();
    } catch (...) {
    }
    Impl &m = *impl_;
    {
        std::lock_guard<std::mutex> lock(m.mu);
        m.stop = true;
    }
    m.qcv.notify_all();
    if (m.worker.joinable()) m.worker.join();
    if (m.be)
        for (void *&p : m.stage)
            if (p) m.be->pinned_free(p);
}

static void ensure_backend(std::unique_ptr<StorageBackend> &be)
{
    if (!be) be = make_cuda_backend();
}

DeviceView TieredStorage::acquire(std::string_view name)
{
    Impl &m = *impl_;
    const int i = m.index_of(name);
    if (i < 0) throw std::runtime_error("tensor not found: " + std::string(name));
    const TensorView &t = m.tensor(i);
    std::unique_lock<std::mutex> lock(m.mu);
    ensure_backend(m.be);
    Impl::Slot &s = m.slots[size_t(i)];
    m.cv.wait(lock, [&] { return s.state != Impl::Loading; }); // join an upload the prefetcher has in flight
    if (s.state == Impl::Resident) m.st.hits++;
    else m.load(i, lock, false);
    m.lru_remove(i);
    s.pins++;
    if (s.ready_valid) {
        // the copy may still be in flight on the store's copy stream: order the consumer stream behind it
        const uint64_t ticket = s.ready;
        s.ready_valid = false;
        lock.unlock();
        m.be->consumer_wait(ticket, m.consumer);
    }
    return DeviceView{s.device, t.bytes, t.dtype, &t.shape};
}

void TieredStorage::release(std::string_view name) noexcept
{
    Impl &m = *impl_;
    const int i = m.index_of(name);
    if (i < 0) return;
    std::lock_guard<std::mutex> lock(m.mu);
    Impl::Slot &s = m.slots[size_t(i)];
    if (s.pins == 0) return;
    if (--s.pins == 0 && s.state == Impl::Resident) m.lru_push(i); // most recently used end
}

bool TieredStorage::prefetch(std::string_view name)
{
    Impl &m = *impl_;
    const int i = m.index_of(name);
    if (i < 0) return false;
    std::lock_guard<std::mutex> lock(m.mu);
    ensure_backend(m.be);
    Impl::Slot &s = m.slots[size_t(i)];
    if (s.state != Impl::Absent || s.queued) return true;
    s.queued = true;
    m.queue.push_back(i);
    m.st.prefetches++;
    if (!m.worker.joinable()) m.worker = std::thread([&m] { m.worker_main(); });
    m.qcv.notify_one();
    return true;
}

MemoryTier TieredStorage::tier(std::string_view name) const
{
    const Impl &m = *impl_;
    const int i = m.index_of(name);
    if (i < 0) throw std::runtime_error("tensor not found: " + std::string(name));
    std::lock_guard<std::mutex> lock(m.mu);
    const Impl::Slot &s = m.slots[size_t(i)];
    if (s.state == Impl::Resident) return MemoryTier::device;
    return s.pinned ? MemoryTier::host_pinned : MemoryTier::nvme_mapped;
}

void TieredStorage::reserve(uint64_t bytes)
{
    Impl &m = *impl_;
    std::lock_guard<std::mutex> lock(m.mu);
    ensure_backend(m.be);
    m.make_room(bytes, false);
    m.reserved += bytes;
}

void TieredStorage::unreserve(uint64_t bytes) noexcept
{
    Impl &m = *impl_;
    std::lock_guard<std::mutex> lock(m.mu);
    m.reserved -= std::min(bytes, m.reserved);
}

uint64_t TieredStorage::reserved_bytes() const noexcept
{
    std::lock_guard<std::mutex> lock(impl_->mu);
    return impl_->reserved;
}

uint64_t TieredStorage::device_bytes() const noexcept
{
    std::lock_guard<std::mutex> lock(impl_->mu);
    return impl_->used;
}

void TieredStorage::set_host_cache_bytes(uint64_t bytes)
{
    std::lock_guard<std::mutex> lock(impl_->mu);
    impl_->cache_budget = bytes;
}

StorageStats TieredStorage::stats() const
{
    std::lock_guard<std::mutex> lock(impl_->mu);
    return impl_->st;
}

void TieredStorage::clear()
{
    Impl &m = *impl_;
    std::unique_lock<std::mutex> lock(m.mu);
    m.queue.clear();
    for (Impl::Slot &s : m.slots) s.queued = false;
    m.cv.wait(lock, [&] {
        for (const Impl::Slot &s : m.slots)
            if (s.state == Impl::Loading) return false;
        return true;
    });
    if (!m.be) return; // nothing was ever made resident
    m.be->sync_consumer(m.consumer);
    for (size_t i = 0; i < m.slots.size(); i++) {
        Impl::Slot &s = m.slots[i];
        if (s.device) m.be->device_free(s.device);
        if (s.pinned) m.be->pinned_free(s.pinned);
        s = Impl::Slot{};
    }
    m.lru_head = m.lru_tail = m.cache_head = m.cache_tail = -1;
    m.used = 0;
    m.cache_used = 0;
}

} // namespace insignia
