// One-shot all-reduce (sum) of a short fp32 vector over NVLink peer memory: the exchange step of a tensor-parallel
// decode block (one fp32[4096] sum after each row-sharded projection), where a collective library's launch and
// protocol latency, not bandwidth, is the cost.
//
// The reference has no collective call site (it is single-GPU); this is the building block its roadmap names for a
// tensor-parallel run.  Protocol, per rank, ONE kernel, no fence and no separate flag:
//   1. every thread stores its elements of the rank's vector into slot [rank] of EVERY rank's exchange buffer as
//      8-byte words {value, epoch of this call} (plain peer stores, each one atomic: the epoch is the arrival flag
//      of exactly the value it travels with; each GPU's own memory is only ever read by its own SMs);
//   2. it then polls the same elements of every source slot in its own buffer until their epoch is this call's --
//      bounded by the clock; on expiry the error flag is set and the kernel goes on with whatever is there, so the
//      context stays usable;
//   3. it adds the values IN RANK ORDER (every rank gets bit-identical sums) and writes the result in place.
// Two slot sets alternate by epoch parity: a rank can be at most one call ahead of the slowest reader.  The epoch is
// kept in device memory per CTA, so the launch can be captured in a CUDA graph.  No TMA, no multicast, no library
// kernel touches peer memory.
//
// With fewer GPUs than ranks the ranks cannot be separate launches (kernels that wait on one another may not share a
// GPU); insg_allreduce_oneshot_local runs all ranks of a same-process communicator as ONE cooperative launch
// (blockIdx.y = rank), which is how the protocol is tested on a single GPU.
#include "common.cuh"
#include "host_util.h"

#include <algorithm>
#include <cstring>

namespace insg {

constexpr int kArMaxWorld = 8;
constexpr int kArMaxBlocks = 16;
constexpr int kArThreads = 256;

struct ArRank {
    float *data;                    // this rank's vector, reduced in place
    uint2 *slots[kArMaxWorld];      // slots[p]: base of rank p's slot area ([2 sets][world][max_floats] of {value, epoch}), as seen from this rank
    uint32_t *epoch;                // this rank's per-CTA call counters [kArMaxBlocks]
    int *error_flag;                // this rank's; set to 1 when a wait ran out
    int rank;
};

struct ArParams {
    ArRank r[kArMaxWorld]; // r[blockIdx.y]; a real multi-GPU launch uses r[0] only
    int world, count, max_floats, skip_rank; // skip_rank >= 0: that rank of a local launch stays silent (wait self-test)
    unsigned long long timeout_ns;
};

__device__ __forceinline__ unsigned long long ar_now()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void ar_store(uint2 *p, float v, uint32_t e)
{
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(e) : "memory");
}
__device__ __forceinline__ uint2 ar_load(const uint2 *p)
{
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kArThreads) allreduce_oneshot_kernel(const __grid_constant__ ArParams p)
{
    const ArRank &me = p.r[blockIdx.y];
    if (me.rank == p.skip_rank) return;
    const int b = blockIdx.x, nb = gridDim.x, tid = threadIdx.x, W = p.world;
    const uint32_t e = __ldcg(me.epoch + b) + 1u; // this call's epoch (per CTA: no coordination between the CTAs)
    const size_t set_off = size_t(e & 1u) * W * p.max_floats;
    // the vector is cut by position, the same way for every call of a communicator (a CTA's range may be empty for a short
    // vector; its epoch still advances, so the per-CTA epochs of all ranks move in lock step)
    const int nvec = p.count >> 2, per = ((p.max_floats >> 2) + nb - 1) / nb, v0 = min(nvec, b * per), v1 = min(nvec, v0 + per);
    bool expired = false;

    // 1. my elements, each with the epoch, into my slot on every rank
    for (int i = v0 + tid; i < v1; i += kArThreads) {
        const float4 v = __ldcg(reinterpret_cast<const float4 *>(me.data) + i);
        for (int q = 0; q < W; q++) {
            uint2 *dst = me.slots[q] + set_off + size_t(me.rank) * p.max_floats + size_t(i) * 4;
            ar_store(dst, v.x, e);
            ar_store(dst + 1, v.y, e);
            ar_store(dst + 2, v.z, e);
            ar_store(dst + 3, v.w, e);
        }
    }
    // 2 + 3. every source's elements as they arrive (bounded), summed in rank order
    const uint2 *mine = me.slots[me.rank] + set_off;
    const unsigned long long t0 = ar_now();
    for (int i = v0 + tid; i < v1; i += kArThreads) {
        float a[4] = {0.f, 0.f, 0.f, 0.f};
        for (int q = 0; q < W; q++) {
            const uint2 *src = mine + size_t(q) * p.max_floats + size_t(i) * 4;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint2 v = ar_load(src + j);
                while (v.y != e && !expired) {
                    if (ar_now() - t0 > p.timeout_ns) expired = true;
                    else v = ar_load(src + j);
                }
                a[j] += __uint_as_float(v.x);
            }
        }
        reinterpret_cast<float4 *>(me.data)[i] = make_float4(a[0], a[1], a[2], a[3]);
    }
    if (expired && me.error_flag) *me.error_flag = 1;
    __syncthreads();
    if (tid == 0) me.epoch[b] = e;
}

} // namespace insg

using namespace insg;

struct insg_comm {
    int rank = 0, world = 1, max_floats = 0, device = 0;
    uint8_t *base = nullptr;                 // this rank's exchange buffer
    uint8_t *peer[kArMaxWorld] = {};         // every rank's buffer as mapped here (peer[rank] == base)
    bool opened[kArMaxWorld] = {};
    int *error_flag = nullptr;
    unsigned long long timeout_ns = 1000000000ull;
    size_t slot_bytes() const { return size_t(2) * world * max_floats * sizeof(uint2); }
    size_t flag_bytes() const { return 0; }
    size_t total_bytes() const { return slot_bytes() + flag_bytes() + kArMaxBlocks * sizeof(uint32_t) + 64; }
    ArRank view(float *data) const
    {
        ArRank r = {};
        r.data = data;
        for (int q = 0; q < world; q++) {
            r.slots[q] = reinterpret_cast<uint2 *>(peer[q]);
        }
        r.epoch = reinterpret_cast<uint32_t *>(base + slot_bytes() + flag_bytes());
        r.error_flag = error_flag;
        r.rank = rank;
        return r;
    }
};

namespace {
int ar_blocks(int max_floats) { return std::max(1, std::min(kArMaxBlocks, (max_floats / 4 + kArThreads - 1) / kArThreads)); }
int ar_check(const insg_comm *c, const float *data, int count)
{
    if (!c || !data) return fail(INSG_E_ARG, "allreduce: null argument");
    if (count <= 0 || (count & 3) || count > c->max_floats) return fail(INSG_E_SHAPE, "allreduce: count must be a multiple of 4, <= the communicator's size");
    if (reinterpret_cast<uintptr_t>(data) & 15) return fail(INSG_E_ARG, "allreduce: data must be 16-byte aligned");
    for (int q = 0; q < c->world; q++)
        if (!c->peer[q]) return fail(INSG_E_ARG, "allreduce: communicator not connected");
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev != c->device) return fail(INSG_E_ARG, "allreduce: the communicator belongs to another device than the current one");
    return INSG_OK;
}
} // namespace

extern "C" {

insg_comm *insg_comm_create(int rank, int world, int max_floats)
{
    if (world < 1 || world > kArMaxWorld || rank < 0 || rank >= world || max_floats <= 0 || (max_floats & 3)) {
        fail(INSG_E_ARG, "comm_create: 1 <= world <= 8, 0 <= rank < world, max_floats a positive multiple of 4");
        return nullptr;
    }
    insg_comm *c = new insg_comm;
    c->rank = rank; c->world = world; c->max_floats = max_floats;
    cudaError_t e = cudaGetDevice(&c->device);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&c->base), c->total_bytes());
    if (e == cudaSuccess) e = cudaMemset(c->base, 0, c->total_bytes());
    if (e != cudaSuccess) {
        cuda_fail(e, "comm_create");
        if (c->base) cudaFree(c->base);
        delete c;
        return nullptr;
    }
    c->error_flag = reinterpret_cast<int *>(c->base + c->total_bytes() - 64);
    c->peer[rank] = c->base;
    return c;
}

void insg_comm_destroy(insg_comm *c)
{
    if (!c) return;
    for (int q = 0; q < c->world; q++)
        if (c->opened[q]) cudaIpcCloseMemHandle(c->peer[q]);
    if (c->base) cudaFree(c->base);
    delete c;
}

int insg_comm_handle(insg_comm *c, void *handle64)
{
    if (!c || !handle64) return fail(INSG_E_ARG, "comm_handle: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, c->base);
    if (e != cudaSuccess) return cuda_fail(e, "cudaIpcGetMemHandle");
    std::memcpy(handle64, &h, 64);
    return INSG_OK;
}

int insg_comm_connect(insg_comm *c, const void *handles)
{
    if (!c || !handles) return fail(INSG_E_ARG, "comm_connect: null argument");
    for (int q = 0; q < c->world; q++) {
        if (q == c->rank || c->peer[q]) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, static_cast<const uint8_t *>(handles) + size_t(q) * 64, 64);
        void *ptr = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return cuda_fail(e, "cudaIpcOpenMemHandle (is the peer GPU reachable over NVLink / PCIe?)");
        c->peer[q] = static_cast<uint8_t *>(ptr);
        c->opened[q] = true;
    }
    return INSG_OK;
}

int insg_comm_connect_local(insg_comm **comms, int world)
{
    if (!comms || world < 1 || world > kArMaxWorld) return fail(INSG_E_ARG, "comm_connect_local: bad arguments");
    for (int a = 0; a < world; a++) {
        if (!comms[a] || comms[a]->world != world || comms[a]->rank != a) return fail(INSG_E_ARG, "comm_connect_local: comms[i] must be rank i of `world`");
        if (comms[a]->max_floats != comms[0]->max_floats || comms[a]->device != comms[0]->device)
            return fail(INSG_E_ARG, "comm_connect_local: same size and same device for all ranks");
    }
    for (int a = 0; a < world; a++)
        for (int q = 0; q < world; q++) comms[a]->peer[q] = comms[q]->base;
    return INSG_OK;
}

int insg_comm_set_timeout(insg_comm *c, unsigned long long timeout_ns)
{
    if (!c || timeout_ns == 0 || timeout_ns > 10000000000ull) return fail(INSG_E_ARG, "comm_set_timeout: 1 ns .. 10 s");
    c->timeout_ns = timeout_ns;
    return INSG_OK;
}

int insg_comm_error(insg_comm *c, int *host_out, insg_stream_t stream)
{
    if (!c || !host_out) return fail(INSG_E_ARG, "comm_error: null argument");
    cudaError_t e = cudaMemcpyAsync(host_out, c->error_flag, sizeof(int), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    return e == cudaSuccess ? INSG_OK : cuda_fail(e, "comm_error");
}

int insg_comm_reset(insg_comm *c, insg_stream_t stream)
{
    if (!c) return fail(INSG_E_ARG, "comm_reset: null argument");
    const cudaError_t e = cudaMemsetAsync(c->base, 0, c->total_bytes(), stream);
    return e == cudaSuccess ? INSG_OK : cuda_fail(e, "comm_reset");
}

int insg_allreduce_oneshot(insg_comm *c, float *data, int count, insg_stream_t stream)
{
    const int rc = ar_check(c, data, count);
    if (rc != INSG_OK) return rc;
    ArParams p = {};
    p.r[0] = c->view(data);
    p.world = c->world; p.count = count; p.max_floats = c->max_floats; p.skip_rank = -1; p.timeout_ns = c->timeout_ns;
    return launch(allreduce_oneshot_kernel, dim3(ar_blocks(c->max_floats), 1), dim3(kArThreads), 0, stream, false, p);
}

int insg_allreduce_oneshot_local(insg_comm **comms, float **data, int world, int count, int skip_rank, insg_stream_t stream)
{
    if (!comms || !data || world < 1 || world > kArMaxWorld) return fail(INSG_E_ARG, "allreduce_local: bad arguments");
    ArParams p = {};
    for (int a = 0; a < world; a++) {
        const int rc = ar_check(comms[a], data[a], count);
        if (rc != INSG_OK) return rc;
        if (comms[a]->world != world) return fail(INSG_E_ARG, "allreduce_local: world mismatch");
        p.r[a] = comms[a]->view(data[a]);
    }
    p.world = world; p.count = count; p.max_floats = comms[0]->max_floats; p.skip_rank = skip_rank; p.timeout_ns = comms[0]->timeout_ns;
    // the ranks' CTAs wait on one another: a cooperative launch refuses instead of deadlocking when they cannot all be resident
    void *args[] = {&p};
    const cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(allreduce_oneshot_kernel), dim3(ar_blocks(comms[0]->max_floats), world),
                                                      dim3(kArThreads), args, 0, stream);
    return e == cudaSuccess ? INSG_OK : cuda_fail(e, "cooperative launch");
}

} // extern "C"
