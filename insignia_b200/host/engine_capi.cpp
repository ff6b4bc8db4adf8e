// Handle-based C face of the C++ host classes (declarations: include/insignia_b200.h, "engine" section).
#include "insignia_b200.h"
#include "insignia_batch.hpp"
#include "insignia_decode.hpp"

#include <cstring>
#include <stdexcept>
#include <vector>
#include <memory>
#include <string>

namespace insg {
int fail(int code, const std::string &msg);
}

struct insg_engine {
    insignia::ModelFile model;
    std::unique_ptr<insignia::Qwen35Weights> weights;
    std::unique_ptr<insignia::DecodeWorkspace> ws;
    std::unique_ptr<insignia::Qwen35Decode> dec;
    int device = 0;
};

// Several sequences in lock step on the weights of an engine (include/insignia_batch.hpp).
struct insg_batch {
    insg_engine *engine;
    std::unique_ptr<insignia::Qwen35BatchDecode> dec;
};

// Handle over ModelFile + TieredStorage alone (include/insignia_storage.hpp), for callers without C++.
struct insg_storage {
    insignia::ModelFile model;
    std::unique_ptr<insignia::TieredStorage> store;
};

namespace {
template <class F> int storage_guarded(insg_storage *s, F &&f)
{
    if (!s) return insg::fail(INSG_E_ARG, "null storage");
    try {
        return f();
    } catch (const std::exception &ex) {
        return insg::fail(INSG_E_RUNTIME, ex.what());
    }
}

template <class F> int guarded(insg_engine *e, F &&f)
{
    if (!e) return insg::fail(INSG_E_ARG, "null engine");
    try {
        cudaSetDevice(e->device);
        return f();
    } catch (const std::exception &ex) {
        return insg::fail(INSG_E_RUNTIME, ex.what());
    }
}

float *field_ptr(insignia::DecodeWorkspace &x, const std::string &f)
{
    if (f == "hidden") return x.hidden;
    if (f == "norm") return x.norm;
    if (f == "qkv") return x.qkv;
    if (f == "attn_gate") return x.attn_gate;
    if (f == "key") return x.key;
    if (f == "value") return x.value;
    if (f == "z") return x.z;
    if (f == "a") return x.a;
    if (f == "b") return x.b;
    if (f == "core") return x.core;
    if (f == "gate") return x.gate;
    if (f == "up") return x.up;
    if (f == "down") return x.down;
    if (f == "logits") return x.logits;
    if (f == "delta_state") return x.delta_state;
    if (f == "conv_state") return x.conv_state;
    if (f == "kv_keys") return x.kv_keys;
    if (f == "kv_values") return x.kv_values;
    if (f == "mtp_keys") return x.mtp_keys;
    if (f == "mtp_values") return x.mtp_values;
    return nullptr;
}
} // namespace

namespace {
template <class F> int batch_guarded(insg_batch *b, F &&f)
{
    if (!b) return insg::fail(INSG_E_ARG, "null batch");
    try {
        cudaSetDevice(b->engine->device);
        return f();
    } catch (const std::exception &ex) {
        return insg::fail(INSG_E_RUNTIME, ex.what());
    }
}
} // namespace

extern "C" {

insg_storage *insg_storage_open(const char *index_path, uint64_t device_budget_bytes, int host_backend)
{
    if (!index_path) {
        insg::fail(INSG_E_ARG, "null index path");
        return nullptr;
    }
    try {
        auto s = std::make_unique<insg_storage>();
        s->model = insignia::ModelFile(index_path);
        s->store = std::make_unique<insignia::TieredStorage>(s->model, device_budget_bytes, nullptr,
                                                             host_backend ? insignia::make_host_backend() : nullptr);
        return s.release();
    } catch (const std::exception &ex) {
        insg::fail(INSG_E_RUNTIME, ex.what());
        return nullptr;
    }
}
void insg_storage_close(insg_storage *s) { delete s; }
int insg_storage_acquire(insg_storage *s, const char *name, void **data, uint64_t *bytes)
{
    return storage_guarded(s, [&] {
        if (!name) return insg::fail(INSG_E_ARG, "null name");
        const insignia::DeviceView v = s->store->acquire(name);
        if (data) *data = v.data;
        if (bytes) *bytes = v.bytes;
        return int(INSG_OK);
    });
}
int insg_storage_release(insg_storage *s, const char *name)
{
    return storage_guarded(s, [&] {
        if (!name) return insg::fail(INSG_E_ARG, "null name");
        s->store->release(name);
        return int(INSG_OK);
    });
}
int insg_storage_prefetch(insg_storage *s, const char *name)
{
    return storage_guarded(s, [&] {
        if (!name) return insg::fail(INSG_E_ARG, "null name");
        return s->store->prefetch(name) ? 1 : 0;
    });
}
int insg_storage_tier(insg_storage *s, const char *name)
{
    return storage_guarded(s, [&] {
        if (!name) return insg::fail(INSG_E_ARG, "null name");
        return int(s->store->tier(name));
    });
}
int insg_storage_reserve(insg_storage *s, uint64_t bytes)
{
    return storage_guarded(s, [&] {
        s->store->reserve(bytes);
        return int(INSG_OK);
    });
}
int insg_storage_unreserve(insg_storage *s, uint64_t bytes)
{
    return storage_guarded(s, [&] {
        s->store->unreserve(bytes);
        return int(INSG_OK);
    });
}
int insg_storage_set_host_cache(insg_storage *s, uint64_t bytes)
{
    return storage_guarded(s, [&] {
        s->store->set_host_cache_bytes(bytes);
        return int(INSG_OK);
    });
}
int insg_storage_clear(insg_storage *s)
{
    return storage_guarded(s, [&] {
        s->store->clear();
        return int(INSG_OK);
    });
}
uint64_t insg_storage_device_bytes(insg_storage *s) { return s ? s->store->device_bytes() : 0; }
uint64_t insg_storage_reserved_bytes(insg_storage *s) { return s ? s->store->reserved_bytes() : 0; }
int insg_storage_stats(insg_storage *s, uint64_t *out6)
{
    return storage_guarded(s, [&] {
        if (!out6) return insg::fail(INSG_E_ARG, "null output");
        const insignia::StorageStats st = s->store->stats();
        out6[0] = st.uploads; out6[1] = st.upload_bytes; out6[2] = st.evictions; out6[3] = st.hits; out6[4] = st.pinned_cache_hits;
        out6[5] = st.prefetches;
        return int(INSG_OK);
    });
}

insg_engine *insg_engine_create(const char *index_path, const insg_engine_options *opt)
{
    if (!index_path) {
        insg::fail(INSG_E_ARG, "null index path");
        return nullptr;
    }
    insg_engine_options o = {};
    if (opt) o = *opt;
    try {
        auto e = std::make_unique<insg_engine>();
        e->device = o.device;
        e->model = insignia::ModelFile(index_path); // host-only: file errors surface before any CUDA call
        if (cudaSetDevice(o.device) != cudaSuccess) throw std::runtime_error("cudaSetDevice failed");
        e->weights = std::make_unique<insignia::Qwen35Weights>(e->model, o.device_budget_bytes ? o.device_budget_bytes : (16ull << 30));
        insignia::DecodeOptions d;
        d.kv_bf16 = o.kv_dtype == INSG_KV_BF16;
        d.gate_elementwise = o.gate_elementwise != 0;
        d.accurate_trig = o.accurate_trig != 0;
        d.persistent = o.persistent != 0;
        d.prefill_tcgen05 = o.prefill_mma_sync == 0;
        d.use_graph = o.use_graph != 0;
        d.use_pdl = o.use_pdl != 0;
        d.gemv_tcgen05 = o.gemv_tcgen05 != 0;
        d.prepared_inputs = o.gemv_unprepared == 0;
        if (o.n_layers > 0) d.n_layers = o.n_layers;
        if (o.vocab > 0) d.vocab = o.vocab;
        if (d.n_layers > insignia::Qwen35Shape::layers || d.vocab > insignia::Qwen35Shape::vocab || (d.vocab & 15))
            throw std::runtime_error("n_layers <= 32 and vocab <= 248320, a multiple of 16");
        e->ws = std::make_unique<insignia::DecodeWorkspace>(o.max_context > 0 ? o.max_context : 4096, nullptr, d);
        e->dec = std::make_unique<insignia::Qwen35Decode>(*e->weights, *e->ws);
        return e.release();
    } catch (const std::exception &ex) {
        insg::fail(INSG_E_RUNTIME, ex.what());
        return nullptr;
    }
}

void insg_engine_destroy(insg_engine *e)
{
    if (!e) return;
    cudaSetDevice(e->device);
    e->dec.reset();
    e->ws.reset();
    e->weights.reset();
    delete e;
}

int insg_engine_embed(insg_engine *e, int token)
{
    return guarded(e, [&] {
        e->weights->embed(token, e->ws->hidden);
        return INSG_OK;
    });
}
int insg_engine_layer(insg_engine *e, int layer)
{
    return guarded(e, [&] {
        e->dec->layer(layer);
        return INSG_OK;
    });
}
int insg_engine_forward_token(insg_engine *e, int token)
{
    return guarded(e, [&] {
        e->dec->forward_token(token);
        return INSG_OK;
    });
}
int insg_engine_forward_tokens(insg_engine *e, const int *tokens, int count)
{
    return guarded(e, [&] {
        e->dec->forward_tokens(tokens, count);
        return int(INSG_OK);
    });
}
int insg_engine_logits_argmax(insg_engine *e)
{
    return guarded(e, [&] { return e->dec->logits_argmax(); });
}
int insg_engine_decode_token(insg_engine *e, int token)
{
    return guarded(e, [&] { return e->dec->decode_token(token); });
}
int insg_engine_mtp_draft(insg_engine *e, int token)
{
    return guarded(e, [&] { return e->dec->mtp_draft(token); });
}
int insg_engine_generate(insg_engine *e, int first_token, int count, int *out_tokens)
{
    return guarded(e, [&] {
        if (!out_tokens && count > 0) return insg::fail(INSG_E_ARG, "null output");
        const std::vector<int> t = e->dec->generate(first_token, count);
        if (!t.empty()) std::memcpy(out_tokens, t.data(), t.size() * sizeof(int));
        return int(INSG_OK);
    });
}
int insg_engine_prime_speculative(insg_engine *e, const int *prompt, int count)
{
    return guarded(e, [&] { return e->dec->prime_speculative(prompt, count); });
}
int insg_engine_generate_speculative(insg_engine *e, int first_token, int count, int *out_tokens, int *accepted, const int *forced_drafts)
{
    return guarded(e, [&] {
        if (!out_tokens && count > 0) return insg::fail(INSG_E_ARG, "null output");
        const std::vector<int> t = e->dec->generate_speculative(first_token, count, accepted, forced_drafts);
        if (!t.empty()) std::memcpy(out_tokens, t.data(), t.size() * sizeof(int));
        return int(INSG_OK);
    });
}
int insg_engine_profile_gemv_chain(insg_engine *e, int replays, float *ms_per_token, uint64_t *bytes, int *launches)
{
    return guarded(e, [&] {
        if (!ms_per_token || !bytes || !launches) return insg::fail(INSG_E_ARG, "null output");
        e->dec->profile_gemv_chain(replays, ms_per_token, bytes, launches);
        return int(INSG_OK);
    });
}
int insg_engine_set_program_option(insg_engine *e, const char *key, long long value)
{
    return guarded(e, [&] {
        if (!key) return insg::fail(INSG_E_ARG, "null key");
        e->dec->set_program_option(key, value);
        return int(INSG_OK);
    });
}
int insg_engine_selftest_barrier_timeout(insg_engine *e)
{
    return guarded(e, [&] { return e->dec->selftest_barrier_timeout() ? 1 : 0; });
}
int insg_engine_position(insg_engine *e) { return e ? e->ws->position : INSG_E_ARG; }
int insg_engine_set_position(insg_engine *e, int position)
{
    if (!e || position < 0) return insg::fail(INSG_E_ARG, "bad position");
    e->ws->position = position;
    return INSG_OK;
}
int insg_engine_reset(insg_engine *e)
{
    return guarded(e, [&] {
        cudaStreamSynchronize(e->dec->execution_stream());
        e->ws->reset();
        cudaStreamSynchronize(e->ws->stream);
        return INSG_OK;
    });
}
int insg_engine_read(insg_engine *e, const char *field, float *out, uint64_t count)
{
    return guarded(e, [&] {
        float *src = field ? field_ptr(*e->ws, field) : nullptr;
        if (!src || !out) return insg::fail(INSG_E_ARG, "unknown workspace field");
        cudaStream_t st = e->dec->execution_stream();
        if (cudaMemcpyAsync(out, src, count * sizeof(float), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
            cudaStreamSynchronize(st) != cudaSuccess)
            return insg::fail(INSG_E_CUDA, cudaGetErrorString(cudaGetLastError()));
        return int(INSG_OK);
    });
}
int insg_engine_write(insg_engine *e, const char *field, const float *in, uint64_t count)
{
    return guarded(e, [&] {
        float *dst = field ? field_ptr(*e->ws, field) : nullptr;
        if (!dst || !in) return insg::fail(INSG_E_ARG, "unknown workspace field");
        cudaStream_t st = e->dec->execution_stream();
        if (cudaMemcpyAsync(dst, in, count * sizeof(float), cudaMemcpyHostToDevice, st) != cudaSuccess ||
            cudaStreamSynchronize(st) != cudaSuccess)
            return insg::fail(INSG_E_CUDA, cudaGetErrorString(cudaGetLastError()));
        return int(INSG_OK);
    });
}
insg_batch *insg_batch_create(insg_engine *e, int sequences, int max_context)
{
    if (!e) {
        insg::fail(INSG_E_ARG, "null engine");
        return nullptr;
    }
    try {
        cudaSetDevice(e->device);
        auto b = std::make_unique<insg_batch>();
        b->engine = e;
        insignia::BatchOptions o;
        const insignia::DecodeOptions &d = e->ws->options;
        o.kv_bf16 = d.kv_bf16;
        o.gate_elementwise = d.gate_elementwise;
        o.accurate_trig = d.accurate_trig;
        o.use_graph = d.use_graph;
        o.n_layers = d.n_layers;
        o.vocab = d.vocab;
        b->dec = std::make_unique<insignia::Qwen35BatchDecode>(*e->weights, sequences, max_context > 0 ? max_context : e->ws->max_context, nullptr, o);
        return b.release();
    } catch (const std::exception &ex) {
        insg::fail(INSG_E_RUNTIME, ex.what());
        return nullptr;
    }
}
void insg_batch_destroy(insg_batch *b)
{
    if (!b) return;
    cudaSetDevice(b->engine->device);
    delete b;
}
int insg_batch_forward_tokens(insg_batch *b, const int *tokens)
{
    return batch_guarded(b, [&] {
        b->dec->forward_tokens(tokens);
        return int(INSG_OK);
    });
}
int insg_batch_decode_tokens(insg_batch *b, const int *tokens, int *next)
{
    return batch_guarded(b, [&] {
        b->dec->decode_tokens(tokens, next);
        return int(INSG_OK);
    });
}
int insg_batch_generate(insg_batch *b, const int *first_tokens, int count, int *out)
{
    return batch_guarded(b, [&] {
        b->dec->generate(first_tokens, count, out);
        return int(INSG_OK);
    });
}
int insg_batch_reset(insg_batch *b)
{
    return batch_guarded(b, [&] {
        cudaStreamSynchronize(b->dec->execution_stream());
        b->dec->reset();
        cudaStreamSynchronize(b->dec->execution_stream());
        return int(INSG_OK);
    });
}
int insg_batch_position(insg_batch *b) { return b ? b->dec->position() : INSG_E_ARG; }
int insg_batch_read(insg_batch *b, const char *field, int sequence, float *out, uint64_t count)
{
    return batch_guarded(b, [&] {
        const std::string f = field ? field : "";
        if (f == "hidden" && count == 4096) b->dec->read_hidden(sequence, out);
        else if (f == "delta_state") b->dec->read_delta_state(sequence, out, count);
        else return insg::fail(INSG_E_ARG, "unknown batch field");
        return int(INSG_OK);
    });
}
uint64_t insg_batch_launch_count(insg_batch *b) { return b ? b->dec->launch_count() : 0; }
insg_stream_t insg_batch_stream(insg_batch *b) { return b ? b->dec->execution_stream() : nullptr; }

void *insg_engine_buffer(insg_engine *e, const char *field)
{
    if (!e || !field) return nullptr;
    return field_ptr(*e->ws, field);
}
insg_stream_t insg_engine_stream(insg_engine *e) { return e ? e->dec->execution_stream() : nullptr; }
uint64_t insg_engine_launch_count(insg_engine *e) { return e ? e->dec->launch_count() : 0; }
uint64_t insg_engine_device_bytes(insg_engine *e)
{
    return e ? e->weights->storage().device_bytes() + e->weights->packed_bytes() : 0;
}

} // extern "C"
