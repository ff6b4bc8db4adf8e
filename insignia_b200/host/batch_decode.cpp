// insignia::Qwen35BatchDecode: several sequences decoded in lock step on one weight copy (interface and rationale:
// include/insignia_batch.hpp; the per-sequence arithmetic is that of src/decode.cu:14-23).
#include "insignia_batch.hpp"

#include "insignia_b200.h"

#include "decode_plan.hpp"

#include <algorithm>
#include <stdexcept>

namespace insignia {
namespace {
constexpr int kHidden = Qwen35Shape::hidden, kInter = Qwen35Shape::intermediate;
constexpr size_t kStateLayer = size_t(32) * 128 * 128, kConvLayer = size_t(8192) * 3;
const char *const kLM = "language_model";

void cuda_check(cudaError_t e, const char *what)
{
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
void insg_check(int rc)
{
    if (rc != INSG_OK) throw std::runtime_error(insg_last_error());
}
} // namespace

struct Qwen35BatchDecode::Impl {
    int B = 0;      // sequences the kernels run (1 and 2 on the mma.sync kernel, 3..8 on the tcgen05 kernel)
    int layout = 0; // weight layout: 0 mma.sync records (B <= 2), 1 tcgen05 tiles (B >= 3)
    std::vector<DecodeBlock> layers;
    const uint16_t *final_norm{};
    PackedMatrix lm_head;
    QuantMatrix embed;
    bool loaded = false;
    std::vector<std::string> pinned;
    cudaStream_t stream{};
    bool own_stream = false;
    cudaGraphExec_t exec{};
    uint64_t graph_nodes = 0;
    bool warm = false;
    // device buffers, [B][width] unless noted
    float *hidden{}, *qkv{}, *z{}, *a{}, *b{}, *core{}, *qg{}, *key{}, *value{}, *act{}, *logits{};
    float *delta_state{}, *conv_state{}; // [B][24][...]
    void *kv_keys{}, *kv_values{};       // [B][8][ctx][1024]
    void *attn_scratch{};                // [B][insg_gqa_scratch_bytes]
    void *umma_scratch{};
    size_t umma_scratch_bytes = 0, attn_scratch_each = 0, kv_seq_bytes = 0;
    int *d_tokens{}, *d_next{}, *d_position{}, *d_error{}, *d_log{}; // log [ctx + 1][B]
    int *host_tokens{};                  // pinned
    std::vector<void *> allocs;
    template <class T> void alloc(T **p, size_t bytes, const char *what)
    {
        cuda_check(cudaMalloc(reinterpret_cast<void **>(p), bytes), what);
        allocs.push_back(*p);
    }
};

Qwen35BatchDecode::Qwen35BatchDecode(Qwen35Weights &weights, int sequences, int max_context, cudaStream_t stream, const BatchOptions &options)
    : w_(weights), sequences_(sequences), max_context_(max_context), options_(options), impl_(std::make_unique<Impl>())
{
    if (sequences < 1 || sequences > 8) throw std::runtime_error("batch decode: 1..8 sequences");
    if (max_context <= 0) throw std::runtime_error("max_context must be positive");
    Impl &m = *impl_;
    m.B = sequences;
    m.layout = sequences >= 3 ? 1 : 0; // measured: four sequences cost the mma.sync kernel 4.6 ms a step, the tcgen05 kernel less
    if (stream) {
        m.stream = stream;
    } else {
        cuda_check(cudaStreamCreateWithFlags(&m.stream, cudaStreamDefault), "cudaStreamCreate");
        m.own_stream = true;
    }
    const size_t B = size_t(m.B), f = sizeof(float);
    m.alloc(&m.hidden, B * 4096 * f, "cudaMalloc batch");
    m.alloc(&m.qkv, B * 8192 * f, "cudaMalloc batch");
    m.alloc(&m.z, B * 4096 * f, "cudaMalloc batch");
    m.alloc(&m.a, B * 32 * f, "cudaMalloc batch");
    m.alloc(&m.b, B * 32 * f, "cudaMalloc batch");
    m.alloc(&m.core, B * 4096 * f, "cudaMalloc batch");
    m.alloc(&m.qg, B * 8192 * f, "cudaMalloc batch");
    m.alloc(&m.key, B * 1024 * f, "cudaMalloc batch");
    m.alloc(&m.value, B * 1024 * f, "cudaMalloc batch");
    m.alloc(&m.act, B * 12288 * f, "cudaMalloc batch");
    m.alloc(&m.logits, B * size_t(Qwen35Shape::vocab) * f, "cudaMalloc batch logits");
    m.alloc(&m.delta_state, B * 24 * kStateLayer * f, "cudaMalloc batch DeltaNet state");
    m.alloc(&m.conv_state, B * 24 * kConvLayer * f, "cudaMalloc batch convolution history");
    m.kv_seq_bytes = size_t(8) * max_context * 1024 * (options.kv_bf16 ? 2 : 4);
    m.alloc(&m.kv_keys, B * m.kv_seq_bytes, "cudaMalloc batch KV cache");
    m.alloc(&m.kv_values, B * m.kv_seq_bytes, "cudaMalloc batch KV cache");
    m.attn_scratch_each = (insg_gqa_scratch_bytes(max_context) + 255) / 256 * 256;
    m.alloc(&m.attn_scratch, B * m.attn_scratch_each, "cudaMalloc batch attention scratch");
    m.umma_scratch_bytes = insg_umma_gemm_scratch_bytes(kInter, m.B);
    m.alloc(&m.umma_scratch, m.umma_scratch_bytes, "cudaMalloc batch activation image");
    m.alloc(&m.d_tokens, (3 * B + 8) * sizeof(int), "cudaMalloc batch scalars");
    m.d_next = m.d_tokens + B;
    m.d_position = m.d_next + B;
    m.d_error = m.d_position + 1;
    m.alloc(&m.d_log, (size_t(max_context) + 1) * B * sizeof(int), "cudaMalloc batch token log");
    cuda_check(cudaMallocHost(&m.host_tokens, (B + 2) * sizeof(int)), "cudaMallocHost");
    cuda_check(cudaMemsetAsync(m.d_tokens, 0, (3 * B + 8) * sizeof(int), m.stream), "memset");
    cuda_check(cudaMemsetAsync(m.attn_scratch, 0, B * m.attn_scratch_each, m.stream), "memset");
    cuda_check(cudaMemsetAsync(m.hidden, 0, B * 4096 * f, m.stream), "memset");
    reset();
}

Qwen35BatchDecode::~Qwen35BatchDecode()
{
    Impl &m = *impl_;
    cudaStreamSynchronize(m.stream);
    if (m.exec) cudaGraphExecDestroy(m.exec);
    for (void *p : m.allocs) cudaFree(p);
    if (m.host_tokens) cudaFreeHost(m.host_tokens);
    for (const std::string &n : m.pinned) w_.storage().release(n);
    if (m.loaded) w_.release(std::string(kLM) + ".model.embed_tokens");
    if (m.own_stream) cudaStreamDestroy(m.stream);
}

cudaStream_t Qwen35BatchDecode::execution_stream() { return impl_->stream; }

void Qwen35BatchDecode::reset()
{
    Impl &m = *impl_;
    cuda_check(cudaMemsetAsync(m.delta_state, 0, size_t(m.B) * 24 * kStateLayer * sizeof(float), m.stream), "memset DeltaNet state");
    cuda_check(cudaMemsetAsync(m.conv_state, 0, size_t(m.B) * 24 * kConvLayer * sizeof(float), m.stream), "memset convolution history");
    cuda_check(cudaMemsetAsync(m.d_position, 0, sizeof(int), m.stream), "memset position");
    position_ = 0;
}

namespace {
insg_gemv_segment seg(const PackedMatrix &pm, float *out, int epilogue)
{
    insg_gemv_segment s = {};
    s.packed = pm.data;
    s.out = out;
    s.rows = pm.rows;
    s.epilogue = epilogue;
    return s;
}
} // namespace

// embed, all layers, head, commit: what one graph replay does
void Qwen35BatchDecode::enqueue_step()
{
    Impl &m = *impl_;
    const int n = options_.n_layers, B = m.B;
    if (!m.loaded) {
        m.layers.resize(size_t(n));
        Loader L{w_, m.pinned, m.layout};
        for (int l = 0; l < n; l++) {
            const std::string name = std::string(kLM) + ".model.layers." + std::to_string(l);
            if (Qwen35Shape::full_attention(l)) load_attention(L, name, m.layers[size_t(l)]);
            else load_delta(L, name, m.layers[size_t(l)]);
        }
        m.final_norm = L.bf16(std::string(kLM) + ".model.norm.weight", kHidden);
        m.lm_head = w_.packed(std::string(kLM) + ".lm_head", m.layout);
        m.embed = w_.matrix(std::string(kLM) + ".model.embed_tokens");
        m.loaded = true;
    }
    cudaStream_t st = m.stream;
    auto gemv = [&](insg_gemv_op &op) {
        op.tokens = B;
        op.layout = m.layout;
        op.error_flag = m.d_error;
        op.pdl = 1; // every kernel of the step waits for its predecessor before it reads activations
        if (m.layout == 1 && B > 1) {
            op.umma_scratch = m.umma_scratch;
            op.umma_scratch_bytes = m.umma_scratch_bytes;
        }
        insg_check(insg_gemv_fused(&op, st));
        launches_ += (m.layout == 1 && B > 1) ? 2 : 1;
    };
    auto mlp = [&](const DecodeBlock &blk) {
        insg_gemv_op up = {};
        up.in = m.hidden;
        up.norm_w = blk.post_norm;
        up.cols = kHidden;
        up.prologue = INSG_PRO_RMSNORM;
        up.n_segments = 1;
        up.seg[0] = seg(blk.gate, m.act, INSG_EPI_SWIGLU);
        up.seg[0].packed2 = blk.up.data;
        gemv(up);
        insg_gemv_op dn = {};
        dn.in = m.act;
        dn.cols = kInter;
        dn.prologue = INSG_PRO_PLAIN;
        dn.n_segments = 1;
        dn.seg[0] = seg(blk.down, m.hidden, INSG_EPI_RESIDUAL);
        gemv(dn);
    };
    const uint32_t *ew = static_cast<const uint32_t *>(m.embed.weight.data);
    const uint8_t *es = static_cast<const uint8_t *>(m.embed.scales.data);
    for (int s = 0; s < B; s++) {
        insg_check(insg_mxfp4_embed(ew, es, m.hidden + size_t(s) * kHidden, m.d_tokens + s, m.embed.rows, kHidden, 1, st));
        launches_++;
    }
    for (int l = 0; l < n; l++) {
        const DecodeBlock &blk = m.layers[size_t(l)];
        if (!Qwen35Shape::full_attention(l)) {
            const int di = l - l / 4;
            insg_gemv_op in = {};
            in.in = m.hidden;
            in.norm_w = blk.in_norm;
            in.cols = kHidden;
            in.prologue = INSG_PRO_RMSNORM;
            in.n_segments = 4;
            in.seg[0] = seg(blk.qkv, m.qkv, INSG_EPI_CONV_SILU);
            in.seg[0].conv_state = m.conv_state + size_t(di) * kConvLayer;
            in.seg[0].conv_w = blk.conv_w;
            in.seg[0].conv_token_stride = (long long)(24 * kConvLayer); // sequence s's history of this layer
            in.seg[1] = seg(blk.z, m.z, INSG_EPI_STORE);
            in.seg[2] = seg(blk.a, m.a, INSG_EPI_DECAY);
            in.seg[2].A_log = blk.A_log;
            in.seg[2].dt_bias = blk.dt_bias;
            in.seg[3] = seg(blk.b, m.b, INSG_EPI_BETA);
            gemv(in);
            insg_check(insg_deltanet_decode_batch(m.delta_state + size_t(di) * kStateLayer, (long long)(24 * kStateLayer), m.qkv, m.qkv + 2048,
                                                  m.qkv + 4096, m.a, m.b, m.core, B, 8192, 1, st));
            launches_++;
            insg_gemv_op out = {};
            out.in = m.core;
            out.aux = m.z;
            out.norm_w = blk.dn_norm;
            out.cols = 4096;
            out.prologue = INSG_PRO_GATED_RMSNORM;
            out.n_segments = 1;
            out.seg[0] = seg(blk.out, m.hidden, INSG_EPI_RESIDUAL);
            gemv(out);
        } else {
            insg_gemv_op in = {};
            in.in = m.hidden;
            in.norm_w = blk.in_norm;
            in.cols = kHidden;
            in.prologue = INSG_PRO_RMSNORM;
            in.n_segments = 3;
            in.seg[0] = seg(blk.q, m.qg, INSG_EPI_STORE);
            in.seg[1] = seg(blk.k, m.key, INSG_EPI_STORE);
            in.seg[2] = seg(blk.v, m.value, INSG_EPI_STORE);
            gemv(in);
            const size_t layer_off = size_t(l / 4) * max_context_ * 1024 * (options_.kv_bf16 ? 2 : 4);
            {   // every sequence attends over its own cache, all of them in one launch
                insg_attn_op at = {};
                at.qraw = m.qg;
                at.k_raw = m.key;
                at.v = m.value;
                at.q_norm_w = blk.q_norm;
                at.k_norm_w = blk.k_norm;
                at.k_cache = static_cast<uint8_t *>(m.kv_keys) + layer_off;
                at.v_cache = static_cast<uint8_t *>(m.kv_values) + layer_off;
                at.out = m.core;
                at.position = m.d_position;
                at.max_context = max_context_;
                at.kv_dtype = options_.kv_bf16 ? INSG_KV_BF16 : INSG_KV_F32;
                at.fast_trig = options_.accurate_trig ? 0 : 1;
                at.error_flag = m.d_error;
                at.scratch = m.attn_scratch;
                at.scratch_bytes = size_t(B) * m.attn_scratch_each;
                // safe with dependent-launch overlap: the cache rows the launch fetches before its dependency wait were
                // written a whole step ago
                at.pdl = 1;
                insg_check(insg_attention_batch(&at, B, m.kv_seq_bytes, st));
                launches_++;
            }
            insg_gemv_op o = {};
            o.in = m.core;
            o.aux = m.qg;
            o.cols = 4096;
            o.prologue = options_.gate_elementwise ? INSG_PRO_SIGMOID_GATE_QPROJ : INSG_PRO_SIGMOID_GATE_HEAD0;
            o.n_segments = 1;
            o.seg[0] = seg(blk.o, m.hidden, INSG_EPI_RESIDUAL);
            gemv(o);
        }
        mlp(blk);
    }
    insg_gemv_op head = {};
    head.in = m.hidden;
    head.norm_w = m.final_norm;
    head.cols = kHidden;
    head.prologue = INSG_PRO_RMSNORM;
    head.n_segments = 1;
    head.seg[0] = seg(m.lm_head, m.logits, INSG_EPI_STORE);
    head.seg[0].rows = options_.vocab;
    gemv(head);
    insg_check(insg_argmax_rows(m.logits, options_.vocab, options_.vocab, B, m.d_next, st));
    insg_check(insg_commit_tokens(m.d_next, m.d_tokens, m.d_log, max_context_ + 1, m.d_position, B, st));
    launches_ += 2;
}

void Qwen35BatchDecode::run_step()
{
    Impl &m = *impl_;
    if (position_ >= max_context_) throw std::runtime_error("KV cache full");
    if (!options_.use_graph) {
        enqueue_step();
    } else if (!m.exec) {
        if (!m.warm) { // the first step loads and repacks the weights (allocates, synchronises): it runs eagerly
            enqueue_step();
            m.warm = true;
        } else {
            const uint64_t before = launches_;
            cudaGraph_t g = nullptr;
            cuda_check(cudaStreamBeginCapture(m.stream, cudaStreamCaptureModeThreadLocal), "begin graph capture");
            try {
                enqueue_step();
            } catch (...) {
                cudaStreamEndCapture(m.stream, &g);
                if (g) cudaGraphDestroy(g);
                throw;
            }
            cuda_check(cudaStreamEndCapture(m.stream, &g), "end graph capture");
            m.graph_nodes = launches_ - before;
            const cudaError_t e = cudaGraphInstantiate(&m.exec, g, 0);
            cudaGraphDestroy(g);
            cuda_check(e, "instantiate graph");
            cuda_check(cudaGraphLaunch(m.exec, m.stream), "launch graph");
        }
    } else {
        cuda_check(cudaGraphLaunch(m.exec, m.stream), "launch graph");
        launches_ += m.graph_nodes;
    }
    position_++;
}

void Qwen35BatchDecode::forward_tokens(const int *tokens)
{
    Impl &m = *impl_;
    if (!tokens) throw std::runtime_error("batch decode: null token list");
    for (int s = 0; s < m.B; s++) {
        const int t = s < sequences_ ? tokens[s] : 0;
        if (t < 0 || t >= Qwen35Shape::vocab) throw std::runtime_error("token out of range");
        m.host_tokens[s] = t;
    }
    cuda_check(cudaMemcpyAsync(m.d_tokens, m.host_tokens, size_t(m.B) * sizeof(int), cudaMemcpyHostToDevice, m.stream), "copy tokens");
    run_step();
    // the pinned staging buffer is reused by the next call
    cuda_check(cudaStreamSynchronize(m.stream), "synchronize");
}

void Qwen35BatchDecode::decode_tokens(const int *tokens, int *next)
{
    Impl &m = *impl_;
    if (!next) throw std::runtime_error("batch decode: null output");
    forward_tokens(tokens);
    cuda_check(cudaMemcpyAsync(m.host_tokens, m.d_next, size_t(m.B + 2) * sizeof(int), cudaMemcpyDeviceToHost, m.stream), "read tokens");
    cuda_check(cudaStreamSynchronize(m.stream), "synchronize");
    if (m.host_tokens[m.B + 1]) throw std::runtime_error("a bounded wait inside a GPU kernel expired");
    for (int s = 0; s < sequences_; s++) next[s] = m.host_tokens[s];
}

void Qwen35BatchDecode::generate(const int *first_tokens, int count, int *out)
{
    Impl &m = *impl_;
    if (count <= 0) return;
    if (!first_tokens || !out) throw std::runtime_error("batch decode: null argument");
    if (position_ + count > max_context_) throw std::runtime_error("KV cache full");
    for (int s = 0; s < m.B; s++) {
        const int t = s < sequences_ ? first_tokens[s] : 0;
        if (t < 0 || t >= Qwen35Shape::vocab) throw std::runtime_error("token out of range");
        m.host_tokens[s] = t;
    }
    const int start = position_;
    cuda_check(cudaMemcpyAsync(m.d_tokens, m.host_tokens, size_t(m.B) * sizeof(int), cudaMemcpyHostToDevice, m.stream), "copy tokens");
    for (int i = 0; i < count; i++) run_step(); // each step's commit feeds the next
    std::vector<int> log(size_t(count) * m.B);
    cuda_check(cudaMemcpyAsync(log.data(), m.d_log + size_t(start) * m.B, log.size() * sizeof(int), cudaMemcpyDeviceToHost, m.stream), "read tokens");
    cuda_check(cudaStreamSynchronize(m.stream), "synchronize");
    for (int i = 0; i < count; i++)
        for (int s = 0; s < sequences_; s++) out[size_t(i) * sequences_ + s] = log[size_t(i) * m.B + s];
}

void Qwen35BatchDecode::read_hidden(int sequence, float *out)
{
    Impl &m = *impl_;
    if (sequence < 0 || sequence >= sequences_ || !out) throw std::runtime_error("batch decode: bad sequence");
    cuda_check(cudaMemcpyAsync(out, m.hidden + size_t(sequence) * kHidden, kHidden * sizeof(float), cudaMemcpyDeviceToHost, m.stream), "read hidden");
    cuda_check(cudaStreamSynchronize(m.stream), "synchronize");
}

void Qwen35BatchDecode::read_delta_state(int sequence, float *out, uint64_t count)
{
    Impl &m = *impl_;
    if (sequence < 0 || sequence >= sequences_ || !out || count > 24 * kStateLayer) throw std::runtime_error("batch decode: bad sequence");
    cuda_check(cudaMemcpyAsync(out, m.delta_state + size_t(sequence) * 24 * kStateLayer, count * sizeof(float), cudaMemcpyDeviceToHost, m.stream),
               "read state");
    cuda_check(cudaStreamSynchronize(m.stream), "synchronize");
}

} // namespace insignia
