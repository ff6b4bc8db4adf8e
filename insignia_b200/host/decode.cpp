// insignia::DecodeWorkspace / insignia::Qwen35Decode on the fused sm_100a kernels
// (interface: include/insignia_decode.hpp; reference behaviour: src/decode.cu:9-69).
//
// Kernel sequence per token (reference: 18 launches per layer, ~580 per token):
//   embed                                                       1
//   DeltaNet layer : in_proj(qkv|z|a|b) + conv/SiLU/gates, delta step, out_proj+residual,
//                    gate/up + SwiGLU, down + residual           5
//   attention layer: q|k|v proj, norm/RoPE/KV store/split-K attention, o_proj(gated)+residual,
//                    gate/up + SwiGLU, down + residual           5
//   final norm + lm_head + arg-max                               1
// = 162 fused operations per token.  Default: 162 launches replayed from one CUDA graph with programmatic dependent
// launch.  Option `persistent`: the same operations recorded once as a program and executed by ONE persistent
// cooperative launch per token (or per run of tokens), with grid barriers between them (csrc/persistent.cu).
#include "insignia_decode.hpp"

#include "insignia_b200.h"

#include "decode_plan.hpp"

#include <stdexcept>

namespace insignia {
namespace {

constexpr int kHidden = Qwen35Shape::hidden, kInter = Qwen35Shape::intermediate;
// DecodeWorkspace::prep: fp16 image of the normalised-to-be hidden vector, fp16 image of the SwiGLU output, sums of squares
constexpr size_t kPrepHidden = 0, kPrepAct = size_t(2) * kHidden * 2, kPrepSums = kPrepAct + size_t(2) * kInter * 2;
constexpr int kMultiSteps = 8; // token steps per graph in Qwen35Decode::generate
// DecodeWorkspace::multi: activations of up to kChunk consecutive tokens for Qwen35Decode::forward_tokens, [token][width] each
constexpr int kChunk = 4;     // tokens per pass of the mma.sync kernel
constexpr int kBigChunk = 256; // tokens per pass of the tcgen05 kernel (sixteen groups of sixteen)
constexpr size_t kMultiHidden = 0, kMultiQkv = kMultiHidden + size_t(kBigChunk) * 4096, kMultiZ = kMultiQkv + size_t(kBigChunk) * 8192,
                 kMultiA = kMultiZ + size_t(kBigChunk) * 4096, kMultiB = kMultiA + size_t(kBigChunk) * 32,
                 kMultiCore = kMultiB + size_t(kBigChunk) * 32, kMultiQg = kMultiCore + size_t(kBigChunk) * 4096,
                 kMultiKey = kMultiQg + size_t(kBigChunk) * 8192, kMultiValue = kMultiKey + size_t(kBigChunk) * 1024,
                 kMultiAct = kMultiValue + size_t(kBigChunk) * 1024, kMultiQn = kMultiAct + size_t(kBigChunk) * 12288,
                 kMultiTokens = kMultiQn + size_t(kBigChunk) * 4096, kMultiFloats = kMultiTokens + kBigChunk;
constexpr size_t kPrepBytes = kPrepSums + 2 * 296 * sizeof(float); // one row of sums per image
const char *const kLM = "language_model";

void cuda_check(cudaError_t e, const char *what)
{
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
void insg_check(int rc)
{
    if (rc != INSG_OK) throw std::runtime_error(insg_last_error());
}
template <class T> void dev_alloc(T **p, size_t count)
{
    cuda_check(cudaMalloc(reinterpret_cast<void **>(p), count * sizeof(T)), "cudaMalloc workspace");
}

} // namespace

// --------------------------------------------------------------- workspace
DecodeWorkspace::DecodeWorkspace(int ctx, cudaStream_t s) : max_context(ctx), stream(s) { allocate(); }

DecodeWorkspace::DecodeWorkspace(int ctx, cudaStream_t s, const DecodeOptions &o) : max_context(ctx), stream(s), options(o)
{
    allocate();
}

void DecodeWorkspace::allocate()
{
    if (max_context <= 0) throw std::runtime_error("max_context must be positive");
    const size_t kv_scale = options.kv_bf16 ? 2 : 1; // element counts below are in floats
    dev_alloc(&hidden, 4096);
    dev_alloc(&norm, 4096);
    dev_alloc(&qkv, 8192);
    dev_alloc(&attn_gate, 4096);
    dev_alloc(&key, 1024);
    dev_alloc(&value, 1024);
    dev_alloc(&z, 4096);
    dev_alloc(&a, 32);
    dev_alloc(&b, 32);
    dev_alloc(&core, 4096);
    dev_alloc(&gate, 12288);
    dev_alloc(&up, 12288);
    dev_alloc(&down, 4096);
    dev_alloc(&logits, size_t(Qwen35Shape::vocab));
    dev_alloc(&delta_state, size_t(24) * 32 * 128 * 128);
    dev_alloc(&conv_state, size_t(24) * 8192 * 3);
    const size_t kv_floats = (size_t(8) * max_context * 1024 + kv_scale - 1) / kv_scale;
    const size_t mtp_floats = (size_t(max_context) * 1024 + kv_scale - 1) / kv_scale;
    dev_alloc(&kv_keys, kv_floats);
    dev_alloc(&kv_values, kv_floats);
    dev_alloc(&mtp_keys, mtp_floats);
    dev_alloc(&mtp_values, mtp_floats);
    dev_alloc(&d_token, 4 + size_t(max_context) + 1); // token, position, next, pad, then the token log
    d_position = d_token + 1;
    d_next = d_token + 2;
    // one region per token of a prompt chunk; the single-token step uses the first
    cuda_check(cudaMalloc(&attn_scratch, size_t(kBigChunk) * insg_gqa_scratch_bytes(max_context)), "cudaMalloc attention scratch");
    cuda_check(cudaMalloc(&argmax_scratch, insg_gemv_argmax_scratch_bytes()), "cudaMalloc arg-max scratch");
    cuda_check(cudaMalloc(&prep, kPrepBytes), "cudaMalloc prepared inputs");
    cuda_check(cudaMalloc(&multi, kMultiFloats * sizeof(float)), "cudaMalloc multi-token buffers");
    umma_scratch_bytes = insg_umma_gemm_scratch_bytes(kInter, kBigChunk);
    cuda_check(cudaMalloc(&umma_scratch, umma_scratch_bytes), "cudaMalloc tcgen05 activation image");
    cuda_check(cudaMemsetAsync(prep, 0, kPrepBytes, stream), "memset");
    cuda_check(cudaMemsetAsync(attn_scratch, 0, size_t(kBigChunk) * insg_gqa_scratch_bytes(max_context), stream), "memset");
    cuda_check(cudaMemsetAsync(argmax_scratch, 0, 64, stream), "memset");
    cuda_check(cudaMemsetAsync(d_token, 0, (4 + size_t(max_context) + 1) * sizeof(int), stream), "memset");
    // The reference leaves the KV caches uninitialised (src/decode.cu:10); rows are always written before they are read.
    reset();
}

void DecodeWorkspace::reset()
{
    cuda_check(cudaMemsetAsync(delta_state, 0, size_t(24) * 32 * 128 * 128 * 4, stream), "memset delta state");
    cuda_check(cudaMemsetAsync(conv_state, 0, size_t(24) * 8192 * 3 * 4, stream), "memset conv state");
    position = 0;
}

DecodeWorkspace::~DecodeWorkspace()
{
    for (void *p : {(void *)hidden, (void *)norm, (void *)qkv, (void *)attn_gate, (void *)key, (void *)value, (void *)z, (void *)a,
                    (void *)b, (void *)core, (void *)gate, (void *)up, (void *)down, (void *)logits, (void *)delta_state,
                    (void *)conv_state, (void *)kv_keys, (void *)kv_values, (void *)mtp_keys, (void *)mtp_values, (void *)d_token,
                    attn_scratch, argmax_scratch, prep, (void *)multi, umma_scratch})
        cudaFree(p);
}

// --------------------------------------------------------------------- plan
struct Qwen35Decode::Plan {
    using Block = DecodeBlock;
    std::vector<Block> layers;
    std::vector<Block> layers_umma; // the same blocks with their matrices in the tcgen05 tile layout (prompt processing)
    Block mtp;
    bool head_ready = false, embed_ready = false, mtp_ready = false;
    const uint16_t *final_norm{};
    PackedMatrix lm_head;
    QuantMatrix embed;
    const uint16_t *mtp_fc{}, *mtp_norm_e{}, *mtp_norm_h{}, *mtp_norm{};
    std::vector<std::string> pinned;      // tensors held for the lifetime of the plan
    std::vector<std::string> pinned_mats; // matrices held (embed_tokens)
    cudaStream_t stream{};
    bool own_stream = false;
    cudaGraph_t graph{};
    cudaGraphExec_t exec{};
    uint64_t graph_nodes = 0, chunk_nodes = 0;
    bool capturing = false, chunk_warm = false;
    cudaGraphExec_t exec_multi{}; // kMultiSteps token steps in one graph, for device-fed generation
    cudaGraphExec_t exec_chunk{}; // one pass of forward_tokens over kChunk prompt tokens
    int *host_result{}; // pinned: {next token, wait-expired flag}, so the per-token read-back is a true asynchronous copy
    float *spec_state{}, *spec_conv{}, *spec_logits{}; // speculative decode: second DeltaNet state, convolution snapshot, [2][vocab] logits
    int *spec_pair{};                                  // device: the two arg-max results of a verify pass
    int *spec_host{};                                  // pinned: {token, draft} on the way in
    cudaGraphExec_t exec_verify[2]{};                  // the verify pass, by which DeltaNet state buffer is the live one
    cudaGraphExec_t exec_mtp[2]{};                     // the MTP block without / with its head
    int verify_runs[2]{}, mtp_runs[2]{};               // first run of each form is eager (kernel variants set their attributes)
    insg_program *prog{};     // the token step as one persistent launch
    std::vector<std::pair<std::string, long long>> program_options; // applied to every program this engine builds
};

Qwen35Decode::Qwen35Decode(Qwen35Weights &weights, DecodeWorkspace &workspace) : w_(weights), x_(workspace) {}

Qwen35Decode::~Qwen35Decode()
{
    if (!plan_) return;
    Plan &p = *plan_;
    cudaStreamSynchronize(p.stream);
    if (p.exec) cudaGraphExecDestroy(p.exec);
    if (p.exec_multi) cudaGraphExecDestroy(p.exec_multi);
    if (p.exec_chunk) cudaGraphExecDestroy(p.exec_chunk);
    if (p.graph) cudaGraphDestroy(p.graph);
    if (p.prog) insg_program_destroy(p.prog);
    for (void *q : {(void *)p.spec_state, (void *)p.spec_conv, (void *)p.spec_logits, (void *)p.spec_pair}) cudaFree(q);
    if (p.spec_host) cudaFreeHost(p.spec_host);
    for (cudaGraphExec_t e : {p.exec_verify[0], p.exec_verify[1], p.exec_mtp[0], p.exec_mtp[1]})
        if (e) cudaGraphExecDestroy(e);
    for (const std::string &n : p.pinned) w_.storage().release(n);
    for (const std::string &n : p.pinned_mats) w_.release(n);
    if (p.host_result) cudaFreeHost(p.host_result);
    if (p.own_stream) cudaStreamDestroy(p.stream);
}

Qwen35Decode::Plan &Qwen35Decode::plan()
{
    if (!plan_) {
        plan_ = std::make_unique<Plan>();
        plan_->layers.resize(Qwen35Shape::layers);
        plan_->layers_umma.resize(Qwen35Shape::layers);
        if (x_.stream) {
            plan_->stream = x_.stream;
        } else {
            // The legacy default stream cannot be captured into a graph.  A blocking stream keeps the
            // ordering a default-stream caller expects (it synchronises with the legacy stream both ways).
            cuda_check(cudaStreamCreateWithFlags(&plan_->stream, cudaStreamDefault), "cudaStreamCreate");
            plan_->own_stream = true;
        }
        cuda_check(cudaMallocHost(&plan_->host_result, 2 * sizeof(int)), "cudaMallocHost");
    }
    return *plan_;
}

// --------------------------------------------------------------- enqueue helpers
namespace {
struct Ctx {
    DecodeWorkspace &x;
    cudaStream_t st;
    bool pdl;
    uint64_t &launches;
    bool gemv_only;                      // only the fused GEMVs are issued (timing of the weight-streaming chain alone)
    insg_program *rec;                   // non-null: operations are appended to this program instead of being launched
    uint64_t *gemv_bytes;                // optional: algorithmic weight bytes of the GEMVs issued are added here
    bool hidden_prepared = false;        // the previous block left this block's first input prepared
    const uint16_t *next_norm = nullptr; // weight of the RMSNorm that reads this block's output next, when known
    int layout = -1;                     // >= 0: weight layout of the GEMVs issued (else the engine's gemv_tcgen05 option)
    void *prep_hidden() const { return static_cast<uint8_t *>(x.prep) + kPrepHidden; }
    void *prep_act() const { return static_cast<uint8_t *>(x.prep) + kPrepAct; }
    float *prep_sums() const { return reinterpret_cast<float *>(static_cast<uint8_t *>(x.prep) + kPrepSums); }
    bool prepared() const { return x.options.prepared_inputs && !x.options.gemv_tcgen05; }
};

// The block's first GEMV: RMSNorm of the residual stream, from the fp32 vector or from the image the previous block left.
void rmsnorm_input(const Ctx &c, insg_gemv_op &op, const uint16_t *norm_w)
{
    op.cols = kHidden;
    if (c.prepared() && c.hidden_prepared) {
        op.in = static_cast<const float *>(c.prep_hidden());
        op.prologue = INSG_PRO_PREPARED;
        op.prep_partials = c.prep_sums();
        op.prep_rms = 1;
        op.aux = c.x.hidden; // read instead of the image when the producer's sums put the image out of its range
        op.norm_w = norm_w;
    } else {
        op.in = c.x.hidden;
        op.norm_w = norm_w;
        op.x_out = c.x.norm;
        op.prologue = INSG_PRO_RMSNORM;
    }
}

// A GEMV that adds into the residual stream leaves the input of the RMSNorm + GEMV that follows prepared.
void residual_output(const Ctx &c, insg_gemv_segment &s, const uint16_t *following_norm_w)
{
    if (!c.prepared() || !following_norm_w) return;
    s.prep = c.prep_hidden();
    s.prep_w = following_norm_w;
    s.prep_partials = c.prep_sums();
}

uint64_t gemv_weight_bytes(const insg_gemv_op &op)
{
    uint64_t b = 0;
    for (int i = 0; i < op.n_segments; i++)
        b += uint64_t(op.seg[i].rows) * op.cols * 17 / 32 * (op.seg[i].epilogue == INSG_EPI_SWIGLU ? 2 : 1);
    return b;
}

void run_gemv(Ctx &c, insg_gemv_op &op)
{
    op.pdl = c.pdl ? 1 : 0;
    op.layout = c.layout >= 0 ? c.layout : (c.x.options.gemv_tcgen05 ? 1 : 0);
    op.error_flag = c.x.d_token + 3;
    if (op.layout == 1 && op.tokens > 1) {
        op.umma_scratch = c.x.umma_scratch;
        op.umma_scratch_bytes = c.x.umma_scratch_bytes;
    }
    if (c.gemv_bytes) *c.gemv_bytes += gemv_weight_bytes(op);
    if (c.rec) insg_check(insg_program_add_gemv(c.rec, &op));
    else insg_check(insg_gemv_fused(&op, c.st));
    c.launches++;
}

insg_gemv_segment seg(const PackedMatrix &m, float *out, int epilogue)
{
    insg_gemv_segment s = {};
    s.packed = m.data;
    s.out = out;
    s.rows = m.rows;
    s.epilogue = epilogue;
    return s;
}
} // namespace

// The three kernels shared by both block types: post-norm + gate/up + SwiGLU, down + residual.
static void enqueue_mlp_block(Ctx &c, const Qwen35Decode::Plan::Block &b)
{
    // the block's out/o_proj launch has just left the post-norm input prepared (when that mode is on)
    Ctx mid = c;
    mid.hidden_prepared = true;
    insg_gemv_op op = {};
    rmsnorm_input(mid, op, b.post_norm);
    op.n_segments = 1;
    op.seg[0] = seg(b.gate, c.x.gate, INSG_EPI_SWIGLU);
    op.seg[0].packed2 = b.up.data;
    if (c.prepared()) {
        op.seg[0].prep = c.prep_act();
        op.seg[0].prep_partials = c.prep_sums() + 296; // second row: sums of squares of the SwiGLU output
    }
    run_gemv(c, op);

    insg_gemv_op dn = {};
    dn.in = c.prepared() ? static_cast<const float *>(c.prep_act()) : c.x.gate;
    dn.cols = kInter;
    dn.prologue = c.prepared() ? INSG_PRO_PREPARED : INSG_PRO_PLAIN;
    if (c.prepared()) {
        dn.prep_partials = c.prep_sums() + 296;
        dn.aux = c.x.gate;
    }
    dn.n_segments = 1;
    dn.seg[0] = seg(b.down, c.x.hidden, INSG_EPI_RESIDUAL);
    residual_output(c, dn.seg[0], c.next_norm);
    run_gemv(c, dn);
}

static void enqueue_delta_block(Ctx &c, const Qwen35Decode::Plan::Block &b, int di)
{
    DecodeWorkspace &x = c.x;
    insg_gemv_op in = {};
    rmsnorm_input(c, in, b.in_norm);
    in.n_segments = 4;
    in.seg[0] = seg(b.qkv, x.qkv, INSG_EPI_CONV_SILU);
    in.seg[0].conv_state = x.conv_state + size_t(di) * 8192 * 3;
    in.seg[0].conv_w = b.conv_w;
    in.seg[1] = seg(b.z, x.z, INSG_EPI_STORE);
    in.seg[2] = seg(b.a, x.a, INSG_EPI_DECAY);
    in.seg[2].A_log = b.A_log;
    in.seg[2].dt_bias = b.dt_bias;
    in.seg[3] = seg(b.b, x.b, INSG_EPI_BETA);
    run_gemv(c, in);

    if (!c.gemv_only) {
        float *state = x.delta_state + size_t(di) * 32 * 128 * 128;
        if (c.rec) insg_check(insg_program_add_deltanet(c.rec, state, x.qkv, x.qkv + 2048, x.qkv + 4096, x.a, x.b, x.core));
        else insg_check(insg_deltanet_decode(state, x.qkv, x.qkv + 2048, x.qkv + 4096, x.a, x.b, x.core, c.pdl ? 1 : 0, c.st));
        c.launches++;
    }

    insg_gemv_op out = {};
    out.in = x.core;
    out.aux = x.z;
    out.norm_w = b.dn_norm;
    out.cols = 4096;
    out.prologue = INSG_PRO_GATED_RMSNORM;
    out.n_segments = 1;
    out.seg[0] = seg(b.out, x.hidden, INSG_EPI_RESIDUAL);
    residual_output(c, out.seg[0], b.post_norm);
    run_gemv(c, out);

    enqueue_mlp_block(c, b);
}

static void enqueue_attention_block(Ctx &c, const Qwen35Decode::Plan::Block &b, void *kc, void *vc, int position_offset)
{
    DecodeWorkspace &x = c.x;
    insg_gemv_op in = {};
    rmsnorm_input(c, in, b.in_norm);
    in.n_segments = 3;
    in.seg[0] = seg(b.q, x.gate, INSG_EPI_STORE); // interleaved [16][q256|gate256], as the reference (src/decode.cu:19)
    in.seg[1] = seg(b.k, x.key, INSG_EPI_STORE);
    in.seg[2] = seg(b.v, x.value, INSG_EPI_STORE);
    run_gemv(c, in);

    insg_attn_op at = {};
    at.qraw = x.gate;
    at.k_raw = x.key;
    at.v = x.value;
    at.q_norm_w = b.q_norm;
    at.k_norm_w = b.k_norm;
    at.k_cache = kc;
    at.v_cache = vc;
    at.out = x.core;
    at.position = x.d_position;
    at.position_offset = position_offset;
    at.max_context = x.max_context;
    at.kv_dtype = x.options.kv_bf16 ? INSG_KV_BF16 : INSG_KV_F32;
    at.fast_trig = x.options.accurate_trig ? 0 : 1;
    at.error_flag = x.d_token + 3;
    at.scratch = x.attn_scratch;
    at.scratch_bytes = insg_gqa_scratch_bytes(x.max_context);
    at.pdl = c.pdl ? 1 : 0;
    if (!c.gemv_only) {
        if (c.rec) insg_check(insg_program_add_attention(c.rec, &at));
        else insg_check(insg_attention_step(&at, c.st));
        c.launches++;
    }

    insg_gemv_op o = {};
    o.in = x.core;
    o.aux = x.gate;
    o.cols = 4096;
    o.prologue = x.options.gate_elementwise ? INSG_PRO_SIGMOID_GATE_QPROJ : INSG_PRO_SIGMOID_GATE_HEAD0;
    o.n_segments = 1;
    o.seg[0] = seg(b.o, x.hidden, INSG_EPI_RESIDUAL);
    residual_output(c, o.seg[0], b.post_norm);
    run_gemv(c, o);

    enqueue_mlp_block(c, b);
}

// ---- the same blocks over T = 2 or 4 consecutive tokens of the sequence (prompt processing): every GEMV streams its
// weights once for the T tokens; the DeltaNet and attention steps, which are recurrences, run token by token.
namespace {
struct Multi {
    float *hidden, *qkv, *z, *a, *b, *core, *qg, *key, *value, *act, *qn;
    int *tokens;
    int T;
    // speculative verify pass (T == 2): the DeltaNet state is read from dn_in, the state after the first token goes to
    // dn_first and the state after the second to dn_second (bases of [24][32][128][128]); null = the workspace's state in place
    const float *dn_in = nullptr;
    float *dn_first = nullptr, *dn_second = nullptr;
    int rows_hint = 0; // eager passes: the rows the pass's last token attends (the host's position + T); 0 inside a replayed graph
    explicit Multi(DecodeWorkspace &x, int t)
        : hidden(x.multi + kMultiHidden), qkv(x.multi + kMultiQkv), z(x.multi + kMultiZ), a(x.multi + kMultiA), b(x.multi + kMultiB),
          core(x.multi + kMultiCore), qg(x.multi + kMultiQg), key(x.multi + kMultiKey), value(x.multi + kMultiValue),
          act(x.multi + kMultiAct), qn(x.multi + kMultiQn), tokens(reinterpret_cast<int *>(x.multi + kMultiTokens)), T(t)
    {
    }
};

void mlp_block_multi(Ctx &c, const Qwen35Decode::Plan::Block &b, const Multi &u)
{
    insg_gemv_op op = {};
    op.in = u.hidden;
    op.norm_w = b.post_norm;
    op.cols = kHidden;
    op.prologue = INSG_PRO_RMSNORM;
    op.tokens = u.T;
    op.n_segments = 1;
    op.seg[0] = seg(b.gate, u.act, INSG_EPI_SWIGLU);
    op.seg[0].packed2 = b.up.data;
    run_gemv(c, op);

    insg_gemv_op dn = {};
    dn.in = u.act;
    dn.cols = kInter;
    dn.prologue = INSG_PRO_PLAIN;
    dn.tokens = u.T;
    dn.n_segments = 1;
    dn.seg[0] = seg(b.down, u.hidden, INSG_EPI_RESIDUAL);
    run_gemv(c, dn);
}

void delta_block_multi(Ctx &c, const Qwen35Decode::Plan::Block &b, int di, const Multi &u)
{
    DecodeWorkspace &x = c.x;
    insg_gemv_op in = {};
    in.in = u.hidden;
    in.norm_w = b.in_norm;
    in.cols = kHidden;
    in.prologue = INSG_PRO_RMSNORM;
    in.tokens = u.T;
    in.n_segments = 4;
    in.seg[0] = seg(b.qkv, u.qkv, INSG_EPI_CONV_SILU);
    in.seg[0].conv_state = x.conv_state + size_t(di) * 8192 * 3;
    in.seg[0].conv_w = b.conv_w;
    in.seg[1] = seg(b.z, u.z, INSG_EPI_STORE);
    in.seg[2] = seg(b.a, u.a, INSG_EPI_DECAY);
    in.seg[2].A_log = b.A_log;
    in.seg[2].dt_bias = b.dt_bias;
    in.seg[3] = seg(b.b, u.b, INSG_EPI_BETA);
    run_gemv(c, in);

    // all T steps in one launch: the state stays on chip between them.  The kernel fetches its state before the
    // dependent-launch wait, which is safe because the launch before it (the GEMV) does not write state.
    const size_t soff = size_t(di) * 32 * 128 * 128;
    if (u.dn_second)
        insg_check(insg_deltanet_decode_verify(u.dn_in + soff, u.dn_first + soff, u.dn_second + soff, u.qkv, u.qkv + 2048, u.qkv + 4096, u.a, u.b,
                                               u.core, 8192, c.pdl ? 1 : 0, c.st));
    else
        insg_check(insg_deltanet_decode_tokens(x.delta_state + soff, u.qkv, u.qkv + 2048, u.qkv + 4096, u.a, u.b, u.core, u.T, 8192,
                                               c.pdl ? 1 : 0, c.st));
    c.launches++;

    insg_gemv_op out = {};
    out.in = u.core;
    out.aux = u.z;
    out.norm_w = b.dn_norm;
    out.cols = 4096;
    out.prologue = INSG_PRO_GATED_RMSNORM;
    out.tokens = u.T;
    out.n_segments = 1;
    out.seg[0] = seg(b.out, u.hidden, INSG_EPI_RESIDUAL);
    run_gemv(c, out);

    mlp_block_multi(c, b, u);
}

void attention_block_multi(Ctx &c, const Qwen35Decode::Plan::Block &b, void *kc, void *vc, const Multi &u)
{
    DecodeWorkspace &x = c.x;
    insg_gemv_op in = {};
    in.in = u.hidden;
    in.norm_w = b.in_norm;
    in.cols = kHidden;
    in.prologue = INSG_PRO_RMSNORM;
    in.tokens = u.T;
    in.n_segments = 3;
    in.seg[0] = seg(b.q, u.qg, INSG_EPI_STORE);
    in.seg[1] = seg(b.k, u.key, INSG_EPI_STORE);
    in.seg[2] = seg(b.v, u.value, INSG_EPI_STORE);
    run_gemv(c, in);

    // token m sits at the device position + m and sees the rows up to its own: the keys and values of the whole chunk
    // go to the cache first, then every token's attention runs in one launch
    insg_attn_op at = {};
    at.qraw = u.qg;
    at.k_raw = u.key;
    at.v = u.value;
    at.q_norm_w = b.q_norm;
    at.k_norm_w = b.k_norm;
    at.k_cache = kc;
    at.v_cache = vc;
    at.out = u.core;
    at.position = x.d_position;
    at.position_offset = 0;
    at.max_context = x.max_context;
    at.kv_dtype = x.options.kv_bf16 ? INSG_KV_BF16 : INSG_KV_F32;
    at.fast_trig = x.options.accurate_trig ? 0 : 1;
    at.error_flag = x.d_token + 3;
    at.scratch = x.attn_scratch;
    at.scratch_bytes = size_t(kBigChunk) * insg_gqa_scratch_bytes(x.max_context);
    insg_check(insg_attention_chunk(&at, u.T, u.qn, u.rows_hint, c.st));
    c.launches += 2;

    insg_gemv_op o = {};
    o.in = u.core;
    o.aux = u.qg;
    o.cols = 4096;
    o.prologue = x.options.gate_elementwise ? INSG_PRO_SIGMOID_GATE_QPROJ : INSG_PRO_SIGMOID_GATE_HEAD0;
    o.tokens = u.T;
    o.n_segments = 1;
    o.seg[0] = seg(b.o, u.hidden, INSG_EPI_RESIDUAL);
    run_gemv(c, o);

    mlp_block_multi(c, b, u);
}
} // namespace

// ------------------------------------------------------------------ public API
void Qwen35Decode::sync_scalars(int token)
{
    Plan &p = plan();
    insg_check(insg_set_scalars(token >= 0 ? x_.d_token : nullptr, token, x_.d_position, x_.position, p.stream));
    launches_++;
}

void Qwen35Decode::load_embed()
{
    Plan &p = plan();
    if (p.embed_ready) return;
    const std::string base = std::string(kLM) + ".model.embed_tokens";
    p.embed = w_.matrix(base);
    p.pinned_mats.push_back(base);
    if (p.embed.cols != kHidden) throw std::runtime_error("unexpected matrix shape: " + base);
    p.embed_ready = true;
}

void Qwen35Decode::enqueue_embed()
{
    Plan &p = plan();
    load_embed();
    if (gemv_only_) return;
    const uint32_t *w = static_cast<const uint32_t *>(p.embed.weight.data);
    const uint8_t *s = static_cast<const uint8_t *>(p.embed.scales.data);
    if (rec_) insg_check(insg_program_add_embed(rec_, w, s, x_.hidden, x_.d_token, p.embed.rows, kHidden));
    else insg_check(insg_mxfp4_embed(w, s, x_.hidden, x_.d_token, p.embed.rows, kHidden, x_.options.use_pdl ? 1 : 0, p.stream));
    launches_++;
}

// Queues the matrices of block l for background upload, so that they arrive while the block before is being repacked.
void Qwen35Decode::prefetch_block(int l)
{
    if (l < 0 || l >= x_.options.n_layers || plan().layers[l].ready) return;
    const std::string name = std::string(kLM) + ".model.layers." + std::to_string(l);
    if (Qwen35Shape::full_attention(l)) {
        for (const char *m : {"q_proj", "k_proj", "v_proj", "o_proj"}) w_.prefetch(name + ".self_attn." + m);
    } else {
        for (const char *m : {"in_proj_qkv", "in_proj_z", "in_proj_a", "in_proj_b", "out_proj"}) w_.prefetch(name + ".linear_attn." + m);
    }
    for (const char *m : {"gate_proj", "up_proj", "down_proj"}) w_.prefetch(name + ".mlp." + m);
}

void Qwen35Decode::load_block_umma(int l)
{
    Plan &p = plan();
    Plan::Block &b = p.layers_umma[l];
    if (b.ready) return;
    Loader L{w_, p.pinned, 1};
    const std::string name = std::string(kLM) + ".model.layers." + std::to_string(l);
    if (Qwen35Shape::full_attention(l)) load_attention(L, name, b);
    else load_delta(L, name, b);
}

void Qwen35Decode::load_block(int l)
{
    Plan &p = plan();
    Plan::Block &b = p.layers[l];
    if (b.ready) return;
    prefetch_block(l + 1);
    Loader L{w_, p.pinned, x_.options.gemv_tcgen05 ? 1 : 0};
    const std::string name = std::string(kLM) + ".model.layers." + std::to_string(l);
    if (Qwen35Shape::full_attention(l)) load_attention(L, name, b);
    else load_delta(L, name, b);
}

void Qwen35Decode::load_head()
{
    Plan &p = plan();
    if (p.head_ready) return;
    Loader L{w_, p.pinned, x_.options.gemv_tcgen05 ? 1 : 0};
    p.final_norm = L.bf16(std::string(kLM) + ".model.norm.weight", kHidden);
    p.lm_head = w_.packed(std::string(kLM) + ".lm_head", x_.options.gemv_tcgen05 ? 1 : 0);
    if (p.lm_head.cols != kHidden || p.lm_head.rows < x_.options.vocab) throw std::runtime_error("unexpected matrix shape: language_model.lm_head");
    p.head_ready = true;
}

void Qwen35Decode::enqueue_delta(int l, bool hidden_prepared, const uint16_t *next_norm)
{
    Plan &p = plan();
    load_block(l);
    Ctx c{x_, p.stream, x_.options.use_pdl, launches_, gemv_only_, rec_, gemv_bytes_, hidden_prepared, next_norm};
    enqueue_delta_block(c, p.layers[l], l - l / 4);
}

void Qwen35Decode::enqueue_attention(int l, bool hidden_prepared, const uint16_t *next_norm)
{
    Plan &p = plan();
    load_block(l);
    const size_t esz = x_.options.kv_bf16 ? 2 : 4;
    const size_t off = size_t(l / 4) * x_.max_context * 1024 * esz;
    Ctx c{x_, p.stream, x_.options.use_pdl, launches_, gemv_only_, rec_, gemv_bytes_, hidden_prepared, next_norm};
    enqueue_attention_block(c, p.layers[l], reinterpret_cast<uint8_t *>(x_.kv_keys) + off, reinterpret_cast<uint8_t *>(x_.kv_values) + off, 0);
}

void Qwen35Decode::enqueue_head(bool hidden_prepared)
{
    Plan &p = plan();
    load_head();
    Ctx c{x_, p.stream, x_.options.use_pdl, launches_, gemv_only_, rec_, gemv_bytes_, hidden_prepared, nullptr};
    insg_gemv_op op = {};
    rmsnorm_input(c, op, p.final_norm);
    op.n_segments = 1;
    op.seg[0] = seg(p.lm_head, x_.logits, INSG_EPI_LOGITS);
    op.seg[0].rows = x_.options.vocab;
    op.argmax_scratch = x_.argmax_scratch;
    op.token_out = x_.d_next;
    op.token_feedback = x_.d_token;
    op.token_log = x_.d_token + 4;
    op.token_log_capacity = x_.max_context + 1;
    op.position_inout = x_.d_position;
    run_gemv(c, op);
}

cudaStream_t Qwen35Decode::execution_stream() { return plan().stream; }

void Qwen35Decode::delta_layer(int l)
{
    if (l < 0 || l >= 32 || Qwen35Shape::full_attention(l)) throw std::runtime_error("not a DeltaNet layer");
    sync_scalars(-1);
    enqueue_delta(l);
    fused_token_valid_ = false;
}

void Qwen35Decode::attention_layer(int l)
{
    if (l < 0 || l >= 32 || !Qwen35Shape::full_attention(l)) throw std::runtime_error("not a full attention layer");
    if (x_.position >= x_.max_context) throw std::runtime_error("KV cache full");
    sync_scalars(-1);
    enqueue_attention(l);
    fused_token_valid_ = false;
}

void Qwen35Decode::layer(int l)
{
    if (Qwen35Shape::full_attention(l)) attention_layer(l);
    else delta_layer(l);
}

// embed, all layers, head: what one graph replay does
void Qwen35Decode::enqueue_token_step()
{
    Plan &p = plan();
    const int n = x_.options.n_layers;
    for (int l = 0; l < n; l++) load_block(l); // every block's norm weight is needed by the block before it
    load_head();
    enqueue_embed();
    for (int l = 0; l < n; l++) {
        // inside the token step nobody touches hidden between two blocks: each block leaves the next one's input prepared
        const uint16_t *next_norm = l + 1 < n ? p.layers[l + 1].in_norm : p.final_norm;
        if (Qwen35Shape::full_attention(l)) enqueue_attention(l, l > 0, next_norm);
        else enqueue_delta(l, l > 0, next_norm);
    }
    enqueue_head(n > 0);
}

// Records the token step as a program (every weight is made resident first: uploads and repacks allocate and
// synchronise, which a recording tolerates and a running kernel does not need).
void Qwen35Decode::build_program()
{
    Plan &p = plan();
    if (p.prog) return;
    insg_program *g = insg_program_create();
    if (!g) throw std::runtime_error("insg_program_create failed");
    const uint64_t before = launches_;
    rec_ = g;
    try {
        enqueue_token_step();
        rec_ = nullptr;
        insg_check(insg_program_finalize(g));
        for (const auto &kv : p.program_options) insg_check(insg_program_set_option(g, kv.first.c_str(), kv.second));
    } catch (...) {
        rec_ = nullptr;
        launches_ = before;
        insg_program_destroy(g);
        throw;
    }
    launches_ = before;
    p.prog = g;
    p.capturing = true; // every weight is resident now
}

// One persistent launch: n_tokens token steps; token >= 0 is stored as the first input token, and the host's position
// as the device position, by the kernel itself.
void Qwen35Decode::run_program(int n_tokens, int token)
{
    Plan &p = plan();
    build_program();
    insg_check(insg_program_run(p.prog, n_tokens, token, x_.position, x_.d_token, x_.d_position, x_.d_token + 3, p.stream));
    launches_++;
}

void Qwen35Decode::set_program_option(const std::string &key, long long value)
{
    Plan &p = plan();
    if (p.prog) insg_check(insg_program_set_option(p.prog, key.c_str(), value));
    for (auto &kv : p.program_options)
        if (kv.first == key) {
            kv.second = value;
            return;
        }
    p.program_options.emplace_back(key, value);
}

bool Qwen35Decode::selftest_barrier_timeout()
{
    if (!persistent()) throw std::runtime_error("selftest_barrier_timeout needs the persistent token kernel");
    Plan &p = plan();
    build_program();
    insg_check(insg_program_selftest_barrier_timeout(p.prog, 2000000ull, x_.d_token + 3, p.stream)); // 2 ms
    launches_++;
    int *result = p.host_result;
    result[1] = 0;
    cuda_check(cudaMemcpyAsync(result + 1, x_.d_token + 3, sizeof(int), cudaMemcpyDeviceToHost, p.stream), "read status");
    cuda_check(cudaStreamSynchronize(p.stream), "synchronize");
    const bool gave_up = result[1] != 0;
    insg_check(insg_program_recover(p.prog, p.stream));
    cuda_check(cudaMemsetAsync(x_.d_token + 3, 0, sizeof(int), p.stream), "clear status");
    cuda_check(cudaMemsetAsync(x_.attn_scratch, 0, size_t(kBigChunk) * insg_gqa_scratch_bytes(x_.max_context), p.stream), "clear attention tickets");
    cuda_check(cudaMemsetAsync(x_.argmax_scratch, 0, 64, p.stream), "clear arg-max ticket");
    fused_token_valid_ = false;
    return gave_up;
}

bool Qwen35Decode::persistent() const { return x_.options.persistent && !x_.options.gemv_tcgen05; }

void Qwen35Decode::replay_token_step()
{
    Plan &p = plan();
    if (!x_.options.use_graph) {
        enqueue_token_step();
        return;
    }
    if (!p.exec) {
        // First call: run eagerly once (loads and repacks every weight, which allocates and synchronises and
        // therefore cannot happen during capture) -- that eager pass IS this token's step.  The graph is
        // captured on the second call, from then on every step is a replay.
        if (!p.capturing) {
            enqueue_token_step();
            p.capturing = true; // weights are resident now
            return;
        }
        const uint64_t before = launches_;
        cuda_check(cudaStreamBeginCapture(p.stream, cudaStreamCaptureModeThreadLocal), "begin graph capture");
        try {
            enqueue_token_step();
        } catch (...) {
            cudaGraph_t g = nullptr;
            cudaStreamEndCapture(p.stream, &g);
            if (g) cudaGraphDestroy(g);
            throw;
        }
        cuda_check(cudaStreamEndCapture(p.stream, &p.graph), "end graph capture");
        p.graph_nodes = launches_ - before;
        launches_ = before;
        cuda_check(cudaGraphInstantiate(&p.exec, p.graph, 0), "instantiate graph");
        // and kMultiSteps steps as one graph for device-fed generation (built here, once, so that no later call pays for it)
        cudaGraph_t g = nullptr;
        cuda_check(cudaStreamBeginCapture(p.stream, cudaStreamCaptureModeThreadLocal), "begin graph capture");
        try {
            for (int k = 0; k < kMultiSteps; k++) enqueue_token_step();
        } catch (...) {
            cudaStreamEndCapture(p.stream, &g);
            if (g) cudaGraphDestroy(g);
            throw;
        }
        launches_ = before;
        cuda_check(cudaStreamEndCapture(p.stream, &g), "end graph capture");
        const cudaError_t e = cudaGraphInstantiate(&p.exec_multi, g, 0);
        cudaGraphDestroy(g);
        cuda_check(e, "instantiate graph");
        // upload now: otherwise the first launch of each graph pays for it
        cuda_check(cudaGraphUpload(p.exec, p.stream), "upload graph");
        cuda_check(cudaGraphUpload(p.exec_multi, p.stream), "upload graph");
    }
    cuda_check(cudaGraphLaunch(p.exec, p.stream), "launch graph");
    launches_ += p.graph_nodes;
}

void Qwen35Decode::forward_token(int token)
{
    if (token < 0 || token >= Qwen35Shape::vocab) throw std::runtime_error("token out of range");
    if (x_.position >= x_.max_context) throw std::runtime_error("KV cache full"); // also bounds the token log
    if (persistent()) {
        run_program(1, token);
    } else {
        sync_scalars(token);
        replay_token_step();
    }
    x_.position++;
    fused_token_valid_ = true;
}

void Qwen35Decode::forward_tokens(const int *tokens, int count)
{
    if (count <= 0) return;
    if (!tokens) throw std::runtime_error("forward_tokens: null token list");
    for (int i = 0; i < count; i++)
        if (tokens[i] < 0 || tokens[i] >= Qwen35Shape::vocab) throw std::runtime_error("token out of range");
    if (x_.position + count > x_.max_context) throw std::runtime_error("KV cache full");
    if (x_.options.gemv_tcgen05) { // that layout takes one token per launch
        for (int i = 0; i < count; i++) forward_token(tokens[i]);
        return;
    }
    Plan &p = plan();
    const int n = x_.options.n_layers;
    for (int l = 0; l < n; l++) load_block(l);
    load_head();
    load_embed();
    Ctx c{x_, p.stream, x_.options.use_pdl, launches_, false, nullptr, nullptr};
    // Long prompts go through the tcgen05 kernel in passes of up to kBigChunk tokens (sixteen tokens per instruction); what
    // is left, and short prompts, through the mma.sync kernel in passes of four.
    const bool big = x_.options.prefill_tcgen05 && count >= 16;
    if (big)
        for (int l = 0; l < n; l++) load_block_umma(l);
    for (int done = 0; done < count;) {
        const int left = count - done;
        const bool use_umma = big && left >= 8;
        const int T = use_umma ? std::min(left, kBigChunk) : (left >= 4 ? 4 : (left >= 2 ? 2 : 1));
        c.layout = use_umma ? 1 : -1;
        const std::vector<Plan::Block> &blocks = use_umma ? p.layers_umma : p.layers;
        Multi u(x_, T);
        if (use_umma) u.rows_hint = x_.position + T; // eager passes only: a replayed graph must not bake the context length in
        sync_scalars(-1); // the chunk's first position; token m of the chunk sits at position + m
        cuda_check(cudaMemcpyAsync(u.tokens, tokens + done, size_t(T) * sizeof(int), cudaMemcpyHostToDevice, p.stream), "copy tokens");
        auto enqueue_chunk = [&] {
            insg_check(insg_mxfp4_embed_tokens(static_cast<const uint32_t *>(p.embed.weight.data), static_cast<const uint8_t *>(p.embed.scales.data),
                                               u.hidden, u.tokens, T, p.embed.rows, kHidden, c.pdl ? 1 : 0, p.stream));
            launches_++;
            for (int l = 0; l < n; l++) {
                if (Qwen35Shape::full_attention(l)) {
                    const size_t esz = x_.options.kv_bf16 ? 2 : 4;
                    const size_t off = size_t(l / 4) * x_.max_context * 1024 * esz;
                    attention_block_multi(c, blocks[l], reinterpret_cast<uint8_t *>(x_.kv_keys) + off,
                                          reinterpret_cast<uint8_t *>(x_.kv_values) + off, u);
                } else {
                    delta_block_multi(c, blocks[l], l - l / 4, u);
                }
            }
        };
        if (!use_umma && T == kChunk && x_.options.use_graph && p.chunk_warm) {
            // full chunks replay one graph (tokens and position are read from device memory); the first full chunk ran
            // eagerly (first launches of a kernel variant set function attributes)
            const uint64_t before = launches_;
            if (!p.exec_chunk) {
                cudaGraph_t g = nullptr;
                cuda_check(cudaStreamBeginCapture(p.stream, cudaStreamCaptureModeThreadLocal), "begin graph capture");
                try {
                    enqueue_chunk();
                } catch (...) {
                    cudaStreamEndCapture(p.stream, &g);
                    if (g) cudaGraphDestroy(g);
                    throw;
                }
                cuda_check(cudaStreamEndCapture(p.stream, &g), "end graph capture");
                const cudaError_t e = cudaGraphInstantiate(&p.exec_chunk, g, 0);
                cudaGraphDestroy(g);
                cuda_check(e, "instantiate graph");
                p.chunk_nodes = launches_ - before;
            }
            launches_ = before + p.chunk_nodes;
            cuda_check(cudaGraphLaunch(p.exec_chunk, p.stream), "launch graph");
        } else {
            enqueue_chunk();
            p.chunk_warm |= !use_umma && T == kChunk;
        }
        x_.position += T;
        done += T;
        if (done == count) // the sequence's hidden state is the last token's
            cuda_check(cudaMemcpyAsync(x_.hidden, u.hidden + size_t(T - 1) * kHidden, kHidden * sizeof(float), cudaMemcpyDeviceToDevice, p.stream),
                       "copy hidden");
    }
    // logits of the last token (from the fp32 hidden vector; nothing was left prepared); the head also writes the
    // arg-max, so logits_argmax() needs no further launch
    x_.position--;
    sync_scalars(tokens[count - 1]);
    enqueue_head(false);
    x_.position++;
    fused_token_valid_ = true;
    p.capturing = true; // every weight is resident now: the next forward_token may capture its graph
}

// A kernel gave up on a wait: put the barrier state, the tickets and the status word back so that later calls work.
void Qwen35Decode::recover_after_timeout()
{
    Plan &p = plan();
    if (p.prog) insg_program_recover(p.prog, p.stream);
    cudaMemsetAsync(x_.d_token + 3, 0, sizeof(int), p.stream);
    cudaMemsetAsync(x_.attn_scratch, 0, size_t(kBigChunk) * insg_gqa_scratch_bytes(x_.max_context), p.stream);
    cudaMemsetAsync(x_.argmax_scratch, 0, 64, p.stream);
    cudaStreamSynchronize(p.stream);
    fused_token_valid_ = false;
}

int Qwen35Decode::logits_argmax()
{
    Plan &p = plan();
    if (!fused_token_valid_) { // logits were not produced by the fused head: reduce them now
        insg_check(insg_argmax_logits(x_.logits, x_.options.vocab, x_.d_next, p.stream));
        launches_++;
    }
    int *result = p.host_result; // next token, kernel wait-expired flag
    result[0] = -1;
    result[1] = 0;
    cuda_check(cudaMemcpyAsync(result, x_.d_next, 2 * sizeof(int), cudaMemcpyDeviceToHost, p.stream), "read token");
    cuda_check(cudaStreamSynchronize(p.stream), "synchronize");
    if (result[1]) {
        recover_after_timeout();
        throw std::runtime_error("a bounded wait inside a GPU kernel expired");
    }
    return result[0];
}

int Qwen35Decode::decode_token(int token)
{
    forward_token(token);
    return logits_argmax();
}

std::vector<int> Qwen35Decode::generate(int first_token, int count)
{
    std::vector<int> out(size_t(count > 0 ? count : 0));
    if (count <= 0) return out;
    if (first_token < 0 || first_token >= Qwen35Shape::vocab) throw std::runtime_error("token out of range");
    if (x_.position + count > x_.max_context) throw std::runtime_error("KV cache full");
    Plan &p = plan();
    const int start = x_.position;
    if (persistent()) {
        // the kernel loops over the tokens itself: the head feeds its arg-max back and advances the position
        run_program(count, first_token);
        x_.position += count;
        fused_token_valid_ = true;
        int *flag = p.host_result + 1;
        *flag = 0;
        cuda_check(cudaMemcpyAsync(out.data(), x_.d_token + 4 + start, size_t(count) * sizeof(int), cudaMemcpyDeviceToHost, p.stream),
                   "read tokens");
        cuda_check(cudaMemcpyAsync(flag, x_.d_token + 3, sizeof(int), cudaMemcpyDeviceToHost, p.stream), "read status");
        cuda_check(cudaStreamSynchronize(p.stream), "synchronize");
        if (*flag) {
            recover_after_timeout();
            throw std::runtime_error("a bounded wait inside a GPU kernel expired");
        }
        return out;
    }
    sync_scalars(first_token);
    for (int i = 0; i < count;) {
        // The head feeds its arg-max back into d_token and advances d_position, so consecutive steps need nothing from
        // the host.  Once the graphs exist, runs of kMultiSteps steps go out as one graph: the dependent-launch edges
        // then also span the token boundaries, and there is one graph launch per kMultiSteps tokens.
        if (x_.options.use_graph && p.exec_multi && count - i >= kMultiSteps) {
            cuda_check(cudaGraphLaunch(p.exec_multi, p.stream), "launch graph");
            launches_ += p.graph_nodes * kMultiSteps;
            x_.position += kMultiSteps;
            i += kMultiSteps;
        } else {
            replay_token_step();
            x_.position++;
            i++;
        }
    }
    fused_token_valid_ = true;
    cuda_check(cudaMemcpyAsync(out.data(), x_.d_token + 4 + start, size_t(count) * sizeof(int), cudaMemcpyDeviceToHost, p.stream),
               "read tokens");
    cuda_check(cudaStreamSynchronize(p.stream), "synchronize");
    return out;
}

void Qwen35Decode::profile_gemv_chain(int replays, float *ms_per_token, uint64_t *bytes, int *launches)
{
    Plan &p = plan();
    if (!p.capturing && !p.exec && !p.prog) throw std::runtime_error("profile_gemv_chain needs a forwarded token (weights resident)");
    replays = std::max(1, std::min(replays, 64));
    if (x_.position + replays + 2 > x_.max_context) throw std::runtime_error("profile_gemv_chain: not enough context left");
    uint64_t chain_bytes = 0;
    const uint64_t before = launches_;
    cudaGraphExec_t exec = nullptr;
    insg_program *chain = nullptr;
    gemv_only_ = true;
    gemv_bytes_ = &chain_bytes;
    try {
        if (persistent()) {
            chain = insg_program_create();
            if (!chain) throw std::runtime_error("insg_program_create failed");
            rec_ = chain;
            enqueue_token_step();
            rec_ = nullptr;
            insg_check(insg_program_finalize(chain));
            for (const auto &kv : p.program_options) insg_check(insg_program_set_option(chain, kv.first.c_str(), kv.second));
        } else {
            cudaGraph_t graph = nullptr;
            cuda_check(cudaStreamBeginCapture(p.stream, cudaStreamCaptureModeThreadLocal), "begin graph capture");
            try {
                enqueue_token_step();
            } catch (...) {
                cudaStreamEndCapture(p.stream, &graph);
                if (graph) cudaGraphDestroy(graph);
                throw;
            }
            cuda_check(cudaStreamEndCapture(p.stream, &graph), "end graph capture");
            const cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
            cudaGraphDestroy(graph);
            cuda_check(e, "instantiate graph");
        }
    } catch (...) {
        rec_ = nullptr;
        gemv_only_ = false;
        gemv_bytes_ = nullptr;
        launches_ = before;
        if (chain) insg_program_destroy(chain);
        throw;
    }
    gemv_only_ = false;
    gemv_bytes_ = nullptr;
    const int chain_launches = int(launches_ - before);
    launches_ = before;
    auto once = [&] {
        if (chain) insg_check(insg_program_run(chain, 1, -1, -1, nullptr, nullptr, x_.d_token + 3, p.stream));
        else cuda_check(cudaGraphLaunch(exec, p.stream), "launch graph");
    };
    cudaEvent_t a = nullptr, b = nullptr;
    cudaError_t e = cudaSuccess;
    float ms = 0.f;
    try {
        cuda_check(cudaEventCreate(&a), "event");
        cuda_check(cudaEventCreate(&b), "event");
        once(); // warm
        cuda_check(cudaEventRecord(a, p.stream), "event record");
        for (int i = 0; i < replays; i++) once();
        cuda_check(cudaEventRecord(b, p.stream), "event record");
        e = cudaStreamSynchronize(p.stream);
        if (e == cudaSuccess) cudaEventElapsedTime(&ms, a, b);
    } catch (...) {
        if (a) cudaEventDestroy(a);
        if (b) cudaEventDestroy(b);
        if (exec) cudaGraphExecDestroy(exec);
        if (chain) insg_program_destroy(chain);
        throw;
    }
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    if (exec) cudaGraphExecDestroy(exec);
    if (chain) insg_program_destroy(chain);
    cuda_check(e, "synchronize");
    *ms_per_token = ms / float(replays);
    *bytes = chain_bytes;
    *launches = chain_launches;
    fused_token_valid_ = false;
    sync_scalars(-1); // the head operations advanced the device-side position; put the host's view back
}

namespace {
// Runs `enqueue` on the stream: eagerly the first time (kernel variants set their function attributes on first use),
// from then on as a replay of a graph captured on the second call.  The launches must read their variable inputs (tokens,
// position) from device memory.
template <class F> void run_graphed(bool use_graph, cudaStream_t st, cudaGraphExec_t &exec, int &runs, uint64_t &launches, F &&enqueue)
{
    if (!use_graph || runs == 0) {
        enqueue();
        runs++;
        return;
    }
    if (!exec) {
        const uint64_t before = launches;
        cudaGraph_t g = nullptr;
        cuda_check(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal), "begin graph capture");
        try {
            enqueue();
        } catch (...) {
            cudaStreamEndCapture(st, &g);
            if (g) cudaGraphDestroy(g);
            throw;
        }
        cuda_check(cudaStreamEndCapture(st, &g), "end graph capture");
        const cudaError_t e = cudaGraphInstantiate(&exec, g, 0);
        cudaGraphDestroy(g);
        cuda_check(e, "instantiate graph");
        launches = before;
    }
    cuda_check(cudaGraphLaunch(exec, st), "launch graph");
    launches++;
}
} // namespace

int Qwen35Decode::mtp_draft(int token) { return mtp_step(token, true); }

// The MTP block at the current position (reference: src/decode.cu:24-68).  draft = false stops before the head: the call
// then only leaves the position's row in the MTP cache (a speculative decoder needs every row, the prompt's included).
int Qwen35Decode::mtp_step(int token, bool draft)
{
    if (token < 0 || token >= Qwen35Shape::vocab) throw std::runtime_error("token out of range");
    if (x_.position < 1) throw std::runtime_error("mtp_draft needs a forwarded token");
    Plan &p = plan();
    const std::string m = std::string(kLM) + ".mtp";
    if (!p.mtp_ready) {
        Loader L{w_, p.pinned, x_.options.gemv_tcgen05 ? 1 : 0};
        p.mtp_fc = L.bf16(m + ".fc.weight", size_t(kHidden) * 2 * kHidden);
        p.mtp_norm_e = L.bf16(m + ".pre_fc_norm_embedding.weight", kHidden);
        p.mtp_norm_h = L.bf16(m + ".pre_fc_norm_hidden.weight", kHidden);
        p.mtp_norm = L.bf16(m + ".norm.weight", kHidden);
        load_attention(L, m + ".layers.0", p.mtp);
        p.mtp_ready = true;
    }
    if (!p.head_ready || !p.embed_ready) throw std::runtime_error("mtp_draft needs a forwarded token");
    const bool pdl = x_.options.use_pdl;
    sync_scalars(token);
    run_graphed(x_.options.use_graph, p.stream, p.exec_mtp[draft ? 1 : 0], p.mtp_runs[draft ? 1 : 0], launches_, [&] {
        // embedding of the input token and the last hidden state, each normalised, side by side in qkv[8192]
        insg_check(insg_mxfp4_embed(static_cast<const uint32_t *>(p.embed.weight.data), static_cast<const uint8_t *>(p.embed.scales.data),
                                    x_.down, x_.d_token, p.embed.rows, kHidden, 0, p.stream));
        insg_check(insg_rmsnorm_bf16(x_.down, p.mtp_norm_e, nullptr, x_.qkv, 1, kHidden, 0, p.stream));
        insg_check(insg_rmsnorm_bf16(x_.hidden, p.mtp_norm_h, nullptr, x_.qkv + kHidden, 1, kHidden, 0, p.stream));
        insg_check(insg_bf16_gemv(p.mtp_fc, x_.qkv, x_.hidden, kHidden, 2 * kHidden, 0, p.stream)); // overwrites the residual, as the reference
        launches_ += 4;
        Ctx c{x_, p.stream, pdl, launches_, false, nullptr, nullptr};
        enqueue_attention_block(c, p.mtp, x_.mtp_keys, x_.mtp_values, -1); // rotary position / cache row position-1, position rows attended
        if (!draft) return;
        insg_gemv_op op = {};
        op.in = x_.hidden;
        op.norm_w = p.mtp_norm;
        op.x_out = x_.norm;
        op.cols = kHidden;
        op.prologue = INSG_PRO_RMSNORM;
        op.n_segments = 1;
        op.seg[0] = seg(p.lm_head, x_.logits, INSG_EPI_LOGITS);
        op.seg[0].rows = x_.options.vocab;
        op.argmax_scratch = x_.argmax_scratch;
        op.token_out = x_.d_next;
        run_gemv(c, op);
    });
    if (!draft) {
        fused_token_valid_ = false;
        return -1;
    }
    fused_token_valid_ = true;
    return logits_argmax();
}

// ---- speculative greedy decode: draft-1 / verify ---------------------------------------------------------------------
// The reference has the draft half only (src/decode.cu:24-68).  Verification runs the main model on [token, draft] as
// one two-token pass over the weights; the first token's state is always kept, the second one's only when the draft
// was right: the DeltaNet step writes the state after its first token in place and the state after its second into a
// second buffer (accept = swap the two), the convolution history is rebuilt from a snapshot on a reject, and the KV row
// of a rejected draft is simply overwritten later.  Greedy output is identical to plain greedy decode.
int Qwen35Decode::prime_speculative(const int *prompt, int count)
{
    if (!prompt || count < 1) throw std::runtime_error("prime_speculative: empty prompt");
    for (int i = 0; i < count; i++) {
        forward_token(prompt[i]);
        if (i + 1 < count) mtp_step(prompt[i + 1], false); // row i of the MTP cache: hidden state i with the embedding of token i + 1
    }
    return logits_argmax();
}

std::vector<int> Qwen35Decode::generate_speculative(int first_token, int count, int *accepted, const int *forced_drafts)
{
    std::vector<int> out;
    if (accepted) *accepted = 0;
    if (count <= 0) return out;
    if (first_token < 0 || first_token >= Qwen35Shape::vocab) throw std::runtime_error("token out of range");
    if (x_.position + count > x_.max_context) throw std::runtime_error("KV cache full");
    if (x_.options.gemv_tcgen05) throw std::runtime_error("speculative decode runs on the mma.sync weight layout");
    Plan &p = plan();
    const int n = x_.options.n_layers;
    for (int l = 0; l < n; l++) load_block(l);
    load_head();
    load_embed();
    const size_t state_floats = size_t(24) * 32 * 128 * 128, conv_floats = size_t(24) * 8192 * 3;
    if (!p.spec_state) {
        dev_alloc(&p.spec_state, state_floats);
        dev_alloc(&p.spec_conv, conv_floats);
        dev_alloc(&p.spec_logits, size_t(2) * Qwen35Shape::vocab);
        dev_alloc(&p.spec_pair, 2);
        cuda_check(cudaMallocHost(&p.spec_host, 4 * sizeof(int)), "cudaMallocHost");
    }
    Ctx c{x_, p.stream, x_.options.use_pdl, launches_, false, nullptr, nullptr};
    c.layout = 0;
    float *cur = x_.delta_state, *alt = p.spec_state;
    int tok = first_token, hits = 0;
    out.reserve(size_t(count));
    auto settle = [&] { // the workspace's own buffer holds the live state again (plain decode and its graph use that pointer)
        if (cur != x_.delta_state) {
            cuda_check(cudaMemcpyAsync(x_.delta_state, cur, state_floats * sizeof(float), cudaMemcpyDeviceToDevice, p.stream), "copy state");
            std::swap(cur, alt);
        }
    };
    while (int(out.size()) < count) {
        if (count - int(out.size()) == 1) { // one token left: a plain step
            settle();
            tok = decode_token(tok);
            out.push_back(tok);
            break;
        }
        const int P = x_.position;
        const int draft = forced_drafts ? forced_drafts[out.size()] : mtp_draft(tok);
        if (draft < 0 || draft >= Qwen35Shape::vocab) throw std::runtime_error("draft token out of range");
        // ---- verify: tokens [tok, draft] at positions P, P + 1 ----
        Multi u(x_, 2);
        u.dn_in = cur;
        u.dn_first = cur;
        u.dn_second = alt;
        p.spec_host[0] = tok;
        p.spec_host[1] = draft;
        sync_scalars(-1);
        cuda_check(cudaMemcpyAsync(u.tokens, p.spec_host, 2 * sizeof(int), cudaMemcpyHostToDevice, p.stream), "copy tokens");
        const int which = cur == x_.delta_state ? 0 : 1;
        run_graphed(x_.options.use_graph, p.stream, p.exec_verify[which], p.verify_runs[which], launches_, [&] {
            cuda_check(cudaMemcpyAsync(p.spec_conv, x_.conv_state, conv_floats * sizeof(float), cudaMemcpyDeviceToDevice, p.stream), "snapshot history");
            for (int m = 0; m < 2; m++) {
                insg_check(insg_mxfp4_embed(static_cast<const uint32_t *>(p.embed.weight.data), static_cast<const uint8_t *>(p.embed.scales.data),
                                            u.hidden + size_t(m) * kHidden, u.tokens + m, p.embed.rows, kHidden, 0, p.stream));
                launches_++;
            }
            for (int l = 0; l < n; l++) {
                if (Qwen35Shape::full_attention(l)) {
                    const size_t off = size_t(l / 4) * x_.max_context * 1024 * (x_.options.kv_bf16 ? 2 : 4);
                    attention_block_multi(c, p.layers[l], reinterpret_cast<uint8_t *>(x_.kv_keys) + off, reinterpret_cast<uint8_t *>(x_.kv_values) + off, u);
                } else {
                    delta_block_multi(c, p.layers[l], l - l / 4, u);
                }
            }
            insg_gemv_op head = {};
            head.in = u.hidden;
            head.norm_w = p.final_norm;
            head.cols = kHidden;
            head.prologue = INSG_PRO_RMSNORM;
            head.tokens = 2;
            head.n_segments = 1;
            head.seg[0] = seg(p.lm_head, p.spec_logits, INSG_EPI_STORE);
            head.seg[0].rows = x_.options.vocab;
            run_gemv(c, head);
            insg_check(insg_argmax_rows(p.spec_logits, x_.options.vocab, x_.options.vocab, 2, p.spec_pair, p.stream));
            launches_++;
        });
        int *res = p.host_result;
        cuda_check(cudaMemcpyAsync(res, p.spec_pair, 2 * sizeof(int), cudaMemcpyDeviceToHost, p.stream), "read tokens");
        cuda_check(cudaStreamSynchronize(p.stream), "synchronize");
        const int r1 = res[0], r2 = res[1];
        out.push_back(r1);
        if (r1 == draft) { // accepted: both positions stand
            hits++;
            out.push_back(r2);
            std::swap(cur, alt);
            if (!forced_drafts) { // row P of the MTP cache: hidden state P with the embedding of the accepted draft
                cuda_check(cudaMemcpyAsync(x_.hidden, u.hidden, kHidden * sizeof(float), cudaMemcpyDeviceToDevice, p.stream), "copy hidden");
                x_.position = P + 1;
                mtp_step(draft, false);
            }
            cuda_check(cudaMemcpyAsync(x_.hidden, u.hidden + kHidden, kHidden * sizeof(float), cudaMemcpyDeviceToDevice, p.stream), "copy hidden");
            x_.position = P + 2;
            tok = r2;
        } else { // rejected: the state after the first token is the live one
            insg_check(insg_conv_rollback(x_.conv_state, p.spec_conv, (long long)(conv_floats / 3), p.stream));
            launches_++;
            cuda_check(cudaMemcpyAsync(x_.hidden, u.hidden, kHidden * sizeof(float), cudaMemcpyDeviceToDevice, p.stream), "copy hidden");
            x_.position = P + 1;
            tok = r1;
        }
    }
    settle();
    cuda_check(cudaStreamSynchronize(p.stream), "synchronize");
    fused_token_valid_ = false;
    p.capturing = true;
    if (accepted) *accepted = hits;
    return out;
}

} // namespace insignia
