// Token loop of the Qwen3.5-style hybrid: per-sequence workspace + decode driver.
//
// Drop-in for the reference header of the same name (include/insignia_decode.hpp:5-24,
// behaviour: src/decode.cu:9-69): same classes, public fields, methods and error
// strings.  Underneath, each layer is five fused sm_100a operations instead of
// eighteen launches; a token step (forward_token / decode_token / generate) is 162
// launches chained with programmatic dependent launch and replayed from a CUDA graph,
// or, optionally, one persistent cooperative launch that walks all of them.
// Additive members are marked.
#pragma once
#include "insignia_qwen35.hpp"

#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <string>
#include <vector>

struct insg_program;

namespace insignia {

// Additive knobs; the defaults reproduce the reference engine's behaviour.
struct DecodeOptions {
    bool kv_bf16 = false;          // false: fp32 KV cache as the reference (src/decode.cu:10); true: bf16 cache
    bool gate_elementwise = false; // false: head-broadcast attention gate (src/qwen_kernels.cu:36);
                                   // true: element-wise gate (tools/reference_all_layers.py:13)
    bool accurate_trig = false;    // false: __powf/__sinf/__cosf for RoPE (src/ops.cu:9); true: powf/sincosf
    bool persistent = false;       // false: one launch per fused operation (162 per token); true: the token step is ONE
                                   // persistent cooperative launch with grid barriers between the operations (measured
                                   // slower than the graph of launches on B200: the barrier chain costs what the
                                   // dependent-launch chain costs, and its phases cannot overlap one another's tails)
    bool use_graph = true;         // launch per operation: replay the token step from a CUDA graph
    bool use_pdl = true;           // programmatic dependent launch between kernels
    bool gemv_tcgen05 = false;     // true: weights through tcgen05.mma kind::mxf4 (TMA-fed); false: the mma.sync streaming kernel
    bool prepared_inputs = true;   // a GEMV that writes the residual stream or the SwiGLU output also leaves the next GEMV's
                                   // input ready as fp16 pieces (and its sum of squares), so that one starts streaming
                                   // without normalising or converting anything; false: every GEMV prepares its own input
    bool prefill_tcgen05 = true;   // forward_tokens with 16 or more tokens: passes of up to 256 tokens through the tcgen05
                                   // kernel (kind::mxf4, sixteen tokens per instruction; needs a second, tile-layout copy of
                                   // the weights); false: always passes of four tokens through the mma.sync kernel
    int n_layers = Qwen35Shape::layers;
    int vocab = Qwen35Shape::vocab;
};

class INSIGNIA_API DecodeWorkspace final {
public:
    explicit DecodeWorkspace(int max_context = 4096, cudaStream_t stream = nullptr);
    // Additive: options (KV cache element type).
    DecodeWorkspace(int max_context, cudaStream_t stream, const DecodeOptions &options);
    ~DecodeWorkspace();
    DecodeWorkspace(const DecodeWorkspace &) = delete;

    // Public device buffers, same names and extents as the reference (src/decode.cu:10).
    // hidden[4096] is the residual stream; logits[248320]; delta_state[24][32][128][128];
    // conv_state[24][8192][3]; kv_* [8][ctx][1024]; mtp_* [ctx][1024].  With a bf16 cache
    // kv_*/mtp_* point at bf16 storage of the same element count.
    float *hidden{}, *norm{}, *qkv{}, *attn_gate{}, *key{}, *value{}, *z{}, *a{}, *b{}, *core{}, *gate{}, *up{},
        *down{}, *logits{}, *delta_state{}, *conv_state{}, *kv_keys{}, *kv_values{}, *mtp_keys{}, *mtp_values{};
    int max_context{}, position{};
    cudaStream_t stream{};

    // Additive.
    DecodeOptions options{};
    int *d_token{};      // device: token fed to the embedding
    int *d_position{};   // device: rotary position / cache row of the current token
    int *d_next{};       // device: arg-max of the last logits
    void *attn_scratch{};
    void *argmax_scratch{};
    float *multi{};      // device: activations of up to 256 consecutive tokens (forward_tokens)
    void *umma_scratch{}; // device: digit image of the activations for the tcgen05 kernel (forward_tokens)
    size_t umma_scratch_bytes{};
    void *prep{};        // device: prepared GEMV inputs, fp16 [2][4096] + fp16 [2][12288] + fp32 [2][296] sums of squares
    void reset(); // zero recurrent state and position, as a fresh workspace

private:
    void allocate();
};

class INSIGNIA_API Qwen35Decode final {
public:
    Qwen35Decode(Qwen35Weights &weights, DecodeWorkspace &workspace);
    ~Qwen35Decode();
    void delta_layer(int layer);
    void attention_layer(int layer);
    void layer(int layer);
    int decode_token(int token);
    void forward_token(int token);
    // Additive: forward_token for `count` consecutive tokens (a prompt), the GEMVs taking four tokens per pass over the
    // weights; leaves the same state as the loop would, and the logits and arg-max of the last token.
    void forward_tokens(const int *tokens, int count);
    int logits_argmax();
    int mtp_draft(int input_token);

    // Additive: speculative greedy decode, draft-1 / verify (the reference has the draft half only).
    // prime_speculative: the prompt token by token like forward_token, also leaving every position's row in the MTP
    // head's cache; returns the greedy next token.  generate_speculative: `count` tokens, each step one MTP draft and
    // one two-token verify pass of the main model; a right draft yields two tokens per pass, a wrong one is rolled back
    // (DeltaNet state, convolution history).  Output identical to plain greedy decode.  *accepted receives the number of
    // drafts that were right.  forced_drafts (optional, `count` entries): drafts from the caller instead of the MTP head.
    int prime_speculative(const int *prompt, int count);
    std::vector<int> generate_speculative(int first_token, int count, int *accepted = nullptr, const int *forced_drafts = nullptr);

    // Additive: greedy generation with the arg-max fed back on the device; one sync at the end.
    std::vector<int> generate(int first_token, int count);
    uint64_t launch_count() const noexcept { return launches_; }
    cudaStream_t execution_stream();
    // Additive: the fused-GEMV operations of one token step alone (no DeltaNet, attention or embedding work between
    // them), run `replays` times between two events: as a graph of launches with dependent-launch overlap, or with
    // `persistent` as one persistent launch each.  Gives the weight-streaming time of a token.  The sequence state
    // (hidden, convolution history) is meaningless afterwards: reset the workspace before decoding again.
    void profile_gemv_chain(int replays, float *ms_per_token, uint64_t *bytes, int *launches);
    // Additive: an option of the persistent program (insg_program_set_option), e.g. "prefetch_records"; takes effect at
    // once and is applied again to programs built later.
    void set_program_option(const std::string &key, long long value);
    // Additive: failure-detection self-test of the persistent launch: one run whose first grid barrier can never be
    // met, with a short wait limit.  Returns true when the kernel gave up, raised its error status and the engine
    // recovered.  The sequence state is meaningless afterwards (reset the workspace).
    bool selftest_barrier_timeout();
    struct Plan; // resolved weight pointers + captured graph (opaque)

private:
    Plan &plan();
    void sync_scalars(int token);
    void enqueue_embed();
    // hidden_prepared: the launch before left this block's input prepared; next_norm: weight of the RMSNorm that reads
    // this block's output next (the block then leaves that input prepared), or null when the caller may touch hidden
    void load_embed();
    void load_block(int layer);
    void load_block_umma(int layer);
    void prefetch_block(int layer);
    void load_head();
    void enqueue_delta(int layer, bool hidden_prepared = false, const uint16_t *next_norm = nullptr);
    void enqueue_attention(int layer, bool hidden_prepared = false, const uint16_t *next_norm = nullptr);
    void enqueue_head(bool hidden_prepared = false);
    void enqueue_token_step();
    void replay_token_step();
    Qwen35Weights &w_;
    DecodeWorkspace &x_;
    std::unique_ptr<Plan> plan_;
    int mtp_step(int token, bool draft);
    void build_program();
    void run_program(int n_tokens, int token);
    void recover_after_timeout();
    bool persistent() const;
    uint64_t launches_{};
    bool gemv_only_{};            // enqueue only the fused GEMVs (profile_gemv_chain)
    insg_program *rec_{};         // non-null while a program is being recorded
    uint64_t *gemv_bytes_{};      // optional byte counter of the GEMVs enqueued
    bool fused_token_valid_{};
};

} // namespace insignia
