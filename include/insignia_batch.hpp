// Greedy decode of several independent sequences in lock step on ONE copy of the weights.
//
// Additive: the reference decodes one sequence (include/insignia_decode.hpp:5-24, src/decode.cu:14-23).  A batch step
// runs the same fused operations, with every weight matrix streamed once for all sequences: the GEMVs take the
// sequences as the tokens of a several-token launch (two or four through the mma.sync kernel, five to eight through
// the tcgen05 kernel), the DeltaNet step runs one grid row per sequence, the attention step one launch per sequence
// on that sequence's own cache.  Every sequence has its own recurrent state, convolution history and KV cache; all
// advance by one position per step.
#pragma once
#include "insignia_qwen35.hpp"

#include <cuda_runtime.h>

#include <memory>
#include <vector>

namespace insignia {

struct BatchOptions {
    bool kv_bf16 = false;          // as DecodeOptions
    bool gate_elementwise = false;
    bool accurate_trig = false;
    bool use_graph = true;         // replay the step from a CUDA graph
    int n_layers = Qwen35Shape::layers;
    int vocab = Qwen35Shape::vocab;
};

class INSIGNIA_API Qwen35BatchDecode final {
public:
    // sequences: 1..8.  Allocates every per-sequence buffer (about 50 MiB of recurrent state and 64 KiB of fp32 cache per
    // position, per sequence).
    Qwen35BatchDecode(Qwen35Weights &weights, int sequences, int max_context, cudaStream_t stream = nullptr, const BatchOptions &options = {});
    ~Qwen35BatchDecode();
    Qwen35BatchDecode(const Qwen35BatchDecode &) = delete;

    int sequences() const noexcept { return sequences_; }
    int position() const noexcept { return position_; }
    // One step without a read-back (prompt ingestion): tokens[s] goes into sequence s.  Asynchronous.
    void forward_tokens(const int *tokens);
    // One step: next[s] = greedy next token of sequence s.  Synchronises.
    void decode_tokens(const int *tokens, int *next);
    // `count` steps, each sequence's arg-max fed back on the device; out[step * sequences + s].  One synchronisation.
    void generate(const int *first_tokens, int count, int *out);
    void reset();
    // Copies sequence s's residual stream / first `count` floats of its DeltaNet state to the host (tests).
    void read_hidden(int sequence, float *out);
    void read_delta_state(int sequence, float *out, uint64_t count);
    uint64_t launch_count() const noexcept { return launches_; }
    cudaStream_t execution_stream();

private:
    struct Impl;
    void enqueue_step();
    void run_step();
    Qwen35Weights &w_;
    int sequences_{}, max_context_{}, position_{};
    BatchOptions options_{};
    std::unique_ptr<Impl> impl_;
    uint64_t launches_{};
};

} // namespace insignia
