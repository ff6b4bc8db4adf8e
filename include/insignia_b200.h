/*
 * insignia_b200 -- C ABI of the sm_100a decode kernels and of the decode engine.
 *
 * This is the boundary a maintainer of the reference (novysvet/insignia) binds
 * to replace its token loop.  Every entry point takes plain pointers, sizes and
 * a CUDA stream; none allocates device memory or synchronises unless its comment
 * says so.  Return value: 0 on success, a negative INSG_E_* code otherwise
 * (insg_last_error() gives text).  All pointers are DEVICE pointers unless
 * marked "host".  Each comment cites the reference interface the entry point
 * replaces, as path:line in the reference project.
 */
#ifndef INSIGNIA_B200_H
#define INSIGNIA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define INSG_API __attribute__((visibility("default")))
#else
#define INSG_API
#endif

typedef struct CUstream_st *insg_stream_t; /* == cudaStream_t */

enum {
    INSG_OK = 0,
    INSG_E_SHAPE = -1,   /* unsupported or inconsistent sizes            */
    INSG_E_CUDA = -2,    /* a CUDA runtime call or launch failed         */
    INSG_E_ARG = -3,     /* null pointer / bad enum / misaligned pointer */
    INSG_E_RUNTIME = -4, /* host-side std::runtime_error (engine calls)  */
    INSG_E_LIMIT = -5    /* size beyond a documented fixed maximum       */
};

INSG_API const char *insg_last_error(void);  /* host string, thread-local */
INSG_API int insg_version(void);
/* Kept for binary compatibility: this build has no process-wide tuning keys (every launch shape is fixed per kernel;
 * per-engine choices are DecodeOptions), so every key answers INSG_E_ARG. */
INSG_API int insg_tune_set(const char *key /* host */, int value);

/* ------------------------------------------------------------------ MXFP4 */

/* y[rows] = W x, W in the MLX checkpoint layout: U32[rows][cols/8] (nibble j of
 * word i = element 8i+j) + U8[rows][cols/32] E8M0 scales; x, y fp32.
 * cols % 32 == 0.  Replaces mxfp4_gemv_mlx (include/insignia_layout.cuh:48,
 * src/mxfp4.cu:41-77); the warps_per_row knob of the reference has no meaning
 * here and is dropped. */
INSG_API int insg_mxfp4_gemv_mlx(const uint32_t *weight, const uint8_t *scales, const float *x, float *y, int rows,
                                 int cols, insg_stream_t stream);

/* out[cols] = dequantised row `row` (the embedding lookup).  Replaces
 * mxfp4_get_row_mlx (include/insignia_layout.cuh:49, src/mxfp4.cu:132-133). */
INSG_API int insg_mxfp4_get_row_mlx(const uint32_t *weight, const uint8_t *scales, float *out, int row, int cols,
                                    insg_stream_t stream);

/* Same lookup with the row index read from device memory (*device_row), so the call can sit
 * inside a captured CUDA graph; rows outside [0, rows) produce zeros.  Replaces
 * Qwen35Weights::embed (src/qwen35.cu:9) on the engine's path. */
INSG_API int insg_mxfp4_embed(const uint32_t *weight, const uint8_t *scales, float *out, const int *device_row,
                              int rows, int cols, int pdl, insg_stream_t stream);

/* The same lookup for `count` tokens of a prompt pass in one launch: row indices device_rows[0..count), outputs
 * out[m * cols ...].  Each row equals insg_mxfp4_embed's. */
INSG_API int insg_mxfp4_embed_tokens(const uint32_t *weight, const uint8_t *scales, float *out, const int *device_rows,
                                     int count, int rows, int cols, int pdl, insg_stream_t stream);

/* Writes the two device scalars the engine's kernels read (token id, position); either pointer may be NULL. */
INSG_API int insg_set_scalars(int *device_token, int token, int *device_position, int position, insg_stream_t stream);

/* out[rows][cols] fp32 = full dequantisation, bit-exact with the reference's
 * decode of a code and a scale byte (src/mxfp4.cu:50-53: lut[code] * (scale<<23)).
 * Exists so dequantisation can be checked bit for bit. */
INSG_API int insg_mxfp4_dequant_mlx(const uint32_t *weight, const uint8_t *scales, float *out, int rows, int cols,
                                    insg_stream_t stream);

/* y[rows] = W x with W as 17-byte blocks {E8M0 scale, 16 bytes}: byte i of a block holds element i in its low
 * nibble and element 16+i in its high nibble; block b of row r sits at byte (r * cols/32 + b) * 17.  A scale byte
 * of 255 decodes to NaN in this layout's helper.  Replaces mxfp4_gemv (include/insignia_layout.cuh:11-15,45,
 * src/mxfp4.cu:5-35), which the token loop never calls (checkpoints are MLX layout) but the reference's
 * kernel test does (src/test_mxfp4.cu:31). */
INSG_API int insg_mxfp4_gemv_blocks(const void *blocks, const float *x, float *y, int rows, int cols, insg_stream_t stream);

/* The reference's int8 experiment (its microbenchmark only, src/bench_mxfp4_mlx.cu:9-11): quantise x per group
 * of 32 to int8 with scale max|x|/127 (1 for an all-zero group), then y = W x with integer dot products of the
 * doubled E2M1 codes.  Replace quantize_q8_groups and mxfp4_gemv_dp4a (include/insignia_layout.cuh:49-50,
 * src/mxfp4.cu:83-127); warps_per_row is dropped.  Results differ from the fp32 GEMV by the int8 rounding of x. */
INSG_API int insg_quantize_q8_groups(const float *x, int8_t *qx, float *qscale, int cols, insg_stream_t stream);
INSG_API int insg_mxfp4_gemv_dp4a(const uint32_t *weight, const uint8_t *scales, const int8_t *qx, const float *qscale,
                                  float *y, int rows, int cols, insg_stream_t stream);

/* Tile-interleaved weight layout used by the fused GEMV kernels.  Same
 * information and the same byte count as the MLX layout (17 bytes per 32
 * weights): rows are grouped in tiles of 16, K in blocks of 128, and each
 * (tile, block) record is 1024 bytes of nibbles + 64 scale bytes laid out in the
 * order the tensor-core fragments consume them.  rows % 16 == 0, cols % 128 == 0.
 * No reference counterpart: the reference streams the MLX layout directly
 * (src/decode.cu:13). */
INSG_API size_t insg_mxfp4_packed_bytes(int rows, int cols);
INSG_API int insg_mxfp4_repack(const uint32_t *weight, const uint8_t *scales, void *packed, int rows, int cols,
                               insg_stream_t stream);

/* Second packed layout, for the tcgen05 kernel: rows in tiles of 128 (padded with zero weights), K in blocks of
 * 128, one 8704-byte record per (tile, block) = the shared-memory image tcgen05.mma kind::mxf4 reads (canonical
 * K-major 4-bit operand, no swizzle) followed by the 512-byte scale block tcgen05.cp expects.  cols % 128 == 0.
 * Same 17 bytes per 32 weights.  No reference counterpart. */
INSG_API size_t insg_mxfp4_packed_umma_bytes(int rows, int cols);
INSG_API int insg_mxfp4_repack_umma(const uint32_t *weight, const uint8_t *scales, void *packed, int rows, int cols,
                                    insg_stream_t stream);

/* y[m][rows] = W x[m] for m < M (1 <= M <= 4096), W in the packed layout; x is
 * fp32 [M][cols], y fp32 [M][rows].  Plain (no fused prologue/epilogue) form of
 * the kernel the engine runs; replaces Qwen35Decode::linear (src/decode.cu:13).
 * Tokens go through in passes of four (the weights are streamed once per pass). */
INSG_API int insg_mxfp4_gemv_packed(const void *packed, const float *x, float *y, int rows, int cols, int M,
                                    insg_stream_t stream);

/* Y[m][rows] = W x[m] for M tokens on the tcgen05 tensor cores (kind::mxf4, weights in the insg_mxfp4_repack_umma
 * layout, sixteen tokens per instruction, fp32-exact activations as eight balanced base-9 digit columns each); x fp32
 * [M][cols], y fp32
 * [M][rows].  The M >= 8 counterpart of insg_mxfp4_gemv_packed (src/decode.cu:13 applied to M tokens; the reference
 * has no batched form).  scratch: insg_umma_gemm_scratch_bytes(cols, M) of device memory. */
INSG_API size_t insg_umma_gemm_scratch_bytes(int cols, int tokens);
INSG_API int insg_mxfp4_gemm_umma(const void *packed_umma, const float *x, float *y, int rows, int cols, int M, void *scratch,
                                  size_t scratch_bytes, insg_stream_t stream);

/* ---------------------------------------------------------- fused GEMV op */

/* What is done to the activation vector before the contraction. */
enum {
    INSG_PRO_PLAIN = 0,        /* x = in                                                        */
    INSG_PRO_RMSNORM = 1,      /* x = in * rsqrt(mean(in^2)+1e-6) * w_bf16          (src/qwen_kernels.cu:5) */
    INSG_PRO_GATED_RMSNORM = 2,/* per 128-wide head: rmsnorm(in) * w_bf16[128] * silu(aux)  (src/qwen_kernels.cu:5, G) */
    INSG_PRO_SIGMOID_GATE = 3, /* x = in * sigmoid(aux[i])                           (src/qwen_kernels.cu:11) */
    INSG_PRO_SIGMOID_GATE_HEAD0 = 4, /* x = in * sigmoid(aux[(i>>8)*512+256]) : gate element 0 of the head
                                  broadcast over its 256 lanes; aux is the interleaved q_proj output
                                  (src/qwen_kernels.cu:31,36) */
    INSG_PRO_SIGMOID_GATE_QPROJ = 5, /* x = in * sigmoid(aux[(i>>8)*512+256+(i&255)]) : element-wise gate read
                                  from the interleaved q_proj output */
    INSG_PRO_PREPARED = 6      /* `in` is not fp32 but the fp16 image [2][cols] an earlier launch left through
                                  insg_gemv_segment.prep (already multiplied by that launch's prep_w).  With prep_rms
                                  the product is also scaled by rsqrt(sum(prep_partials[0..295]) / cols + 1e-6), which
                                  makes the pair the RMSNorm of INSG_PRO_RMSNORM without this launch reducing anything.
                                  The image has a fixed scale; when the producer's sums say it is not trustworthy (root
                                  mean square outside [1e-3, 1e5], or a value that did not fit) and `aux` is given, the
                                  launch reads the fp32 vector `aux` instead (RMSNorm with norm_w if that is set, else
                                  as is).  One token per launch. */
};

/* What is done with each output row. */
enum {
    INSG_EPI_STORE = 0,     /* out[row] = y                                                     */
    INSG_EPI_RESIDUAL = 1,  /* out[row] += y                                   (src/ops.cu:8)   */
    INSG_EPI_CONV_SILU = 2, /* causal conv4 + SiLU on channel `row` with history  (src/qwen_kernels.cu:7) */
    INSG_EPI_BETA = 3,      /* out[row] = sigmoid(y)                           (src/qwen_kernels.cu:9) */
    INSG_EPI_DECAY = 4,     /* out[row] = -exp(A_log[row]) * softplus(y + dt_bias[row]) (src/qwen_kernels.cu:9) */
    INSG_EPI_SWIGLU = 5,    /* two matrices: out[row] = silu(y_gate) * y_up    (src/ops.cu:7)   */
    INSG_EPI_LOGITS = 6     /* out[row] = y and a running arg-max of the rows  (src/qwen_kernels.cu:20) */
};

/* One matrix (or gate/up pair) inside a fused launch. */
typedef struct insg_gemv_segment {
    const void *packed;      /* packed weights                                         */
    const void *packed2;     /* second matrix for INSG_EPI_SWIGLU, else NULL           */
    float *out;              /* fp32 [rows]                                            */
    int rows;                /* multiple of 16                                         */
    int epilogue;            /* INSG_EPI_*                                             */
    float *conv_state;       /* CONV_SILU: fp32 [rows][3] history, updated             */
    const uint16_t *conv_w;  /* CONV_SILU: bf16 [rows][4]                              */
    const float *A_log;      /* DECAY: fp32 [rows]                                     */
    const uint16_t *dt_bias; /* DECAY: bf16 [rows]                                     */
    /* RESIDUAL / SWIGLU, optional: besides out[], leave the vector ready for a later INSG_PRO_PREPARED launch.
     * prep: fp16 [2][rows] = the two half-precision pieces of out[row] * prep_w[row] / 16 (values beyond
     * +-1e6 saturate).  prep_w: bf16 [rows] multiplier, the weight of the RMSNorm that follows, or NULL for 1.
     * prep_partials (single-segment launches): fp32 [296], entry c = this launch's CTA c's sum of out[row]^2 over
     * its rows (infinite if a value did not fit the image), unused entries zero. */
    void *prep;
    const uint16_t *prep_w;
    float *prep_partials;
    /* CONV_SILU with several tokens.  0: the tokens are consecutive positions of ONE sequence, the history is carried
     * through them in order.  Otherwise the tokens belong to independent sequences (a decode batch) and token m's
     * history is conv_state + m * conv_token_stride floats. */
    long long conv_token_stride;
} insg_gemv_segment;

/* A fused launch: prologue on the shared input vector, up to 4 matrices that
 * all multiply it, an epilogue per matrix.  cols % 128 == 0, cols <= 12288. */
typedef struct insg_gemv_op {
    const float *in;          /* fp32 [cols] (INSG_PRO_PREPARED: the fp16 image [2][cols]) */
    const float *aux;         /* prologue operand (gate / z), or NULL                  */
    const uint16_t *norm_w;   /* bf16 norm weight for the RMSNorm prologues, or NULL   */
    float *x_out;             /* optional: the prologue's result fp32 [cols], or NULL  */
    int cols;
    int prologue;             /* INSG_PRO_*                                            */
    int n_segments;           /* 1..4                                                  */
    insg_gemv_segment seg[4];
    /* INSG_EPI_LOGITS only: partial arg-max scratch (>= insg_gemv_argmax_scratch_bytes(), its
     * first 64 bytes zero before the first call and left zero by every call).  The winning row
     * is written to *token_out and, when non-NULL, to *token_feedback and to
     * token_log[*position_inout] (only while 0 <= *position_inout < token_log_capacity); then
     * *position_inout is incremented (when non-NULL). */
    void *argmax_scratch;
    int *token_out;
    int *token_feedback;
    int *token_log;
    int token_log_capacity;   /* entries of token_log; required (> 0) when token_log is given */
    int *position_inout;
    int layout;               /* weight layout of every segment: 0 = insg_mxfp4_repack records, 1 = insg_mxfp4_repack_umma   */
    int *error_flag;          /* set to 1 if a bounded wait inside the kernel ran out (device int), or NULL                 */
    int pdl;                  /* 1: launch with programmatic dependent launch          */
    const float *prep_partials; /* INSG_PRO_PREPARED: the producer's prep_partials [296], or NULL                        */
    int prep_rms;               /* INSG_PRO_PREPARED: 1 = scale by the RMS factor computed from prep_partials            */
    int tokens;                 /* 0 or 1: one token.  More: consecutive tokens of one sequence in one call (the weights are
                                   streamed once per pass): in, aux and x_out are [tokens][cols], every out is
                                   [tokens][rows]; the convolution history is advanced token by token.  layout 0: 2 or 4
                                   tokens (one launch of the mma.sync kernel); layout 1: any count up to 4096, sixteen tokens
                                   per tcgen05 instruction (needs umma_scratch).  Not with INSG_PRO_PREPARED, prepared
                                   outputs or INSG_EPI_LOGITS. */
    void *umma_scratch;         /* layout 1 with tokens > 1: device scratch of insg_umma_gemm_scratch_bytes(cols, tokens) for
                                   the activations' digit image, rewritten by every call                                      */
    size_t umma_scratch_bytes;
} insg_gemv_op;

INSG_API size_t insg_gemv_argmax_scratch_bytes(void);
INSG_API int insg_gemv_fused(const insg_gemv_op *op /* host */, insg_stream_t stream);

/* ------------------------------------------------- persistent token program */
/* A program is a recorded sequence of the fused operations above (GEMV, DeltaNet step, attention step, embedding
 * lookup) that ONE cooperative launch of one CTA per SM executes back to back, with a grid-wide barrier between
 * operations instead of a kernel boundary: the 162 dependent launches of a token step become one.  The GEMV phases
 * split and sum exactly as insg_gemv_fused does (bit-identical results).  While the SMs sit in barriers and in the
 * small recurrent phases, every warp keeps prefetching the weight records it will need next into L2.
 * No reference counterpart: the reference launches every kernel separately (src/decode.cu:14-23).
 *
 * insg_program_create / _finalize allocate (host memory, then two small device buffers); _run allocates nothing and
 * does not synchronise.  A program is bound to the device that was current at create.  The operations' pointers are
 * baked in, as in a captured graph.  One run at a time per program (runs share the barrier state). */
struct insg_attn_op;
typedef struct insg_program insg_program;
INSG_API insg_program *insg_program_create(void);
INSG_API void insg_program_destroy(insg_program *prog);
/* Append one operation.  The op structs have the meaning they have for insg_gemv_fused / insg_attention_step
 * (pdl, layout and error_flag are ignored; one token per GEMV). */
INSG_API int insg_program_add_gemv(insg_program *prog, const insg_gemv_op *op /* host */);
INSG_API int insg_program_add_deltanet(insg_program *prog, float *state, const float *q16, const float *k16, const float *v32,
                                       const float *g32, const float *beta32, float *out32);
INSG_API int insg_program_add_attention(insg_program *prog, const struct insg_attn_op *op /* host */);
INSG_API int insg_program_add_embed(insg_program *prog, const uint32_t *weight, const uint8_t *scales, float *out,
                                    const int *device_row, int rows, int cols);
/* Uploads the program; no operation can be added afterwards. */
INSG_API int insg_program_finalize(insg_program *prog);
/* Options: "prefetch_records" = how many 1088-byte weight records each warp keeps prefetched into L2 ahead of its own
 * consumption (0 = off, default 24); "timeout_ns" = how long a barrier waits before it gives up (default 2 s). */
INSG_API int insg_program_set_option(insg_program *prog, const char *key /* host */, long long value);
/* Runs the program n_tokens times in one launch (the arg-max feedback of a LOGITS epilogue links consecutive tokens).
 * token / position >= 0 are first stored to *device_token / *device_position by the kernel itself (pass -1 to leave
 * them), followed by one device-wide barrier, so every CTA of the first operation reads the new values.  If a barrier wait runs out, *error_flag (device int, may be NULL) is set to 1, every CTA leaves the kernel and
 * the results are undefined; call insg_program_recover before the next run. */
INSG_API int insg_program_run(insg_program *prog, int n_tokens, int token, int position, int *device_token,
                              int *device_position, int *error_flag, insg_stream_t stream);
INSG_API int insg_program_recover(insg_program *prog, insg_stream_t stream);
/* Failure-detection self-test: runs the program once with every barrier waiting for one CTA more than exists and the
 * given (short, <= 100 ms) timeout, so the first wait runs out: *error_flag becomes 1 and the kernel returns.  Needs a
 * program of at least two operations.  Call insg_program_recover afterwards. */
INSG_API int insg_program_selftest_barrier_timeout(insg_program *prog, unsigned long long timeout_ns, int *error_flag,
                                                   insg_stream_t stream);
INSG_API int insg_program_phase_count(const insg_program *prog);
INSG_API uint64_t insg_program_weight_bytes(const insg_program *prog);

/* ------------------------------------------------------------ DeltaNet */

/* One gated-delta-rule step for 32 value heads (16 q/k heads, head>>1), dk=dv=128.
 * state fp32 [32][128(k)][128(v)] updated in place; q16,k16 fp32 [16][128];
 * v32 fp32 [32][128]; g32, beta32 fp32 [32]; out32 fp32 [32][128].
 * Replaces deltanet_decode (include/insignia_deltanet.cuh:5, src/deltanet.cu:4-14).
 * pdl (all DeltaNet entry points): 1 launches with programmatic stream serialization; the kernel then reads its STATE
 * before the dependency wait and everything else after it.  Precondition: the launch right before it in the stream does
 * not write the state (the engine puts a GEMV there); two pdl = 1 steps on the same state back to back would race, so
 * pass pdl = 0 when nothing separates them. */
INSG_API int insg_deltanet_decode(float *state, const float *q16, const float *k16, const float *v32,
                                  const float *g32, const float *beta32, float *out32, int pdl,
                                  insg_stream_t stream);
/* The same step for `tokens` (1..1024) consecutive positions of the sequence in one launch: the state is read once,
 * kept on chip from step to step and written once (two or more tokens run a kernel that prepares the inputs of 32
 * steps at a time; bit-identical results).  q16/k16/v32 of step m are at + m * qkv_stride floats, g32/beta32 at
 * + m * 32, out32 at + m * 4096.  Same arithmetic as `tokens` calls of insg_deltanet_decode.  No reference counterpart. */
INSG_API int insg_deltanet_decode_tokens(float *state, const float *q16, const float *k16, const float *v32,
                                         const float *g32, const float *beta32, float *out32, int tokens, int qkv_stride,
                                         int pdl, insg_stream_t stream);

/* One step for `sequences` (1..64) independent sequences in one launch (a decode batch): sequence s has its state at
 * state + s * state_stride floats, q16/k16/v32 at + s * qkv_stride, g32/beta32 at + s * 32, out32 at + s * 4096.  Same
 * arithmetic as `sequences` calls of insg_deltanet_decode.  No reference counterpart (it is strictly batch 1). */
INSG_API int insg_deltanet_decode_batch(float *state, long long state_stride, const float *q16, const float *k16, const float *v32,
                                        const float *g32, const float *beta32, float *out32, int sequences, int qkv_stride, int pdl,
                                        insg_stream_t stream);

/* Two consecutive steps for a speculative verify pass: reads `state`, writes the state after the first step to
 * state_first (may be `state` itself: in place) and the state after the second step to state_second (a different
 * buffer), so the caller continues from either.  Inputs of step m at + m * qkv_stride / + m * 32, outputs at
 * + m * 4096, as insg_deltanet_decode_tokens.  No reference counterpart (it has no verify step, src/decode.cu:24-68). */
INSG_API int insg_deltanet_decode_verify(const float *state, float *state_first, float *state_second, const float *q16,
                                         const float *k16, const float *v32, const float *g32, const float *beta32, float *out32,
                                         int qkv_stride, int pdl, insg_stream_t stream);
/* Convolution history [channels][3] after a rejected second token: from the history after two tokens (`state`, in
 * place) and the history before them (`snapshot`).  No reference counterpart. */
INSG_API int insg_conv_rollback(float *state, const float *snapshot, long long channels, insg_stream_t stream);

/* ------------------------------------------------------------ attention */

/* KV cache element type. */
enum { INSG_KV_F32 = 0, INSG_KV_BF16 = 1 };

/* Bytes of scratch insg_gqa_decode needs for `tokens` cached tokens. */
INSG_API size_t insg_gqa_scratch_bytes(int tokens);

/* Split-K flash-decode for 16 query heads over 4 kv heads, head_dim 256, scale
 * 1/16: out[16][256] = softmax(q K^T / 16) V over `tokens` cache rows; cache
 * layout [token][4][256] of fp32 or bf16.  q fp32 [16][256] already normalised
 * and rotated.  `scratch` holds the per-split partials (see
 * insg_gqa_scratch_bytes); its first 64 bytes must be zero before the first call
 * and are left zero by every call.  Replaces gqa_decode
 * (include/insignia_attention.cuh:4, src/attention.cu:4-5), without its ~12K-token
 * shared-memory limit. */
INSG_API int insg_gqa_decode(const float *q, const void *k_cache, const void *v_cache, float *out, int tokens,
                             int kv_dtype, void *scratch, size_t scratch_bytes, insg_stream_t stream);

/* The same attention as insg_gqa_decode for callers that must not allocate device memory and have
 * no scratch buffer to hand over: code running inside a stream capture or a real-time serving
 * loop where cudaMalloc is forbidden or would synchronise, and plug-in hosts whose allocator the
 * library may not touch.  The split partials go to a fixed array inside the library image
 * (about 600 KB per GPU that loads the library, kept until the process exits), so there is no
 * scratch argument.  Limits and rules: at most 262144 cached tokens (INSG_E_LIMIT beyond);
 * every call on a device shares that one array, so two calls that overlap on the GPU (different
 * streams, or different threads) race -- serialise them; every call looks the array's address up
 * (cudaGetSymbolAddress, which allocates nothing), and the first such lookup on a device may load
 * the library's code there, so make the first call before any stream capture begins.  Calls no
 * cudaMalloc / cudaFree or other allocating routine.  No counterpart in the reference, whose
 * gqa_decode keeps its scores in dynamic shared memory (src/attention.cu:4-5). */
INSG_API int insg_gqa_decode_noalloc(const float *q, const void *k_cache, const void *v_cache, float *out, int tokens,
                                     int kv_dtype, insg_stream_t stream);

/* Fused attention step of the engine: per-head RMSNorm of q and k (bf16 weights,
 * eps 1e-6), partial RoPE on dims 0..63 at *position (theta 1e7, rotate-half,
 * skipped at position 0), store of k,v at cache row *position, then the same
 * split-K attention over *position+1 rows.  qraw is the interleaved q_proj
 * output [16][q256|gate256]; k_raw, v fp32 [4][256].  Replaces
 * split_q_gate + qwen35_qk_norm_rope_gate + store_kv + gqa_decode
 * (src/qwen_kernels.cu:15,31; src/ops.cu:9; src/attention.cu:4). */
typedef struct insg_attn_op {
    const float *qraw;
    const float *k_raw;
    const float *v;
    const uint16_t *q_norm_w; /* bf16 [256] */
    const uint16_t *k_norm_w; /* bf16 [256] */
    void *k_cache;
    void *v_cache;
    float *out;               /* fp32 [16][256]                                       */
    const int *position;      /* device int: cache row / rotary position of this token */
    int position_offset;      /* added to *position (the MTP head passes -1)          */
    int max_context;
    int kv_dtype;
    int fast_trig;            /* 1: __powf/__sinf/__cosf as the reference (src/ops.cu:9), 0: accurate */
    void *scratch;
    size_t scratch_bytes;
    int pdl;
    int *error_flag;          /* device int set to 1 if a bounded wait inside the kernel ran out (bf16 cache, long contexts:
                                 rows are staged by bulk copies with mbarrier completion), or NULL */
} insg_attn_op;
INSG_API int insg_attention_step(const insg_attn_op *op /* host */, insg_stream_t stream);
/* `tokens` consecutive tokens of one sequence in two launches (prompt processing): op describes token 0 (rotary position
 * and cache row *position + position_offset); token m takes qraw + m * 8192, k_raw + m * 1024, v + m * 1024, writes
 * out + m * 4096 and cache row + m, and attends the rows up to its own.  scratch: tokens * insg_gqa_scratch_bytes(.)
 * bytes whose first 64 bytes per token are zero before the first use (the kernel leaves them zero); q_scratch: device,
 * tokens * 4096 floats.  rows_hint: 0, or an upper bound of the rows the LAST token of the chunk attends (*position +
 * position_offset + tokens) when the host knows it: short contexts then start fewer CTAs; a hint that turns out too
 * small raises *op->error_flag.  op->pdl is ignored (plain stream order).  Same math per token as insg_attention_step. */
INSG_API int insg_attention_chunk(const insg_attn_op *op /* host */, int tokens, float *q_scratch, int rows_hint, insg_stream_t stream);
/* One step for `sequences` independent sequences at the same position in ONE launch (a decode batch): op describes
 * sequence 0; sequence s takes qraw + s * 8192, k_raw + s * 1024, v + s * 1024, writes out + s * 4096, and has its
 * caches at k_cache / v_cache + s * cache_stride_bytes.  scratch: sequences * insg_gqa_scratch_bytes(.) bytes, the first
 * 64 bytes per sequence zero before the first use.  Same math per sequence as insg_attention_step.  No reference
 * counterpart (it is strictly batch 1). */
INSG_API int insg_attention_batch(const insg_attn_op *op /* host */, int sequences, size_t cache_stride_bytes, insg_stream_t stream);

/* ------------------------------------------------ tensor-parallel exchange */
/* One-shot all-reduce (sum) of a short fp32 vector over NVLink peer memory, for the exchange step of a tensor-parallel
 * decode block.  No reference counterpart: the reference is single-GPU and has no collective call site.
 *
 * One process per GPU: every rank calls insg_comm_create (allocates its exchange buffer on the current device),
 * insg_comm_handle (64 bytes to all-gather among the ranks by any host channel), insg_comm_connect (maps the peers'
 * buffers).  insg_allreduce_oneshot then is ONE kernel per rank: peer stores of the rank's vector into every rank's
 * buffer as 8-byte {value, call number} words (the call number is the arrival flag of the value it travels with: no
 * fence, no separate flag), a bounded wait for the other ranks' words, the sum in rank order (bit-identical on every
 * rank), in place.  count: a multiple of 4, <= max_floats; data 16-byte aligned; every rank must call with the same count, in
 * the same order.  If a wait runs out (default 1 s, insg_comm_set_timeout) the rank's error flag is set
 * (insg_comm_error reads it, synchronising the stream) and the result is undefined; insg_comm_reset on every rank,
 * with no call in flight anywhere, makes the communicator usable again.  Capturable in a CUDA graph. */
typedef struct insg_comm insg_comm;
INSG_API insg_comm *insg_comm_create(int rank, int world /* 1..8 */, int max_floats);
INSG_API void insg_comm_destroy(insg_comm *c);
INSG_API int insg_comm_handle(insg_comm *c, void *handle64 /* host, 64 bytes out */);
INSG_API int insg_comm_connect(insg_comm *c, const void *handles /* host, world x 64 bytes, in rank order */);
INSG_API int insg_comm_set_timeout(insg_comm *c, unsigned long long timeout_ns);
INSG_API int insg_comm_error(insg_comm *c, int *host_out, insg_stream_t stream);
INSG_API int insg_comm_reset(insg_comm *c, insg_stream_t stream);
INSG_API int insg_allreduce_oneshot(insg_comm *c, float *data, int count, insg_stream_t stream);
/* All ranks in one process on ONE GPU (tests, development): comms[i] = rank i of `world`, created on the same device.
 * The ranks run as one cooperative launch (their CTAs wait on one another, so they may not be separate launches).
 * skip_rank >= 0 leaves that rank silent: the others' waits run out and set their error flags (failure-detection test). */
INSG_API int insg_comm_connect_local(insg_comm **comms /* host array */, int world);
INSG_API int insg_allreduce_oneshot_local(insg_comm **comms, float **data /* host array of device pointers */, int world, int count,
                                          int skip_rank, insg_stream_t stream);

/* ----------------------------------------------- stand-alone small kernels */
/* One entry point per reference free function, same argument meaning. */

/* src/qwen_kernels.cu:6 (rmsnorm_bf16 / gated_rmsnorm_bf16); gate may be NULL */
INSG_API int insg_rmsnorm_bf16(const float *x, const uint16_t *w, const float *gate, float *y, int rows, int cols,
                               int zero_centered, insg_stream_t stream);
/* src/ops.cu:6 (rmsnorm_zero_centered, fp32 weight, 1+w) */
INSG_API int insg_rmsnorm_zero_centered(const float *x, const float *w, float *y, int rows, int cols, float eps,
                                        insg_stream_t stream);
/* src/ops.cu:6 (rmsnorm_gated_silu: fp32 weight used as is, result times silu(gate)) */
INSG_API int insg_rmsnorm_gated_silu(const float *x, const float *w, const float *gate, float *y, int rows, int cols,
                                     float eps, insg_stream_t stream);
/* src/qwen_kernels.cu:8 */
INSG_API int insg_causal_conv4_silu(float *x, float *state, const uint16_t *w, int channels, insg_stream_t stream);
/* src/qwen_kernels.cu:10 */
INSG_API int insg_deltanet_parameters(float *a, float *b, const float *A_log, const uint16_t *dt_bias, int heads,
                                      insg_stream_t stream);
/* src/ops.cu:10 (the reference's unused `gate` argument is dropped) */
INSG_API int insg_qk_norm_rope(float *q, float *k, const uint16_t *q_w, const uint16_t *k_w, int position,
                               int fast_trig, insg_stream_t stream);
/* src/ops.cu:7,8 */
INSG_API int insg_silu_mul(const float *gate, const float *up, float *y, int n, insg_stream_t stream);
INSG_API int insg_residual_add(float *x, const float *delta, int n, insg_stream_t stream);
/* src/qwen_kernels.cu:11,16,32,37,27 */
INSG_API int insg_sigmoid_mul(float *x, const float *gate, int n, insg_stream_t stream);
INSG_API int insg_store_kv(const float *k, const float *v, void *k_cache, void *v_cache, int position,
                           int kv_dtype, insg_stream_t stream);
INSG_API int insg_split_q_gate(const float *interleaved, float *q, float *gate, insg_stream_t stream);
INSG_API int insg_expand_gate_heads(const float *head_gate, float *gate256, insg_stream_t stream);
INSG_API int insg_concat(const float *a, const float *b, float *out, int n, insg_stream_t stream);
/* src/qwen_kernels.cu:21 ; ties resolve to the lowest index */
INSG_API int insg_argmax_logits(const float *logits, int n, int *device_token, insg_stream_t stream);
/* The same arg-max for `count` rows of logits [count][stride] at once (one per sequence of a decode batch), and the end
 * of a batch step: tokens[i] = next[i], log[*position][i] = next[i] (while *position < capacity), then ++*position.
 * No reference counterpart (it decodes one sequence). */
INSG_API int insg_argmax_rows(const float *logits, long long stride, int n, int count, int *device_tokens, insg_stream_t stream);
INSG_API int insg_commit_tokens(const int *next, int *tokens, int *log, int capacity, int *position, int n, insg_stream_t stream);
/* src/qwen_kernels.cu:26 : y[rows] = W_bf16[rows][cols] x (mtp.fc) */
INSG_API int insg_bf16_gemv(const uint16_t *w, const float *x, float *y, int rows, int cols, int pdl,
                            insg_stream_t stream);

/* -------------------------------------------------------------- storage */
/* Handle-based face of ModelFile + TieredStorage (include/insignia_model.hpp:20-40, include/insignia_storage.hpp:15-31 of
 * the reference; behaviour src/storage.cu:5-11): a byte budget of device memory, acquire = make resident + pin,
 * release = unpin, least-recently-used eviction of unpinned tensors, and the reference's error texts ("tensor not
 * found: ...", "tensor exceeds device budget", "device budget exhausted by pinned tensors") through insg_last_error().
 * Additive: background prefetch, the tier a tensor is in (0 mapped file, 1 pinned host memory, 2 device), a pinned-host
 * cache tier, and reservations that charge other weight memory to the same budget.  host_backend = 1 replaces device
 * memory by host memory so that the residency logic can run on a machine without a GPU (testing only).
 * These allocate and may synchronise. */
typedef struct insg_storage insg_storage;
INSG_API insg_storage *insg_storage_open(const char *index_path /* host, UTF-8 */, uint64_t device_budget_bytes, int host_backend);
INSG_API void insg_storage_close(insg_storage *s);
INSG_API int insg_storage_acquire(insg_storage *s, const char *name, void **data /* out, may be NULL */, uint64_t *bytes /* out */);
INSG_API int insg_storage_release(insg_storage *s, const char *name);
INSG_API int insg_storage_prefetch(insg_storage *s, const char *name); /* 1 queued or already there, 0 absent from the file */
INSG_API int insg_storage_tier(insg_storage *s, const char *name);
INSG_API int insg_storage_reserve(insg_storage *s, uint64_t bytes);
INSG_API int insg_storage_unreserve(insg_storage *s, uint64_t bytes);
INSG_API int insg_storage_set_host_cache(insg_storage *s, uint64_t bytes);
INSG_API int insg_storage_clear(insg_storage *s);
INSG_API uint64_t insg_storage_device_bytes(insg_storage *s);
INSG_API uint64_t insg_storage_reserved_bytes(insg_storage *s);
/* out6 (host): uploads, uploaded bytes, evictions, hits, pinned-cache hits, prefetch requests */
INSG_API int insg_storage_stats(insg_storage *s, uint64_t *out6);

/* --------------------------------------------------------------- engine */
/* Handle-based face of the C++ host classes (ModelFile, Qwen35Weights,
 * DecodeWorkspace, Qwen35Decode: include/insignia_model.hpp, insignia_qwen35.hpp,
 * insignia_decode.hpp of the reference) for callers that cannot include C++
 * headers.  These DO allocate (at create) and DO synchronise where noted. */
typedef struct insg_engine insg_engine;

typedef struct insg_engine_options {
    uint64_t device_budget_bytes; /* TieredStorage budget (src/storage.cu:6); 0 = 16 GiB        */
    int max_context;              /* DecodeWorkspace ctx (src/decode.cu:10); 0 = 4096            */
    int kv_dtype;                 /* INSG_KV_F32 (the reference's cache) or INSG_KV_BF16        */
    int gate_elementwise;         /* 0: head-broadcast gate as the reference engine
                                     (src/qwen_kernels.cu:36); 1: element-wise gate as its NumPy
                                     tools (tools/reference_all_layers.py:13)                   */
    int accurate_trig;            /* 0: fast intrinsics for RoPE as the reference; 1: sincosf   */
    int use_graph;                /* 1: capture the token step in a CUDA graph                  */
    int use_pdl;                  /* 1: programmatic dependent launch between kernels           */
    int gemv_tcgen05;             /* 1: tcgen05 kind::mxf4 GEMV; 0: mma.sync register-streaming GEMV */
    int n_layers;                 /* 0 = 32                                                     */
    int vocab;                    /* 0 = 248320 (rows of lm_head used for logits)               */
    int device;                   /* CUDA device ordinal                                        */
    int persistent;               /* 0: one launch per fused operation (162 per token), replayed from a CUDA graph when
                                     use_graph is set; 1: a token step is ONE persistent cooperative launch (insg_program_*) */
    int prefill_mma_sync;         /* 0: insg_engine_forward_tokens sends 16 or more tokens through the tcgen05 kernel in passes
                                     of up to 256 (second copy of the weights in its tile layout); 1: always passes of four
                                     through the mma.sync kernel */
    int gemv_unprepared;          /* 0: a GEMV that writes the residual stream or the SwiGLU output leaves the next
                                     GEMV's input prepared (insg_gemv_segment.prep); 1: every GEMV converts its own */
} insg_engine_options;

INSG_API insg_engine *insg_engine_create(const char *index_path /* host, UTF-8 */, const insg_engine_options *opt);
INSG_API void insg_engine_destroy(insg_engine *e);
/* Qwen35Weights::embed into workspace.hidden (src/qwen35.cu:9, src/test_full_model.cu:6) */
INSG_API int insg_engine_embed(insg_engine *e, int token);
/* Qwen35Decode::layer (src/decode.cu:20) */
INSG_API int insg_engine_layer(insg_engine *e, int layer);
/* Qwen35Decode::forward_token (src/decode.cu:21): asynchronous */
INSG_API int insg_engine_forward_token(insg_engine *e, int token);
/* Qwen35Decode::logits_argmax (src/decode.cu:22): synchronises, returns the token id (>=0) */
/* Additive: insg_engine_forward_token for `count` consecutive tokens (host array), four tokens per pass over the
 * weights; same resulting state, logits and arg-max of the last token.  No reference counterpart (its prompt loop is
 * src/generate_ids.cu:4). */
INSG_API int insg_engine_forward_tokens(insg_engine *e, const int *tokens /* host */, int count);
INSG_API int insg_engine_logits_argmax(insg_engine *e);
/* Qwen35Decode::decode_token (src/decode.cu:23): synchronises, returns the token id (>=0) */
INSG_API int insg_engine_decode_token(insg_engine *e, int token);
/* Qwen35Decode::mtp_draft (src/decode.cu:24): synchronises, returns the draft token id */
INSG_API int insg_engine_mtp_draft(insg_engine *e, int token);
/* Greedy generation without a host round trip per token: feeds `first_token`, then each
 * arg-max back in, `count` times; writes the `count` produced ids to out_tokens (host).
 * Synchronises once at the end.  No reference counterpart (its loop is src/generate_ids.cu:4). */
INSG_API int insg_engine_generate(insg_engine *e, int first_token, int count, int *out_tokens /* host */);
/* Speculative greedy decode, draft-1 / verify, on top of Qwen35Decode::mtp_draft (src/decode.cu:24-68; the reference has
 * no verify step).  prime: the prompt (host array) token by token, every position's row left in the MTP cache; returns
 * the greedy next token (>= 0).  generate: `count` tokens into out_tokens (host); each step one MTP draft and one
 * two-token verify pass; a wrong draft is rolled back, so the ids equal plain greedy decode; *accepted (host, may be
 * NULL) = drafts that were right; forced_drafts (host, `count` ints, may be NULL) replaces the MTP head as the draft
 * source.  Synchronises every step. */
INSG_API int insg_engine_prime_speculative(insg_engine *e, const int *prompt /* host */, int count);
INSG_API int insg_engine_generate_speculative(insg_engine *e, int first_token, int count, int *out_tokens /* host */,
                                              int *accepted /* host */, const int *forced_drafts /* host */);
/* The fused-GEMV operations of one token step alone, run `replays` (1..64) times between two CUDA events (one
 * CUDA graph of launches with dependent-launch overlap per replay, or with `persistent` one persistent launch):
 * *ms_per_token = time of one replay, *bytes = the algorithmic weight bytes of those operations, *launches = their
 * count.  Needs one forwarded token first.  The sequence state is meaningless afterwards (call insg_engine_reset).
 * Synchronises.  No reference counterpart. */
INSG_API int insg_engine_profile_gemv_chain(insg_engine *e, int replays, float *ms_per_token, uint64_t *bytes, int *launches);
/* Sets an option of the engine's persistent token program (see insg_program_set_option), now and for programs it builds
 * later: "prefetch_records" = 1088-byte weight records each warp keeps requested into L2 ahead of its own consumption
 * (0 = off). */
INSG_API int insg_engine_set_program_option(insg_engine *e, const char *key /* host */, long long value);
/* Failure-detection self-test of the persistent token kernel: one run whose first grid barrier can never be met, with a
 * 2 ms wait limit.  Returns 1 when the kernel gave up, raised its error status and the engine recovered; 0 when the
 * status was not raised; negative on error.  Synchronises; call insg_engine_reset afterwards. */
INSG_API int insg_engine_selftest_barrier_timeout(insg_engine *e);
INSG_API int insg_engine_position(insg_engine *e);
INSG_API int insg_engine_set_position(insg_engine *e, int position);
/* Re-zeroes the recurrent state and position (what constructing a fresh DecodeWorkspace does). */
INSG_API int insg_engine_reset(insg_engine *e);
/* Copies a workspace buffer to the host: "hidden", "logits", "delta_state", "conv_state", ... */
INSG_API int insg_engine_read(insg_engine *e, const char *field, float *out /* host */, uint64_t count);
/* Device pointer of a workspace buffer (for callers that post-process on the GPU). */
INSG_API void *insg_engine_buffer(insg_engine *e, const char *field);
/* Counterpart of insg_engine_read: copies `count` floats from host memory into a workspace buffer (the reference's
 * drivers write x.hidden directly, src/test_full_model.cu:6).  Synchronises. */
INSG_API int insg_engine_write(insg_engine *e, const char *field, const float *in /* host */, uint64_t count);
INSG_API insg_stream_t insg_engine_stream(insg_engine *e);
/* Kernel launches issued by the engine since creation (own kernels only). */
INSG_API uint64_t insg_engine_launch_count(insg_engine *e);
INSG_API uint64_t insg_engine_device_bytes(insg_engine *e);

/* ---------------------------------------------------------------- batch */
/* 1..8 independent sequences decoded in lock step on the weights of an engine (ONE copy of the weights; every weight
 * matrix is streamed once per step for all sequences): insignia::Qwen35BatchDecode of include/insignia_batch.hpp.  Each
 * sequence has its own recurrent state and KV cache (allocated at create, max_context <= 0 takes the engine's).  No
 * reference counterpart: the reference decodes one sequence (include/insignia_decode.hpp:5-24).  The batch must be
 * destroyed before its engine. */
typedef struct insg_batch insg_batch;
INSG_API insg_batch *insg_batch_create(insg_engine *e, int sequences, int max_context);
INSG_API void insg_batch_destroy(insg_batch *b);
/* one step, tokens[s] into sequence s (host array of `sequences` ints); no read-back */
INSG_API int insg_batch_forward_tokens(insg_batch *b, const int *tokens /* host */);
/* one step; next[s] (host) = greedy next token of sequence s; synchronises */
INSG_API int insg_batch_decode_tokens(insg_batch *b, const int *tokens /* host */, int *next /* host */);
/* count steps with the arg-max fed back on the device; out[step * sequences + s] (host); synchronises once */
INSG_API int insg_batch_generate(insg_batch *b, const int *first_tokens /* host */, int count, int *out /* host */);
INSG_API int insg_batch_reset(insg_batch *b);
INSG_API int insg_batch_position(insg_batch *b);
/* "hidden" (count 4096) or "delta_state" (first count floats) of one sequence to the host */
INSG_API int insg_batch_read(insg_batch *b, const char *field, int sequence, float *out /* host */, uint64_t count);
INSG_API uint64_t insg_batch_launch_count(insg_batch *b);
INSG_API insg_stream_t insg_batch_stream(insg_batch *b);

#ifdef __cplusplus
}
#endif
#endif /* INSIGNIA_B200_H */
