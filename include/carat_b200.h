/* C ABI of libcarat_b200: the speculative-decoding step of the Carat Gemma-4 runtime, written for
 * NVIDIA B200 (sm_100a).
 *
 * Conventions
 *  - Every function returns 0 on success and a negative code on failure; the message is available
 *    from carat_b200_last_error() on the calling thread. Invalid arguments are rejected before any
 *    launch, so a failed call leaves device state untouched.
 *  - Pointers named device_* (and all tensor arguments) are device memory on the current device.
 *    `stream` is a cudaStream_t passed as void*; NULL is the legacy default stream.
 *  - BF16 tensors are row-major unless stated; FP8 means e4m3 (finite, saturating, max 448).
 *  - Citations name the reference interface each entry point stands in for
 *    (paths inside the Gradiated/carat tree).
 */
#ifndef CARAT_B200_H
#define CARAT_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define CARAT_B200_API __attribute__((visibility("default")))
#else
#define CARAT_B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Library ------------------------------------------------------------------------------------ */

/* Thread-local text of the most recent failure. */
CARAT_B200_API const char *carat_b200_last_error(void);

/* ABI version of this header (bumped on incompatible changes). */
CARAT_B200_API int carat_b200_abi_version(void);

/* Kernels that wait on hardware barriers give up after a bounded time and record a code in a
 * per-device word instead of hanging. Synchronises the device, returns the code in *code
 * (0 = healthy) and clears it. */
CARAT_B200_API int carat_b200_device_error(int *code);

/* Runs the bounded-wait error path once, harmlessly: one CTA waits about a millisecond on a
 * barrier that nothing arrives on, gives up, records code 90 in the error word and ends normally.
 * device_report receives three ints: 1 if the wait gave up, 1 if a second wait in the same CTA
 * then returned at once (the CTA-wide give-up flag), and the cycles that second wait took.
 * carat_b200_device_error() afterwards returns 90 once and 0 from then on. No counterpart in the
 * reference (its kernels have no device-side waits to bound). */
CARAT_B200_API int carat_b200_selftest_bounded_wait(int *device_report, void *stream);

/* FP8 linear ---------------------------------------------------------------------------------- */

/* output[rows, output_width] = bf16((input_scale * weight_scale) *
 *                                   input_e4m3[rows, input_width] . weight_e4m3[output_width, input_width]^T)
 * with fp32 accumulation. rows <= 256, input_width a multiple of 16, operands 16-byte aligned.
 * `workspace` holds split-K partial sums and must be at least
 * carat_b200_fp8_linear_workspace_bytes() bytes (may be NULL when that is 0).
 * Replaces carat::Fp8Linear::run with Fp8Scaling::tensor (include/carat/linear.h:32-41,
 * cuda/linear.cu:645-803). */
CARAT_B200_API int carat_b200_fp8_linear(const void *fp8_input, const float *device_input_scale,
                          const void *fp8_weight, const float *device_weight_scale,
                          void *bf16_output, int rows, int input_width, int output_width,
                          void *workspace, size_t workspace_bytes, void *stream);

CARAT_B200_API size_t carat_b200_fp8_linear_workspace_bytes(int rows, int input_width, int output_width);

/* The same linear for callers that cannot allocate device memory where they need it (a serving
 * loop whose allocator is frozen once the model is loaded, a plugin with a fixed memory budget
 * its host framework will not let it grow): the split-K partial sums live in an 8 MiB array built
 * into the library image, so no workspace is passed and the call makes no cudaMalloc / cudaFree
 * or other allocating call. This entry point has no counterpart in the reference.
 *  - Shapes whose split-K scratch (carat_b200_fp8_linear_workspace_bytes) exceeds
 *    CARAT_B200_STATIC_SCRATCH_BYTES are rejected with an error; use carat_b200_fp8_linear for
 *    those.
 *  - The first call on each device looks the array's device address up, and the first call of
 *    each shape class (row bucket 32 / 64 / 128 / 192 / 256, with or without split-K) configures its
 *    kernel; under lazy module loading the very first call also makes the driver load the module
 *    that holds the 8 MiB. Make those first calls during set-up.
 *  - All calls on a device share the one array: calls that overlap on the GPU (different streams,
 *    no dependency) race on it. Nothing in it has to be zero between calls; every launch
 *    overwrites the part it reads. Every GPU that loads the library holds the array until exit.
 *  - A bounded wait that runs out inside this entry point records its code in a word that lives
 *    in the library image too; carat_b200_device_error() reports and clears it like the codes of
 *    every other entry point. */
#define CARAT_B200_STATIC_SCRATCH_BYTES (8u * 1024u * 1024u)
CARAT_B200_API int carat_b200_fp8_linear_static(const void *fp8_input,
                                                const float *device_input_scale,
                                                const void *fp8_weight,
                                                const float *device_weight_scale,
                                                void *bf16_output, int rows, int input_width,
                                                int output_width, void *stream);

/* The gate_up projection with the reference's GeGLU (gelu_tanh_gate_bf16, cuda/ops.cu:228-284;
 * called between the two MLP linears in cuda/layer_runner.cu:318-347) in the linear's epilogue:
 * fp8_weight is [2 * gated_width, input_width] e4m3, gate rows first, and
 *   bf16_activated[row, j] = bf16(gelu_tanh(g) * u),  g = bf16(x_scale * w_scale * acc_gate[row, j]),
 * u likewise from row gated_width + j: what carat_b200_fp8_linear followed by the GeGLU row
 * operation gives. *device_amax_bits receives the float bits of the largest |activated|. When
 * fp8_output is not NULL the same launch also quantises the rows for the down projection:
 * *device_output_scale = max / 448 (1 when 0), fp8_output[rows, gated_width] = e4m3(x / scale).
 * gated_width must be a multiple of 64. One launch of at most one CTA per SM (its phases meet at
 * grid-wide barriers with bounded waits). workspace: carat_b200_fp8_linear_geglu_workspace_bytes() bytes. */
CARAT_B200_API size_t carat_b200_fp8_linear_geglu_workspace_bytes(int rows, int input_width,
                                                                  int gated_width);
CARAT_B200_API int carat_b200_fp8_linear_geglu(const void *fp8_input,
                                               const float *device_input_scale,
                                               const void *fp8_weight,
                                               const float *device_weight_scale,
                                               void *bf16_activated,
                                               unsigned int *device_amax_bits, void *fp8_output,
                                               float *device_output_scale, int rows,
                                               int input_width, int gated_width, void *workspace,
                                               size_t workspace_bytes, void *stream);

/* Fused LM head: device_tokens[row] = argmax_n bf16(scale * input[row] . weight[n]), ties to the
 * lowest n, without writing the logits. `device_keys` is rows * 8 bytes of scratch.
 * Replaces run_decode_lm_head + argmax_bf16_rows (cuda/batch_model_runner.cu:840-853,
 * cuda/ops.cu:935-981, 1566-1579). */
CARAT_B200_API int carat_b200_fp8_linear_argmax(const void *fp8_input, const float *device_input_scale,
                                 const void *fp8_weight, const float *device_weight_scale,
                                 int *device_tokens, void *device_keys, int rows, int input_width,
                                 int output_width, void *stream);

/* Same contract as carat_b200_fp8_linear computed one output per thread without tensor cores.
 * A device-side cross-check for tests at sizes a CPU cannot finish; no step path calls it. */
CARAT_B200_API int carat_b200_fp8_linear_check(const void *fp8_input, const float *device_input_scale,
                                const void *fp8_weight, const float *device_weight_scale,
                                void *bf16_output, int rows, int input_width, int output_width,
                                void *stream);

/* BF16 linear ----------------------------------------------------------------------------------- */

/* output[rows, output_width] = bf16(input_bf16[rows, input_width] . weight_bf16[output_width,
 * input_width]^T) with fp32 accumulation: the weight-streaming kernel of carat_b200_fp8_linear
 * with 16-bit operands (tcgen05 kind::f16) and no scales. rows <= 256, input_width a multiple of
 * 8, operands 16-byte aligned; callers with more rows (prefill chunks) call it per 256 rows.
 * `workspace` as for carat_b200_fp8_linear, sized by carat_b200_bf16_linear_workspace_bytes().
 * Replaces carat::Bf16Linear::run (include/carat/linear.h:13-26, cuda/linear.cu:534-643: cuBLAS),
 * the linear of the drafter's default precision (cuda/assistant_runner.cu:147-160) and of BF16
 * prefill (cuda/layer_runner.cu:611-728). */
CARAT_B200_API int carat_b200_bf16_linear(const void *bf16_input, const void *bf16_weight,
                                          void *bf16_output, int rows, int input_width,
                                          int output_width, void *workspace,
                                          size_t workspace_bytes, void *stream);

CARAT_B200_API size_t carat_b200_bf16_linear_workspace_bytes(int rows, int input_width,
                                                             int output_width);

/* Fused BF16 LM head: device_tokens[row] = argmax_n bf16(input[row] . weight[n]), ties to the
 * lowest n, logits never stored. Replaces Bf16Linear::run + argmax_bf16_rows as the drafter's
 * default LM head does them (cuda/assistant_runner.cu:313-318). */
CARAT_B200_API int carat_b200_bf16_linear_argmax(const void *bf16_input, const void *bf16_weight,
                                                 int *device_tokens, void *device_keys, int rows,
                                                 int input_width, int output_width, void *stream);

/* INT4 weight-only linear (W4A16) --------------------------------------------------------------- */

/* Quantises a bf16 [output_width, input_width] weight in K-local groups of `group_width` (128 or
 * 256) values: scale = bf16(max|w| / 7) (1.0 for an all-zero group), code = clamp(rint(w / scale),
 * -7, 7). packed_row_major: output_width * input_width / 2 bytes, even K in the low nibble;
 * bf16_scales: [input_width / group_width, output_width] (group-major).
 * Replaces quantize_bf16_int4_kernel (cuda/int4_bf16_linear.cu:95-136), same layouts. */
CARAT_B200_API int carat_b200_int4_quantize_weight(const void *bf16_weight, void *packed_row_major,
                                                   void *bf16_scales, int output_width,
                                                   int input_width, int group_width, void *stream);

/* One-time reordering of the packed codes into the order the linear kernel streams (same size).
 * Replaces the cutlass::reorder_tensor step of the reference's constructor
 * (cuda/int4_bf16_linear.cu:268-276). */
CARAT_B200_API int carat_b200_int4_reorder_weight(const void *packed_row_major, void *reordered,
                                                  int output_width, int input_width, void *stream);

/* output[rows, output_width] = bf16(input_bf16[rows, input_width] . W^T) with
 * W[n, k] = bf16(code[n, k] * scale[k / group_width, n]) and fp32 accumulation. rows <= 128,
 * output_width a multiple of 8, operands 16-byte aligned. `workspace` as for carat_b200_fp8_linear
 * (size from carat_b200_int4_linear_workspace_bytes).
 * Replaces carat::Int4Bf16Linear::run (include/carat/linear.h:70-90), whose constructor performs
 * the two calls above. */
CARAT_B200_API int carat_b200_int4_linear(const void *bf16_input, const void *reordered_weight,
                                          const void *bf16_scales, void *bf16_output, int rows,
                                          int input_width, int output_width, int group_width,
                                          void *workspace, size_t workspace_bytes, void *stream);

CARAT_B200_API size_t carat_b200_int4_linear_workspace_bytes(int rows, int input_width,
                                                             int output_width);

/* Same contract computed one output per thread from the row-major codes; a device-side
 * cross-check for tests, no step path calls it. */
CARAT_B200_API int carat_b200_int4_linear_check(const void *bf16_input, const void *packed_row_major,
                                                const void *bf16_scales, void *bf16_output, int rows,
                                                int input_width, int output_width, int group_width,
                                                void *stream);

/* Activation quantisation and fused row operators ----------------------------------------------- */

/* All of these quantise a [rows, width] bf16 tensor to e4m3 with one tensor-wide scale:
 * *device_scale = amax / 448 (1.0 when amax == 0), value = e4m3(x * (1 / scale)), saturating
 * (carat::quantize_bf16_to_fp8_e4m3 and its _from_row_amax / _from_amax_values forms,
 * include/carat/linear.h:93-110, cuda/linear.cu:76-296). rows <= 256, width a multiple of 8 and
 * at most 32768. `device_scratch` is one 32-bit word the call clears and uses for the running
 * maximum. Each call is one cooperative launch. */

/* Plain quantisation. */
CARAT_B200_API int carat_b200_quantize_bf16_to_fp8(const void *bf16_input, void *fp8_output, float *device_scale,
                                    void *device_scratch, int rows, int width, void *stream);

/* The maximum is already known (float bits in *device_amax_bits, e.g. from
 * carat_b200_fp8_linear_geglu): scale = max / 448 (1 when 0), e4m3(x / scale). One ordinary launch,
 * no grid barrier; the _from_row_amax form of the reference (include/carat/linear.h:97-99) with
 * the row maxima already reduced. `elements` a multiple of eight. */
CARAT_B200_API int carat_b200_quantize_bf16_to_fp8_from_amax(const void *bf16_input,
                                                             const unsigned int *device_amax_bits,
                                                             void *fp8_output, float *device_scale,
                                                             size_t elements, void *stream);

/* Same contract for a tensor of any size (weights at load time): three ordinary launches, the
 * reference's non-cooperative branch (cuda/linear.cu:117-153,261-271; used by
 * Fp8WeightArena::quantize, cuda/device_weights.cu:200-263). */
CARAT_B200_API int carat_b200_quantize_bf16_tensor_to_fp8(const void *bf16_input, void *fp8_output,
                                                          float *device_scale,
                                                          void *device_scratch, size_t elements,
                                                          void *stream);

/* normalized = bf16(rmsnorm(input) * weight) [stored to bf16_normalized when not NULL], then
 * quantised. Replaces rms_norm_bf16_with_row_amax + quantize_..._from_row_amax
 * (include/carat/cuda_ops.h:10-16, cuda/layer_runner.cu:241-262). */
CARAT_B200_API int carat_b200_rms_norm_quantize(const void *bf16_input, const void *bf16_weight,
                                 void *bf16_normalized, void *fp8_output, float *device_scale,
                                 void *device_scratch, int rows, int width, float epsilon,
                                 void *stream);

/* first = bf16(rmsnorm(input) * weight + residual) -> bf16_first; second = bf16(rmsnorm(first) *
 * next_weight) -> quantised. Replaces rms_norm_add_and_norm_bf16_with_row_amax + quantiser
 * (include/carat/cuda_ops.h:19-29, cuda/layer_runner.cu:306-330). */
CARAT_B200_API int carat_b200_rms_norm_add_and_norm_quantize(const void *bf16_input, const void *bf16_weight,
                                              const void *bf16_residual,
                                              const void *bf16_next_weight, void *bf16_first,
                                              void *fp8_output, float *device_scale,
                                              void *device_scratch, int rows, int width,
                                              float epsilon, void *stream);

/* activated = bf16(gelu_tanh(gate) * up) from rows packed [gate | up] (2 * width columns), then
 * quantised. Replaces gelu_tanh_gate_rows_bf16_with_block_amax + reduce_block_amax_to_rows +
 * quantiser (include/carat/cuda_ops.h:36-44, cuda/layer_runner.cu:331-347). */
CARAT_B200_API int carat_b200_gelu_gate_quantize(const void *bf16_packed_gate_up, void *fp8_output,
                                  float *device_scale, void *device_scratch, int rows, int width,
                                  void *stream);

/* output = bf16(bf16(rmsnorm(input) * weight + residual) * scalar) -> bf16_output; then
 * bf16(rmsnorm(output) * next_weight) [-> bf16_next when not NULL] -> quantised: the layer tail
 * (rms_norm_add_scale_bf16, include/carat/cuda_ops.h:30-32) fused with the norm that follows it. */
CARAT_B200_API int carat_b200_rms_norm_add_scale_then_norm_quantize(
    const void *bf16_input, const void *bf16_weight, const void *bf16_residual,
    const void *bf16_scalar, void *bf16_output, const void *bf16_next_weight, void *bf16_next,
    void *fp8_output, float *device_scale, void *device_scratch, int rows, int width,
    float epsilon, void *stream);

/* Attention-side operators ---------------------------------------------------------------------- */

/* bf16 cos/sin tables [positions, head_dim] (cuda/qkv.cu:44-64 rope_cache_kernel): sliding layers
 * theta^(-2i/D) for every pair; proportional (global) layers only for i < D/8. */
CARAT_B200_API int carat_b200_rope_tables(void *bf16_cosine, void *bf16_sine, int positions, int head_dim,
                           float theta, int proportional, void *stream);

/* Q: per-head rmsnorm * weight -> bf16 -> rotate-half RoPE -> bf16, stored
 * [requests, query_heads, depth, head_dim]. K likewise, V = rmsnorm without weight (from the K
 * slice when key_equals_value); both stored [requests, kv_heads, depth, head_dim].
 * packed rows are [Q | K | V] (V absent when key_equals_value). head_dim is 64, 256 or 512. Every
 * tensor pointer must be 16-byte aligned (head vectors move in 8- and 16-byte pieces).
 * Replaces Gemma4QkvPostprocessor::run_prefill_uniform (include/carat/qkv.h:40-47,
 * cuda/qkv.cu:387-475). */
CARAT_B200_API int carat_b200_qkv_postprocess(const void *bf16_packed, const void *bf16_query_norm,
                               const void *bf16_key_norm, const void *bf16_cosine,
                               const void *bf16_sine, void *bf16_queries, void *bf16_keys,
                               void *bf16_values, const int *device_positions, int requests,
                               int depth, int query_heads, int kv_heads, int head_dim,
                               int key_equals_value, int table_positions, float epsilon,
                               void *stream);

/* Verify attention of `depth` (<= 16) proposal rows per request over that request's cache plus the
 * proposals. caches: [requests, kv_heads, capacity, head_dim] (logical position p in row
 * p % capacity); queries [requests, query_heads, depth, head_dim]; output
 * [requests * depth, query_heads * head_dim].
 *  - window > 0: sliding ring. The proposals' K/V are passed on the side as
 *    [requests, kv_heads, depth, head_dim] and the ring is left untouched.
 *  - window = 0 with new_keys/new_values NULL: causal attention over a linear cache that already
 *    holds the proposals at rows position .. position + depth - 1.
 * scores is scratch of requests * query_heads * depth * score_stride bf16, score_stride a multiple
 * of 8 and >= 16 + the participating cache rows rounded up to 128 (cache rows = min(max_position,
 * capacity) for a ring, max_position + depth for a linear cache).
 * head_dim 256 / 512 with capacity % 128 == 0 runs on tensor cores (tcgen05 + TMA), head_dim 64 on
 * CUDA cores. Replaces GemmCausalPrefillAttention::run_uniform_batch / run_uniform_ring_batch
 * (include/carat/prefill_gemm_attention.h:24-47). */
CARAT_B200_API int carat_b200_verify_attention(const void *bf16_queries, const void *bf16_key_caches,
                                const void *bf16_value_caches, const void *bf16_new_keys,
                                const void *bf16_new_values, const int *device_positions,
                                void *bf16_output, void *bf16_scores, int score_stride,
                                int requests, int depth, int query_heads, int kv_heads,
                                int head_dim, int capacity, int window, int max_position,
                                void *stream);

/* Same contract on CUDA cores for every head_dim: the device-side cross-check of the tensor-core
 * kernels; no step path calls it for head_dim 256 / 512. */
CARAT_B200_API int carat_b200_verify_attention_check(
    const void *bf16_queries, const void *bf16_key_caches, const void *bf16_value_caches,
    const void *bf16_new_keys, const void *bf16_new_values, const int *device_positions,
    void *bf16_output, void *bf16_scores, int score_stride, int requests, int depth,
    int query_heads, int kv_heads, int head_dim, int capacity, int window, int max_position,
    void *stream);

/* Rollback primitives with the reference's signatures
 * (include/carat/cuda_ops.h:124-135, cuda/ops.cu:827-871,1485-1525). */
CARAT_B200_API int carat_b200_backup_kv_ring_spans(const void *const *device_key_sources,
                                    const void *const *device_value_sources, void *backup_keys,
                                    void *backup_values, const int *device_position_starts,
                                    int requests, int heads, int tokens, int head_dim,
                                    int source_capacity, void *stream);
CARAT_B200_API int carat_b200_restore_kv_ring_suffixes(const void *backup_keys, const void *backup_values,
                                        void *const *device_key_destinations,
                                        void *const *device_value_destinations,
                                        const int *device_position_starts,
                                        const int *device_accepted_tokens, int requests, int heads,
                                        int tokens, int head_dim, int destination_capacity,
                                        void *stream);

/* Row argmax over bf16 values, ties to the lowest index
 * (argmax_bf16_rows, include/carat/cuda_ops.h:149-151, cuda/ops.cu:935-981). */
CARAT_B200_API int carat_b200_argmax_bf16_rows(const void *bf16_values, int rows, int elements,
                                int *device_output, void *stream);

/* Greedy prefix-accept on the device (the host loop of cuda/batch_model_runner.cu:1735-1759):
 * accepted[r] = longest prefix with proposals[r][i] == (i == 0 ? target_first[r] :
 * predictions[r][i-1]), capped by caps[r] (NULL = depth); next[r] = accepted == 0 ?
 * target_first[r] : predictions[r][accepted-1]. */
CARAT_B200_API int carat_b200_greedy_prefix_accept(const int *device_proposals, const int *device_target_first,
                                    const int *device_predictions, const int *device_caps,
                                    int requests, int depth, int *device_accepted,
                                    int *device_next_tokens, void *stream);

/* Runner ------------------------------------------------------------------------------------------ */

/* One decoder layer's attention shape (carat::Gemma4LayerConfig, include/carat/gemma4_config.h:14-26). */
typedef struct carat_b200_layer_shape {
  int32_t global_attention; /* 0 = sliding window ring, 1 = global */
  int32_t query_heads;
  int32_t kv_heads;
  int32_t head_dim;         /* 64, 256 or 512 */
  float rope_theta;
  int32_t key_equals_value;
} carat_b200_layer_shape;

/* carat::Gemma4Config (include/carat/gemma4_config.h:28-43), the fields the path reads. */
typedef struct carat_b200_model_config {
  int32_t hidden_size;
  int32_t intermediate_size;
  int32_t vocabulary_size;
  int32_t sliding_window;
  float rms_norm_epsilon;
  int32_t layer_count;
  const carat_b200_layer_shape *layers;
} carat_b200_model_config;

/* Device pointers of one layer's segments, named as in the reference's weight plan
 * (src/weight_plan.cpp:37-82). Norm weights and the scalar are bf16 (DeviceWeightArena::at);
 * matrices are e4m3 row-major [out, in] with one fp32 scale (Fp8WeightArena::at / ::scale,
 * cuda/device_weights.cu:200-263). Every matrix pointer must be 16-byte aligned. */
typedef struct carat_b200_layer_weights {
  const void *input_norm;
  const void *q_norm;
  const void *k_norm;
  const void *qkv;
  const float *qkv_scale;
  const void *o;
  const float *o_scale;
  const void *post_attention_norm;
  const void *pre_mlp_norm;
  const void *gate_up;
  const float *gate_up_scale;
  const void *down;
  const float *down_scale;
  const void *post_mlp_norm;
  const void *scalar;
} carat_b200_layer_weights;

typedef struct carat_b200_model_weights {
  const void *token_embedding;            /* bf16 [vocabulary, hidden] */
  const void *token_embedding_fp8;        /* e4m3 copy used as the tied LM head */
  const float *token_embedding_scale;
  const void *final_norm;
  const carat_b200_layer_weights *layers; /* layer_count entries */
} carat_b200_model_weights;

/* Drafter shape. The reference hard-codes hidden 1024, intermediate 8192, 32 query heads and four
 * layers of which the last is global (cuda/assistant_runner.cu:22-27,166-170); here they are
 * parameters. Layer i attends the target's last layer of the kind layer_global[i] selects. */
typedef struct carat_b200_assistant_config {
  int32_t hidden_size;
  int32_t intermediate_size;
  int32_t query_heads;
  int32_t layer_count;
  const int32_t *layer_global; /* layer_count entries, 0 = sliding, 1 = global */
  float rms_norm_epsilon;
} carat_b200_assistant_config;

/* Drafter segments (src/weight_plan.cpp:84-128); all matrices e4m3 + scale (the reference's
 * CARAT_ASSISTANT_FP8_MODE=all, cuda/assistant_runner.cu:147-160). `qkv` holds the `q` segment;
 * k_norm is unused. */
typedef struct carat_b200_assistant_weights {
  const void *token_embedding;   /* e4m3 [vocabulary, hidden]: the drafter's LM head */
  const float *token_embedding_scale;
  const void *pre_projection;    /* e4m3 [hidden, 2 * target hidden] */
  const float *pre_projection_scale;
  const void *post_projection;   /* e4m3 [target hidden, hidden] */
  const float *post_projection_scale;
  const void *final_norm;
  const carat_b200_layer_weights *layers;
} carat_b200_assistant_weights;

/* The drafter's matrices in bf16 (carat::DeviceWeightArena::at of the assistant plan,
 * src/weight_plan.cpp:84-128), needed for the reference's default drafter precision. */
typedef struct carat_b200_assistant_bf16_layer {
  const void *q;
  const void *o;
  const void *gate_up;
  const void *down;
} carat_b200_assistant_bf16_layer;

typedef struct carat_b200_assistant_bf16_weights {
  const void *token_embedding;   /* bf16 [vocabulary, hidden] */
  const void *pre_projection;    /* bf16 [hidden, 2 * target hidden] */
  const void *post_projection;   /* bf16 [target hidden, hidden] */
  const carat_b200_assistant_bf16_layer *layers;
} carat_b200_assistant_bf16_weights;

/* Values of CARAT_ASSISTANT_FP8_MODE in the reference (cuda/assistant_runner.cu:29-43). */
#define CARAT_B200_ASSISTANT_FP8_OFF 0      /* every drafter linear in bf16: the reference's default */
#define CARAT_B200_ASSISTANT_FP8_LM_HEAD 1  /* bf16, except the drafter's LM head in e4m3 */
#define CARAT_B200_ASSISTANT_FP8_ALL 2      /* every drafter linear in e4m3 */

typedef struct carat_b200_runner carat_b200_runner;

/* Builds a runner with `batch` request slots of `maximum_context` tokens on the current device:
 * KV arenas (zero-filled, per layer K then V, each [slot][kv_head][capacity][head_dim] bf16 with
 * capacity = min(maximum_context, sliding_window) for sliding layers), proposal staging,
 * workspaces and RoPE tables. Weights are borrowed and must outlive the runner. assistant and
 * assistant_weights may both be NULL. Replaces the Gemma4BatchModelRunner constructor
 * (include/carat/batch_model_runner.h:24-28, cuda/batch_model_runner.cu:255-606). */
CARAT_B200_API int carat_b200_runner_create(const carat_b200_model_config *config,
                             const carat_b200_model_weights *weights, int batch,
                             int maximum_context, const carat_b200_assistant_config *assistant,
                             const carat_b200_assistant_weights *assistant_weights,
                             carat_b200_runner **runner);
CARAT_B200_API void carat_b200_runner_destroy(carat_b200_runner *runner);

/* INT4 weight-only variant of the target's MLP linears (gate_up and down; group_width 128 or 256,
 * bf16 activations, no e4m3 quantisation of their inputs). The codes are the reordered ones of
 * carat_b200_int4_reorder_weight, the scales those of carat_b200_int4_quantize_weight; the caller
 * keeps them alive. A step then takes at most 128 rows (carat::Int4Bf16Linear::supports_rows,
 * cuda/int4_bf16_linear.cu:326-328). layers == NULL switches back to the e4m3 linears. The
 * reference has this linear (include/carat/linear.h:70-90) but its runner never selects it for the
 * MLP (include/carat/linear.h:47-51), so there is no reference method this replaces. */
typedef struct carat_b200_int4_mlp_layer {
  const void *gate_up_codes;   /* [2 * intermediate, hidden / 2] bytes, reordered */
  const void *gate_up_scales;  /* bf16 [hidden / group_width, 2 * intermediate] */
  const void *down_codes;      /* [hidden, intermediate / 2] bytes, reordered */
  const void *down_scales;     /* bf16 [intermediate / group_width, hidden] */
} carat_b200_int4_mlp_layer;
CARAT_B200_API int carat_b200_runner_use_int4_mlp(carat_b200_runner *runner,
                                                  const carat_b200_int4_mlp_layer *layers,
                                                  int layer_count, int group_width);

enum {
  /* Throughput runs only: every proposal counts as matching, so maximum_accepted alone sets the
   * accepted length (used to inject accept lengths with random-init weights). */
  CARAT_B200_VERIFY_ASSUME_MATCH = 1
};

/* proposals is [requests][depth] row-major. Writes accepted_tokens[requests] and
 * next_tokens[requests]; advances each slot by its accepted count; rejected sliding-ring rows are
 * left exactly as they were; returns after the results are on the host. Error texts match the
 * reference's exceptions. Replaces Gemma4BatchModelRunner::verify_greedy_proposals
 * (include/carat/batch_model_runner.h:55-60, cuda/batch_model_runner.cu:1617-1810). */
CARAT_B200_API int carat_b200_runner_verify_greedy_proposals(carat_b200_runner *runner, const int *proposals,
                                              int requests, int depth,
                                              const int *target_first_tokens, const int *slots,
                                              const int *maximum_accepted_tokens, int flags,
                                              int *accepted_tokens, int *next_tokens);

/* Plain decode: token_ids[row] becomes resident in slots[row] (each slot at most once, none empty
 * or full), every listed slot advances by one position, and next_tokens[row] receives the greedy
 * next token. The forward is the verify forward with one row per slot, so the slot's final hidden
 * state for the drafter is refreshed as well. Returns after the results are on the host. Error
 * texts match the reference's exceptions ("invalid ragged token batch", "invalid or repeated
 * ragged slot", "ragged slot is empty or full"). Replaces Gemma4BatchModelRunner::append_ragged
 * (include/carat/batch_model_runner.h:55, cuda/batch_model_runner.cu:1544-1615); the reference's
 * launch-graph cache for this call has no counterpart because the step is a short chain of
 * dependent launches already overlapped by programmatic dependent launch. */
CARAT_B200_API int carat_b200_runner_append_ragged(carat_b200_runner *runner, const int *token_ids,
                                                   const int *slots, int count, int *next_tokens);

/* proposals_out is [requests][depth]. forced_first_tokens may be NULL. Replaces
 * Gemma4BatchModelRunner::draft_four and Gemma4AssistantRunner::draft_four
 * (include/carat/batch_model_runner.h:62-65, include/carat/assistant_runner.h:20-26,
 * cuda/assistant_runner.cu:218-338). */
CARAT_B200_API int carat_b200_runner_draft(carat_b200_runner *runner, const int *last_tokens, const int *slots,
                            const int *forced_first_tokens, int requests, int depth,
                            int *proposals_out);

/* Makes `count` tokens resident in an empty or partly filled slot by running them through the FP8
 * verify forward `chunk` (<= 8) rows at a time with every row accepted, and returns the greedy
 * next token. An interim stand-in for prefill_slot_chunk (include/carat/batch_model_runner.h:38-41):
 * the reference prefills in BF16 (cuda/batch_model_runner.cu:1274-1275). */
CARAT_B200_API int carat_b200_runner_prefill_slot_fp8(carat_b200_runner *runner, int slot, const int *tokens,
                                       int count, int chunk, int *next_token);

/* Copies the resident KV rows (the first min(position, capacity) rows of every KV head of every
 * layer), the slot's hidden-state hand-off row and the position of source_slot to
 * destination_slot, so a request that shares a prompt prefix starts from it. copied_bytes (may be
 * NULL) receives the KV bytes copied. Errors: "invalid cache slot clone", "source cache slot is
 * empty or full". Replaces Gemma4BatchModelRunner::clone_slot
 * (include/carat/batch_model_runner.h:54, cuda/batch_model_runner.cu:1507-1542). */
CARAT_B200_API int carat_b200_runner_clone_slot(carat_b200_runner *runner, int source_slot,
                                                int destination_slot, uint64_t *copied_bytes);

/* include/carat/batch_model_runner.h:66-72 */
CARAT_B200_API int carat_b200_runner_reset_slot(carat_b200_runner *runner, int slot);
CARAT_B200_API int carat_b200_runner_seed_empty_cache_for_benchmark(carat_b200_runner *runner, int position);
/* Benchmark helper with no counterpart in the reference: like
 * seed_empty_cache_for_benchmark but with one position per slot (`positions` has batch entries),
 * so a synthetic request mix with ragged context lengths can be timed without a prefill. */
CARAT_B200_API int carat_b200_runner_seed_slot_positions(carat_b200_runner *runner,
                                                         const int *positions);
CARAT_B200_API int carat_b200_runner_batch(const carat_b200_runner *runner);
CARAT_B200_API int carat_b200_runner_slot_position(const carat_b200_runner *runner, int slot, int *position);
CARAT_B200_API int carat_b200_runner_has_assistant(const carat_b200_runner *runner);

/* Inspection (tests and tools). */

/* Target argmax of every row of the last verify call, [requests * depth]. */
CARAT_B200_API int carat_b200_runner_last_predictions(carat_b200_runner *runner, int *predictions, int count);
/* Device pointers owned by the runner: which = 0 key cache of `layer`, 1 value cache of `layer`
 * ([slot][kv_head][capacity][head_dim] bf16), 2 hidden-by-slot table [batch, hidden] bf16,
 * 3 final-normed hidden rows of the last verify call [requests * depth, hidden] bf16,
 * 4 the drafter's final-normed hidden rows of its last draft step [requests, drafter hidden],
 * 5 the drafter's carried hidden rows after its last draft step [requests, hidden],
 * 6-12 the last layer's workspaces as the last verify call left them: packed QKV projection,
 * queries, attention output, post-attention residual, gate|up projection, the e4m3 activation
 * buffer, and the fp32 activation scales (four per layer). */
CARAT_B200_API int carat_b200_runner_device_pointer(carat_b200_runner *runner, int which, int layer,
                                     void **pointer, size_t *bytes);
/* Copies `bytes` bytes starting `offset` bytes into one of those buffers to `destination` (host or
 * device memory) after the runner's stream has drained. */
CARAT_B200_API int carat_b200_runner_read(carat_b200_runner *runner, int which, int layer,
                                          size_t offset, void *destination, size_t bytes);
/* The opposite copy, for buffers 0-2 only (KV caches, hidden-by-slot table): restores state saved
 * with carat_b200_runner_read, e.g. to move a slot's KV rows between runners or to start a test
 * from a known cache. Positions are set separately (carat_b200_runner_seed_slot_positions, which
 * zero-fills the caches, so call it first). No counterpart in the reference, whose clone_slot
 * (cuda/batch_model_runner.cu:1499-1542) copies inside one runner. */
CARAT_B200_API int carat_b200_runner_write(carat_b200_runner *runner, int which, int layer,
                                           size_t offset, const void *source, size_t bytes);
/* Device time of the last verify / draft call in milliseconds (CUDA events on the runner's
 * stream, kernels only). */
CARAT_B200_API int carat_b200_runner_last_device_ms(const carat_b200_runner *runner, float *verify_ms,
                                     float *draft_ms);
/* Kernel launches issued by the last verify / draft call. */
CARAT_B200_API int carat_b200_runner_last_launches(const carat_b200_runner *runner, int *verify_launches,
                                    int *draft_launches);
/* Request placement ------------------------------------------------------------------------------- */

/* carat::SlotView (src/runtime/slot_policy.h:13-19): what the scheduler knows about one slot. */
typedef struct carat_b200_slot_view {
  const int *cached_tokens;   /* token ids resident in the slot's KV, host memory */
  int32_t cached_count;
  int32_t occupied;           /* a request is decoding or prefilling in it */
  uint64_t age;               /* smaller = touched longer ago (eviction order) */
  int32_t prefilling;
} carat_b200_slot_view;

/* One replica (one GPU, one runner) as the box-level router sees it. */
typedef struct carat_b200_replica_view {
  const carat_b200_slot_view *slots;
  int32_t slot_count;
  int32_t queued_requests;    /* admitted to this replica but not in a slot yet */
  int32_t alive;              /* 0: the replica left; never chosen */
} carat_b200_replica_view;

#define CARAT_B200_PLACED 0
#define CARAT_B200_NO_FREE_SLOT 1
#define CARAT_B200_RESERVE_BLOCKED 2

/* carat::PlacementDecision (src/runtime/slot_policy.h:27-37) plus the chosen replica. */
typedef struct carat_b200_placement {
  int32_t decision;           /* CARAT_B200_PLACED / NO_FREE_SLOT / RESERVE_BLOCKED */
  int32_t replica;
  int32_t destination;        /* slot the request goes to */
  int32_t source;             /* slot whose cached prefix it reuses, -1 = none */
  uint64_t prefix_tokens;     /* length of that prefix */
} carat_b200_placement;

/* The reference's slot choice inside one replica: carat::select_placement
 * (src/runtime/slot_policy.cpp:22-84), same decisions on the same views. Host only. */
CARAT_B200_API int carat_b200_select_placement(const int *input_ids, int input_count,
                                               const carat_b200_slot_view *slots, int slot_count,
                                               int idle_cache_reserve_slots,
                                               carat_b200_placement *placement);

/* Box-level routing over independent full-model replicas, which the single-GPU reference does
 * not have: the replica whose placement reuses the longest cached prefix, then the least loaded
 * (occupied slots + queued requests), then the lowest index; replicas that left are skipped.
 * RESERVE_BLOCKED when no replica can place the request and at least one was held back by its
 * idle-cache reserve. Host only; no data moves between replicas. */
CARAT_B200_API int carat_b200_route_request(const int *input_ids, int input_count,
                                            const carat_b200_replica_view *replicas,
                                            int replica_count, int idle_cache_reserve_slots,
                                            carat_b200_placement *placement);

/* Weight pipeline ---------------------------------------------------------------------------------- */

/* One execution segment of a loaded model (carat::WeightSegment, include/carat/weight_plan.h:18-24,
 * plus where it lives on the device). Names are the reference's: token_embedding,
 * layer.N.{input_norm,q_norm,k_norm,qkv,o,post_attention_norm,pre_mlp_norm,gate_up,down,
 * post_mlp_norm,scalar}, final_norm; the drafter adds pre_projection, post_projection and
 * layer.N.q (src/weight_plan.cpp:37-128). */
typedef struct carat_b200_weight_segment {
  char name[96];
  int32_t rank;             /* 1 or 2 */
  uint64_t shape[2];        /* [out, in] for matrices */
  uint64_t arena_offset;    /* bytes from the start of the bf16 arena, 256-byte aligned */
  uint64_t byte_size;       /* bf16 bytes */
  const void *bf16;         /* device pointer (DeviceWeightArena::at) */
  const void *fp8;          /* e4m3 bytes, NULL for vectors or when not quantised (Fp8WeightArena::at) */
  const float *fp8_scale;   /* one fp32 on the device (Fp8WeightArena::scale) */
} carat_b200_weight_segment;

typedef struct carat_b200_weights carat_b200_weights;

/* Reads a Hugging Face model directory (model.safetensors.index.json + shards, or a single
 * model.safetensors), builds the execution plan with the reference's checks and messages, uploads
 * every BF16 segment into one device arena (fused qkv and gate_up segments are stacked from their
 * source tensors) and, when quantize_fp8 is non-zero, quantises every matrix to e4m3 with one
 * tensor scale on the device as it arrives. `assistant` NULL loads the target described by
 * `config`; otherwise the drafter, whose pre/post projections take the target's hidden size and
 * vocabulary from `config`. Replaces ShardedSafetensors::open + WeightPlan::gemma4 /
 * gemma4_assistant + DeviceWeightArena::load + Fp8WeightArena::quantize (src/safetensors.cpp,
 * src/weight_plan.cpp:198-222, cuda/device_weights.cu:100-263). */
CARAT_B200_API int carat_b200_weights_load(const char *model_directory,
                                           const carat_b200_model_config *config,
                                           const carat_b200_assistant_config *assistant,
                                           int quantize_fp8, carat_b200_weights **weights);
CARAT_B200_API void carat_b200_weights_destroy(carat_b200_weights *weights);
CARAT_B200_API int carat_b200_weights_segment_count(const carat_b200_weights *weights);
CARAT_B200_API int carat_b200_weights_segment(const carat_b200_weights *weights, int index,
                                              carat_b200_weight_segment *segment);
/* "missing execution weight NAME" when there is no such segment (WeightPlan::at). */
CARAT_B200_API int carat_b200_weights_find(const carat_b200_weights *weights, const char *name,
                                           carat_b200_weight_segment *segment);
/* The weight-only INT4 form of every layer's MLP matrices, built on the device from the loaded
 * bf16 segments "layer.N.gate_up" / "layer.N.down": codes and group scales with the reference's
 * rule and layouts (quantize_bf16_int4_kernel, cuda/int4_bf16_linear.cu:95-136), the codes then
 * reordered for the kernel (the place of cutlass::reorder_tensor, :268-276). group_width 128 or
 * 256. carat_b200_weights_int4_mlp_layers copies out one entry per layer, ready for
 * carat_b200_runner_use_int4_mlp (layers may be NULL to ask for the count only). The buffers live
 * as long as `weights`. */
CARAT_B200_API int carat_b200_weights_quantize_int4_mlp(carat_b200_weights *weights,
                                                        int group_width);
CARAT_B200_API int carat_b200_weights_int4_mlp_layers(const carat_b200_weights *weights,
                                                      carat_b200_int4_mlp_layer *layers,
                                                      int capacity, int *layer_count,
                                                      int *group_width);

/* The plan alone, as text, without touching a device (validate_gemma4_weights and the inspect
 * tool's view): "arena_bytes N" then one line per segment, "NAME shape .. offset N bytes N
 * sources TENSOR@OFFSET ..". *needed receives the size including the terminator; the text is
 * written when buffer_bytes suffices. */
CARAT_B200_API int carat_b200_weights_plan_text(const char *model_directory,
                                                const carat_b200_model_config *config,
                                                const carat_b200_assistant_config *assistant,
                                                char *buffer, size_t buffer_bytes, size_t *needed);

/* The target's matrices in bf16 (carat::DeviceWeightArena::at: layer.N.qkv / o / gate_up / down,
 * row-major [out, in]); the tied LM head is the bf16 token embedding the runner already holds.
 * Needed only for BF16 prefill. */
typedef struct carat_b200_layer_bf16_weights {
  const void *qkv;
  const void *o;
  const void *gate_up;
  const void *down;
} carat_b200_layer_bf16_weights;

CARAT_B200_API int carat_b200_runner_set_bf16_weights(carat_b200_runner *runner,
                                                      const carat_b200_layer_bf16_weights *layers,
                                                      int layer_count);

/* BF16 prompt prefill, one chunk per listed slot: for request r the tokens
 * token_ids[r][position .. position + min(chunk_tokens, remaining)) are made resident, where
 * position is the slot's current position (0 for a reset slot, the cached prefix length after
 * clone_slot) and token_counts[r] the prompt's length. has_prediction[r] = 1 and predictions[r] =
 * the greedy next token only when that request's whole prompt is now resident; its final-normed
 * last hidden row is then handed to the drafter's table. Every linear runs in bf16 even when
 * decode runs in e4m3, as in the reference (cuda/batch_model_runner.cu:1274-1275).
 * Replaces Gemma4BatchModelRunner::prefill_slots_chunks (and, with one slot, prefill_slot_chunk;
 * with chunk_tokens >= every remainder, prefill_slots_suffix's result for a cold cache):
 * include/carat/batch_model_runner.h:37-47, cuda/batch_model_runner.cu:1066-1125,1230-1355.
 * Inside, a chunk is walked in steps of at most eight tokens per request through the same
 * attention kernels the verify step uses; rows of different requests never mix in bf16, so the
 * walk does not change results. Needs carat_b200_runner_set_bf16_weights. */
CARAT_B200_API int carat_b200_runner_prefill_slots_chunks(
    carat_b200_runner *runner, const int *slots, const int *const *token_ids,
    const int *token_counts, int requests, int chunk_tokens, int *predictions,
    int *has_prediction);

/* Selects the drafter's precision like the reference's CARAT_ASSISTANT_FP8_MODE
 * (cuda/assistant_runner.cu:29-43,147-160). A runner starts in CARAT_B200_ASSISTANT_FP8_ALL when
 * it was created with e4m3 drafter matrices; OFF and LM_HEAD need the bf16 matrices (`bf16`, kept
 * by reference like every weight), LM_HEAD and ALL need the e4m3 ones given at creation
 * ("assistant FP8 mode requires quantized assistant weights" otherwise, the reference's text).
 * A drafter created without e4m3 matrices (every matrix pointer of carat_b200_assistant_weights
 * NULL, norms still given) must be put in OFF mode before its first draft. */
CARAT_B200_API int carat_b200_runner_set_assistant_precision(
    carat_b200_runner *runner, int mode, const carat_b200_assistant_bf16_weights *bf16);

#ifdef __cplusplus
}
#endif

#endif /* CARAT_B200_H */
