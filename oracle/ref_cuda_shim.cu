// TEST INFRASTRUCTURE ONLY: an extern "C" face on the reference's own CUDA code, compiled for
// sm_100a from where its sources lie (see the `ref_cuda` target of the Makefile beside this file)
// so that GPU tests can run the reference's operators and its whole batch runner next to the
// new kernels on the same inputs. Nothing in the product links or loads the resulting library.
//
// What is linked: the reference's cuda/{ops,linear,qkv,prefill_gemm_attention,gemm_attention,
// attention,layer_runner,batch_model_runner,assistant_runner}.cu and src/{gemma4_config,json}.cpp,
// unmodified, with the CUDA toolkit and cuBLAS/cuBLASLt only. The parts of the reference that
// need other libraries are not compiled; the few classes and functions the linked sources still
// name are defined here as placeholders that refuse to run:
//   * carat::CudnnPrefillAttention (cuDNN graph API: BF16 sliding prefill),
//   * carat::Int4Fp8Linear / Int4Bf16Linear (CUTLASS, off unless an environment switch asks),
//   * the wgmma global-attention helpers of hopper_attention.cu (sm_90a only).
// The weight arenas (carat::DeviceWeightArena / Fp8WeightArena) are also defined here: instead of
// reading safetensors they hand out device pointers the test supplies, through the reference's
// own at(name) / scale(name) interface (include/carat/device_weights.h).
#include "carat/assistant_runner.h"
#include "carat/attention.h"
#include "carat/batch_model_runner.h"
#include "carat/cuda_ops.h"
#include "carat/device_weights.h"
#include "carat/gemm_attention.h"
#include "carat/gemma4_config.h"
#include "carat/linear.h"
#include "carat/prefill_attention.h"
#include "carat/prefill_gemm_attention.h"
#include "carat/qkv.h"

#include <cuda_runtime.h>

#include <cstring>
#include <map>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>

namespace carat {

#include "ref_arenas.inc"

// ---------------------------------------------------------------------------- placeholders
struct CudnnPrefillAttention::Implementation {};
CudnnPrefillAttention::CudnnPrefillAttention() = default;
CudnnPrefillAttention::~CudnnPrefillAttention() = default;
void CudnnPrefillAttention::run(const void *, const void *, const void *, void *, int, int, int,
                                int, int, int, int, int, cudaStream_t) {
  throw std::runtime_error("cuDNN prefill attention is not part of the test oracle build");
}

struct Int4Fp8Linear::Implementation {};
Int4Fp8Linear::Int4Fp8Linear(const void *, int, int, int, int, int) {
  throw std::runtime_error("INT4 FP8 linear is not part of the test oracle build");
}
Int4Fp8Linear::~Int4Fp8Linear() = default;
bool Int4Fp8Linear::supports_rows(int) const { return false; }
void Int4Fp8Linear::run(const void *, void *, int, cudaStream_t, int) {
  throw std::runtime_error("INT4 FP8 linear is not part of the test oracle build");
}
std::size_t Int4Fp8Linear::allocated_bytes() const { return 0; }

struct Int4Bf16Linear::Implementation {};
Int4Bf16Linear::Int4Bf16Linear(const void *, int, int, int, bool) {
  throw std::runtime_error("INT4 BF16 linear is not part of the test oracle build");
}
Int4Bf16Linear::~Int4Bf16Linear() = default;
bool Int4Bf16Linear::supports_rows(int) const { return false; }
void Int4Bf16Linear::run(const void *, void *, int, cudaStream_t, int) {
  throw std::runtime_error("INT4 BF16 linear is not part of the test oracle build");
}
std::size_t Int4Bf16Linear::allocated_bytes() const { return 0; }

[[noreturn]] static void no_hopper() {
  throw std::runtime_error("wgmma attention helpers are not part of the test oracle build");
}
void grouped_global_pv_wgmma_fp8_rs(const void *, const void *, void *, void *, int, int, int, int,
                                    int, int, int, cudaStream_t) {
  no_hopper();
}
void grouped_global_pv_wgmma_int8_rs(const void *, const void *, const float *, void *, void *, int,
                                     int, int, int, int, int, int, cudaStream_t) {
  no_hopper();
}
void grouped_global_qk_wgmma_int8_block128(const void *, const float *, const void *, const float *,
                                           void *, int, int, int, int, int, int, cudaStream_t,
                                           int) {
  no_hopper();
}
void quantize_grouped_global_value_span_wgmma_fp8(const void *, void *, int, int, int, int, int,
                                                  cudaStream_t) {
  no_hopper();
}
void quantize_grouped_global_value_span_wgmma_int8(const void *, void *, float *, int, int, int,
                                                   int, int, cudaStream_t) {
  no_hopper();
}
void quantize_grouped_global_decode_values_wgmma_fp8(const void *, void *, const int *, const int *,
                                                     int, int, int, int, int, cudaStream_t) {
  no_hopper();
}
void quantize_grouped_global_probabilities_wgmma_fp8(const void *, void *, int, int, int, int,
                                                     cudaStream_t) {
  no_hopper();
}
void quantize_grouped_global_decode_values_wgmma_int8(const void *, void *, float *, const int *,
                                                      const int *, int, int, int, int, int,
                                                      cudaStream_t) {
  no_hopper();
}

} // namespace carat

// ---------------------------------------------------------------------------- C face
// Every call returns with the device drained, so a fault shows up at the call that caused it.
#define REF_FACE_AFTER_CALL() cudaDeviceSynchronize()
#include "ref_face_helpers.inc"

namespace {

carat::Fp8Linear &fp8_linear() {
  static carat::Fp8Linear linear(carat::Fp8Scaling::tensor);
  return linear;
}
carat::Bf16Linear &bf16_linear() {
  static carat::Bf16Linear linear;
  return linear;
}
carat::Gemma4QkvPostprocessor &qkv_postprocessor(int maximum_positions) {
  static std::map<int, std::unique_ptr<carat::Gemma4QkvPostprocessor>> made;
  auto &entry = made[maximum_positions];
  if (!entry)
    entry = std::make_unique<carat::Gemma4QkvPostprocessor>(maximum_positions);
  return *entry;
}
carat::GemmCausalPrefillAttention &prefill_attention(int tokens, int heads, int requests) {
  static std::map<std::tuple<int, int, int>, std::unique_ptr<carat::GemmCausalPrefillAttention>>
      made;
  auto &entry = made[std::make_tuple(tokens, heads, requests)];
  if (!entry)
    entry = std::make_unique<carat::GemmCausalPrefillAttention>(tokens, heads, requests);
  return *entry;
}
carat::GemmGroupedDecodeAttention &decode_attention(int batch, int kv_heads, int group,
                                                    int context) {
  static std::map<std::tuple<int, int, int, int>,
                  std::unique_ptr<carat::GemmGroupedDecodeAttention>>
      made;
  auto &entry = made[std::make_tuple(batch, kv_heads, group, context)];
  if (!entry)
    entry = std::make_unique<carat::GemmGroupedDecodeAttention>(batch, kv_heads, group, context);
  return *entry;
}

} // namespace

extern "C" {

const char *ref_last_error(void) { return last_error.c_str(); }

// ---- include/carat/linear.h:93-110
int ref_quantize_bf16_to_fp8_e4m3(const void *input, void *output, float *scale,
                                  size_t elements) {
  return guarded([&] { carat::quantize_bf16_to_fp8_e4m3(input, output, scale, elements, nullptr); });
}
int ref_quantize_bf16_to_fp8_e4m3_from_row_amax(const void *input, void *output, float *scale,
                                                const float *row_amax, int rows, int width) {
  return guarded([&] {
    carat::quantize_bf16_to_fp8_e4m3_from_row_amax(input, output, scale, row_amax, rows, width,
                                                   nullptr);
  });
}
int ref_quantize_bf16_to_fp8_e4m3_from_amax_values(const void *input, void *output, float *scale,
                                                   const float *amax_values, int amax_count,
                                                   int rows, int width) {
  return guarded([&] {
    carat::quantize_bf16_to_fp8_e4m3_from_amax_values(input, output, scale, amax_values,
                                                      amax_count, rows, width, nullptr);
  });
}
// ---- include/carat/linear.h:13-41
int ref_fp8_linear_run(const void *fp8_input, const float *input_scale, const void *fp8_weight,
                       const float *weight_scale, void *bf16_output, int rows, int input_width,
                       int output_width) {
  return guarded([&] {
    fp8_linear().run(fp8_input, input_scale, fp8_weight, weight_scale, bf16_output, rows,
                     input_width, output_width, nullptr);
  });
}
// Launches only (no synchronisation), for timing a sequence with CUDA events on stream 0.
int ref_fp8_linear_launch(const void *fp8_input, const float *input_scale, const void *fp8_weight,
                          const float *weight_scale, void *bf16_output, int rows, int input_width,
                          int output_width) {
  try {
    fp8_linear().run(fp8_input, input_scale, fp8_weight, weight_scale, bf16_output, rows,
                     input_width, output_width, nullptr);
    return 0;
  } catch (const std::exception &error) {
    last_error = error.what();
    return -1;
  }
}
int ref_quantize_argmax_launch(const void *bf16_input, void *fp8_scratch, float *scale_scratch,
                               const void *fp8_weight, const float *weight_scale,
                               void *bf16_logits, int *tokens, void *argmax_workspace, int rows,
                               int input_width, int output_width) {
  // The reference's unfused LM-head chain: quantise -> cuBLASLt FP8 GEMM -> row argmax
  // (cuda/batch_model_runner.cu:840-853,938-940).
  try {
    carat::quantize_bf16_to_fp8_e4m3(bf16_input, fp8_scratch, scale_scratch,
                                     static_cast<size_t>(rows) * input_width, nullptr);
    fp8_linear().run(fp8_scratch, scale_scratch, fp8_weight, weight_scale, bf16_logits, rows,
                     input_width, output_width, nullptr);
    carat::argmax_bf16_rows(bf16_logits, rows, output_width, tokens, argmax_workspace, nullptr);
    return 0;
  } catch (const std::exception &error) {
    last_error = error.what();
    return -1;
  }
}
int ref_bf16_linear_run(const void *input, const void *weight, void *output, int rows,
                        int input_width, int output_width) {
  return guarded(
      [&] { bf16_linear().run(input, weight, output, rows, input_width, output_width, nullptr); });
}

// ---- include/carat/cuda_ops.h
int ref_rms_norm_bf16(const void *input, const void *weight, void *output, size_t rows,
                      size_t width, float epsilon) {
  return guarded([&] { carat::rms_norm_bf16(input, weight, output, rows, width, epsilon, nullptr); });
}
int ref_rms_norm_bf16_with_row_amax(const void *input, const void *weight, void *output,
                                    float *row_amax, size_t rows, size_t width, float epsilon) {
  return guarded([&] {
    carat::rms_norm_bf16_with_row_amax(input, weight, output, row_amax, rows, width, epsilon,
                                       nullptr);
  });
}
int ref_rms_norm_add_and_norm_bf16(const void *input, const void *weight, const void *residual,
                                   const void *next_weight, void *residual_output,
                                   void *normalized_output, size_t rows, size_t width,
                                   float epsilon) {
  return guarded([&] {
    carat::rms_norm_add_and_norm_bf16(input, weight, residual, next_weight, residual_output,
                                      normalized_output, rows, width, epsilon, nullptr);
  });
}
int ref_rms_norm_add_and_norm_bf16_with_row_amax(const void *input, const void *weight,
                                                 const void *residual, const void *next_weight,
                                                 void *residual_output, void *normalized_output,
                                                 float *row_amax, size_t rows, size_t width,
                                                 float epsilon) {
  return guarded([&] {
    carat::rms_norm_add_and_norm_bf16_with_row_amax(input, weight, residual, next_weight,
                                                    residual_output, normalized_output, row_amax,
                                                    rows, width, epsilon, nullptr);
  });
}
int ref_rms_norm_add_scale_bf16(const void *input, const void *weight, const void *residual,
                                const void *scalar, void *output, size_t rows, size_t width,
                                float epsilon) {
  return guarded([&] {
    carat::rms_norm_add_scale_bf16(input, weight, residual, scalar, output, rows, width, epsilon,
                                   nullptr);
  });
}
int ref_gelu_tanh_gate_rows_bf16(const void *packed_gate_up, void *output, int rows, int width) {
  return guarded([&] { carat::gelu_tanh_gate_rows_bf16(packed_gate_up, output, rows, width, nullptr); });
}
int ref_gelu_tanh_gate_rows_bf16_with_block_amax(const void *packed_gate_up, void *output,
                                                 float *block_amax, int rows, int width) {
  return guarded([&] {
    carat::gelu_tanh_gate_rows_bf16_with_block_amax(packed_gate_up, output, block_amax, rows,
                                                    width, nullptr);
  });
}
int ref_reduce_block_amax_to_rows(const float *block_amax, float *row_amax, int rows,
                                  int blocks_per_row) {
  return guarded(
      [&] { carat::reduce_block_amax_to_rows(block_amax, row_amax, rows, blocks_per_row, nullptr); });
}
int ref_embedding_batch_bf16(const void *embedding, const int *tokens, void *output, int batch,
                             int vocabulary, int hidden, float scale) {
  return guarded([&] {
    carat::embedding_batch_bf16(embedding, tokens, output, batch, vocabulary, hidden, scale,
                                nullptr);
  });
}
int ref_token_to_head_batch_bf16(const void *input, void *output, int requests, int tokens,
                                 int heads, int head_dimension) {
  return guarded([&] {
    carat::token_to_head_batch_bf16(input, output, requests, tokens, heads, head_dimension,
                                    nullptr);
  });
}
int ref_head_to_token_batch_bf16(const void *input, void *output, int requests, int tokens,
                                 int heads, int head_dimension) {
  return guarded([&] {
    carat::head_to_token_batch_bf16(input, output, requests, tokens, heads, head_dimension,
                                    nullptr);
  });
}
int ref_head_to_token_batch_bf16_with_block_amax(const void *input, void *output,
                                                 float *block_amax, int requests, int tokens,
                                                 int heads, int head_dimension) {
  return guarded([&] {
    carat::head_to_token_batch_bf16_with_block_amax(input, output, block_amax, requests, tokens,
                                                    heads, head_dimension, nullptr);
  });
}
int ref_backup_kv_ring_spans_bf16(const void *const *key_sources, const void *const *value_sources,
                                  void *backup_keys, void *backup_values, const int *positions,
                                  int requests, int heads, int tokens, int head_dimension,
                                  int capacity) {
  return guarded([&] {
    carat::backup_kv_ring_spans_bf16(key_sources, value_sources, backup_keys, backup_values,
                                     positions, requests, heads, tokens, head_dimension, capacity,
                                     nullptr);
  });
}
int ref_restore_kv_ring_suffixes_bf16(const void *backup_keys, const void *backup_values,
                                      void *const *key_destinations,
                                      void *const *value_destinations, const int *positions,
                                      const int *accepted, int requests, int heads, int tokens,
                                      int head_dimension, int capacity) {
  return guarded([&] {
    carat::restore_kv_ring_suffixes_bf16(backup_keys, backup_values, key_destinations,
                                         value_destinations, positions, accepted, requests, heads,
                                         tokens, head_dimension, capacity, nullptr);
  });
}
size_t ref_argmax_bf16_workspace_bytes(int elements) {
  return carat::argmax_bf16_workspace_bytes(elements);
}
int ref_argmax_bf16_rows(const void *values, int rows, int elements, int *output,
                         void *workspace) {
  return guarded([&] { carat::argmax_bf16_rows(values, rows, elements, output, workspace, nullptr); });
}

// ---- include/carat/qkv.h
int ref_qkv_run_prefill_uniform_direct(int maximum_positions, const void *packed_qkv,
                                       const void *query_norm, const void *key_norm,
                                       void *queries, void *const *key_caches,
                                       void *const *value_caches, const int *positions,
                                       int requests, int tokens, int query_heads, int kv_heads,
                                       int head_dimension, int key_equals_value, int capacity,
                                       float epsilon) {
  return guarded([&] {
    qkv_postprocessor(maximum_positions)
        .run_prefill_uniform_direct(packed_qkv, query_norm, key_norm, queries, key_caches,
                                    value_caches, positions, requests, tokens, query_heads,
                                    kv_heads, head_dimension, key_equals_value != 0, capacity,
                                    epsilon, nullptr);
  });
}
int ref_qkv_run_prefill_uniform(int maximum_positions, const void *packed_qkv,
                                const void *query_norm, const void *key_norm, void *queries,
                                void *staged_keys, void *staged_values, const int *positions,
                                int requests, int tokens, int query_heads, int kv_heads,
                                int head_dimension, int key_equals_value,
                                int staged_position_start, int staged_capacity, float epsilon) {
  return guarded([&] {
    qkv_postprocessor(maximum_positions)
        .run_prefill_uniform(packed_qkv, query_norm, key_norm, queries, staged_keys, staged_values,
                             positions, requests, tokens, query_heads, kv_heads, head_dimension,
                             key_equals_value != 0, staged_position_start, staged_capacity,
                             epsilon, nullptr);
  });
}
int ref_qkv_run_query_ragged(int maximum_positions, const void *projected, const void *query_norm,
                             void *queries, const int *positions, int batch, int query_heads,
                             int head_dimension, int global_attention, float epsilon) {
  return guarded([&] {
    qkv_postprocessor(maximum_positions)
        .run_query_ragged(projected, query_norm, queries, positions, batch, query_heads,
                          head_dimension, global_attention != 0, epsilon, nullptr);
  });
}

// ---- include/carat/prefill_gemm_attention.h
int ref_attention_run_uniform_batch(int maximum_tokens, int maximum_query_heads,
                                    int maximum_requests, const void *query,
                                    const void *const *key_caches,
                                    const void *const *value_caches, void *output,
                                    const int *positions, int requests, int query_heads,
                                    int kv_heads, int query_tokens, int maximum_kv_tokens,
                                    int capacity, int head_dimension) {
  return guarded([&] {
    prefill_attention(maximum_tokens, maximum_query_heads, maximum_requests)
        .run_uniform_batch(query, key_caches, value_caches, output, positions, requests,
                           query_heads, kv_heads, query_tokens, maximum_kv_tokens, capacity,
                           head_dimension, nullptr);
  });
}
int ref_attention_run_uniform_ring_batch(int maximum_tokens, int maximum_query_heads,
                                         int maximum_requests, const void *query,
                                         const void *const *key_caches,
                                         const void *const *value_caches, const void *backup_keys,
                                         const void *backup_values, void *output,
                                         const int *positions, int requests, int query_heads,
                                         int kv_heads, int query_tokens, int ring_capacity,
                                         int head_dimension) {
  return guarded([&] {
    prefill_attention(maximum_tokens, maximum_query_heads, maximum_requests)
        .run_uniform_ring_batch(query, key_caches, value_caches, backup_keys, backup_values,
                                output, positions, requests, query_heads, kv_heads, query_tokens,
                                ring_capacity, head_dimension, nullptr);
  });
}
// ---- include/carat/gemm_attention.h
int ref_decode_attention_run_ragged(int maximum_batch, int maximum_kv_heads, int maximum_group,
                                    int maximum_context, const void *query, const void *keys,
                                    const void *values, void *output, const int *positions,
                                    const int *slots, int batch, int maximum_slots, int kv_heads,
                                    int query_group, int maximum_context_length,
                                    int head_dimension, int capacity) {
  return guarded([&] {
    decode_attention(maximum_batch, maximum_kv_heads, maximum_group, maximum_context)
        .run_ragged(query, keys, values, output, positions, slots, batch, maximum_slots, kv_heads,
                    query_group, maximum_context_length, head_dimension, nullptr, capacity);
  });
}

#include "ref_runner_face.inc"

// ---- carat::Gemma4AssistantRunner on its own (include/carat/assistant_runner.h:11-32): the
// caller supplies the target embedding, the hidden-by-slot table and the two shared KV layers as
// raw device pointers, exactly as Gemma4BatchModelRunner::draft_four does.
struct ref_assistant {
  std::unique_ptr<carat::DeviceWeightArena> weights;
  std::unique_ptr<carat::Fp8WeightArena> fp8;
  std::unique_ptr<carat::Gemma4AssistantRunner> runner;
};

ref_assistant *ref_assistant_create(const ref_segment *bf16, int bf16_count,
                                    const ref_segment *fp8, int fp8_count, int maximum_batch,
                                    int maximum_context) {
  try {
    auto made = std::make_unique<ref_assistant>();
    const carat::ShardedSafetensors none;
    made->weights = carat::DeviceWeightArena::load(table_of(bf16, bf16_count), none);
    if (fp8 != nullptr && fp8_count > 0) {
      made->fp8 = carat::Fp8WeightArena::quantize(table_of(fp8, fp8_count), *made->weights,
                                                  carat::Fp8Scaling::tensor);
    }
    made->runner = std::make_unique<carat::Gemma4AssistantRunner>(
        *made->weights, made->fp8.get(), maximum_batch, maximum_context);
    return made.release();
  } catch (const std::exception &error) {
    last_error = error.what();
    return nullptr;
  }
}

void ref_assistant_destroy(ref_assistant *assistant) { delete assistant; }

int ref_assistant_draft_four(ref_assistant *assistant, const void *target_embedding,
                             const void *target_hidden_by_slot, const int *last_tokens,
                             const int *context_positions, const int *slots,
                             const int *forced_first, int requests, int maximum_slots, int depth,
                             const void *sliding_keys, const void *sliding_values,
                             int sliding_capacity, const void *global_keys,
                             const void *global_values, int global_capacity, int *proposals) {
  return guarded([&] {
    const std::vector<int> last(last_tokens, last_tokens + requests);
    const std::vector<int> contexts(context_positions, context_positions + requests);
    const std::vector<int> slot_list(slots, slots + requests);
    const std::vector<int> forced = forced_first == nullptr
                                        ? std::vector<int>{}
                                        : std::vector<int>(forced_first, forced_first + requests);
    const auto drafted = assistant->runner->draft_four(
        target_embedding, target_hidden_by_slot, last, contexts, slot_list, forced, maximum_slots,
        depth, sliding_keys, sliding_values, sliding_capacity, global_keys, global_values,
        global_capacity);
    for (int request = 0; request < requests; ++request)
      std::memcpy(proposals + request * depth, drafted[static_cast<size_t>(request)].data(),
                  sizeof(int) * depth);
  });
}

} // extern "C"
