// Row-wise fused operators of the verify / draft step. Each one produces a bf16 activation row the
// way the reference does (same fp32 math, same bf16 rounding points) and, in the same launch,
// quantises the whole [rows, width] tensor to e4m3 with the reference's tensor-wide scale rule
// (amax / 448, cuda/linear.cu:76-115). The tensor-wide maximum couples all rows, so the kernels are
// cooperative launches: one CTA per row, an atomic maximum, one grid barrier, then every CTA
// quantises its row straight from shared memory. Nothing is re-read from HBM.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace carat_b200 {

// Where a quantised activation goes, plus the running maximum that must be zero before the launch.
struct QuantTarget {
  void *fp8_output;        // [rows, width] e4m3
  float *scale;            // one fp32: amax / 448 (1.0 when amax == 0)
  unsigned int *amax_bits; // scratch word, zero on entry
  // Optional bf16 scratch [rows, width]: lets the call run as two launches when there are more
  // rows than the device holds CTAs at once (the one-launch form needs a grid barrier). Without
  // it such calls fail. The embedding entry point then expects its scratch words pre-cleared.
  void *two_launch_rows = nullptr;
  // When fp8_output is null the call stops after the bf16 row: it is stored here and nothing is
  // quantised (the consumer is a linear with bf16 activations; scale and amax_bits are unused).
  void *bf16_output = nullptr;
  // Optional word for the one-launch form's grid barrier: it must be the word right after
  // `amax_bits`, the pair eight-byte aligned and zero on entry (the kernel reads both with one
  // load; the count stays in the word afterwards, so the caller clears the pair before its next
  // use). With it the
  // kernel counts its CTAs in on this word and is launched as an ordinary kernel; without it the
  // launch is cooperative and uses the cooperative-groups grid barrier. The difference matters in
  // a chain: a cooperative launch does not overlap with its neighbours under programmatic
  // dependent launch, an ordinary one does (measured: 0.45 ms of a 13.9 ms verify step). Either
  // way the grid is no larger than what the device holds at once, and the wait on the word is
  // bounded: `barrier_error` receives code 7 if it runs out.
  unsigned int *barrier_word = nullptr;
  int *barrier_error = nullptr;
};

// Sum of split-K partials: value = bf16((sum_s partial[s]) * input_scale * weight_scale).
struct PartialSource {
  const float *partial;      // [splits, rows, width] fp32
  int splits;
  const float *input_scale;  // device scalars of the linear that produced the partials
  const float *weight_scale;
  // Optional: pieces beyond valid_splits[row / rows_per_group] were never written and are skipped
  // (attention chunk partials: one count per request, rows_per_group = depth).
  const int *valid_splits = nullptr;
  int rows_per_group = 1;
};

// Tensor-scale quantisation of a tensor of any size in three launches (amax, scale, convert), the
// form the reference uses for weights at load time (cuda/linear.cu:117-153,261-271).
// *amax_bits must be zero on entry.
int launch_quant_tensor(const void *input, void *fp8_output, float *scale,
                        unsigned int *amax_bits, size_t elements, cudaStream_t stream);

// hidden = bf16(embedding[token] * bf16(sqrt(width))) (cuda/ops.cu:321-335); normalized =
// bf16(rmsnorm(hidden) * norm_weight) (cuda/ops.cu:27-68) -> e4m3. Also zeroes `clear_words`
// 32-bit words at `clear_base` (the per-step amax scratch) before anything uses them.
int launch_embed_norm_quant(const void *embedding, const int *tokens, int vocabulary,
                            const void *norm_weight, void *hidden_out, QuantTarget target,
                            int rows, int width, float epsilon, unsigned int *clear_base,
                            int clear_words, cudaStream_t stream);

// Drafter input row: [ bf16(embedding[token] * bf16(sqrt(width))) | hidden[source_row] ] -> e4m3 over
// 2 * width columns (cuda/assistant_runner.cu:279-285). source_row = row_indices[r] when
// row_indices is given (first draft step: gather from the per-slot table), else r.
int launch_embed_concat_quant(const void *embedding, const int *tokens, int vocabulary,
                              const void *hidden, const int *row_indices, QuantTarget target,
                              int rows, int width, cudaStream_t stream);

// normalized = bf16(rmsnorm(input) * norm_weight) -> e4m3 (cuda/layer_runner.cu:241-262 without the
// intermediate bf16 tensor). When normalized_out is not null the bf16 rows are stored too.
int launch_norm_quant(const void *input, const void *norm_weight, void *normalized_out,
                      QuantTarget target, int rows, int width, float epsilon,
                      cudaStream_t stream);

// Plain tensor-scale quantisation of a bf16 tensor (cuda/linear.cu:76-115). When `partials` is
// given (attention split over key chunks) the bf16 input is first formed as
// bf16(sum_c partials[c]) from [chunks, rows, width] fp32. `request_chunks` (may be null: every
// chunk counts) holds, per group of `rows_per_request` rows, how many chunks were written.
int launch_quant(const void *input, const float *chunk_partials, int chunks,
                 const int *request_chunks, int rows_per_request, QuantTarget target, int rows,
                 int width, cudaStream_t stream);

// projected = source (bf16 tensor or split-K partials); first = bf16(rmsnorm(projected) * w1 +
// residual); second = bf16(rmsnorm(first) * w2) -> e4m3 (cuda/ops.cu:87-179,
// cuda/layer_runner.cu:306-330). `first_out` receives the new residual stream.
int launch_post_attention_norms_quant(const void *projected, PartialSource source,
                                      const void *norm_weight, const void *residual,
                                      const void *next_norm_weight, void *first_out,
                                      QuantTarget target, int rows, int width, float epsilon,
                                      cudaStream_t stream);

// The last columns of a packed [gate | up] row when the linear that produced it left them as fp32
// K-piece partial sums (launch_linear_bf16_tail): [splits, rows, width] covering packed columns
// first_column .. first_column + width, all inside the up half. partial == nullptr: no tail.
struct TailSource {
  const float *partial;
  int splits;
  int first_column;
  int width;
  const float *input_scale;
  const float *weight_scale;
};

// activated = bf16(gelu_tanh(gate) * up) from rows packed [gate | up] -> e4m3
// (cuda/ops.cu:228-284).
int launch_geglu_quant(const void *packed_gate_up, TailSource tail, QuantTarget target, int rows,
                       int width, cudaStream_t stream);

// down = source; output = bf16(bf16(rmsnorm(down) * w + residual) * scalar)
// (cuda/ops.cu:181-217); then next = bf16(rmsnorm(output) * next_norm_weight) -> e4m3, which is
// the following layer's input norm or the final norm. `next_out` (may be null) stores the bf16
// rows of `next` (the final-normed hidden state the drafter receives).
int launch_layer_output_norm_quant(const void *down, PartialSource source, const void *norm_weight,
                                   const void *residual, const void *scalar, void *output,
                                   const void *next_norm_weight, void *next_out,
                                   QuantTarget target, int rows, int width, float epsilon,
                                   cudaStream_t stream);

// e4m3 rows from bf16 rows whose tensor-wide maximum is already in target.amax_bits (left there by
// the producer of the rows, e.g. the gated linear epilogue): scale = max / 448 to target.scale,
// e4m3(x / scale) to target.fp8_output. No grid barrier; `elements` a multiple of eight.
int launch_quantize_rows(const void *bf16_rows, QuantTarget target, size_t elements,
                         cudaStream_t stream);

#ifdef __CUDACC__
// tanh-form GELU of the reference's GeGLU (cuda/ops.cu:228-284), shared by the stand-alone GeGLU
// kernel and the gated linear epilogue so that both round identically.
__device__ __forceinline__ float gelu_tanh(float value) {
  constexpr float coefficient = 0.7978845608028654F;
  return 0.5F * value * (1.0F + tanhf(coefficient * (value + 0.044715F * value * value * value)));
}
#endif

} // namespace carat_b200
