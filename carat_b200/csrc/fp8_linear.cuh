// Host-side interface of the weight-streaming linear for up to 256 activation rows: e4m3 operands
// with tensor scales (the decode / verify path) or bf16 operands without scales (the drafter's
// default precision and BF16 prefill), one kernel template for both.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace carat_b200 {

// One launch description. Tensor maps are encoded once (weights and activation buffers of the
// runner never move) and captured by value into the kernel parameters.
//
// The kernel is persistent: at most `ctas` CTAs (one per SM) walk the list of work items
// (128-feature tile x K piece), so barrier set-up, TMEM allocation and pipeline fill are paid once
// per CTA and a tile's epilogue overlaps the next tile's loads (two TMEM accumulators).
struct LinearPlan {
  CUtensorMap weight_map;
  CUtensorMap input_map;
  int rows{0};
  int input_width{0};
  int output_width{0};
  int padded_rows{0};       // UMMA N: 32, 64, 128, 192 or 256
  int tiles{0};             // output-feature tiles of 128
  int k_blocks{0};          // 128-byte K blocks
  int ctas{0};              // persistent CTAs (multiprocessor count)
  int splits{1};            // K pieces per tile when there are fewer tiles than SMs
  int k_blocks_per_split{0};
  // When there are more tiles than SMs and the last round is short, the last `tail_tiles` tiles
  // may be cut into `tail_splits` K pieces (launch_linear_bf16_tail); 0 = no such tail.
  int tail_tiles{0};
  int tail_splits{1};
  int tail_k_blocks_per_split{0};
  int element_bytes{1};     // 1: e4m3 operands; 2: bf16 operands (scales are then ignored)
  // Gated plan (make_gated_linear_plan): the weight is [gate rows | up rows], output_width is
  // 2 * gated_width, a tile pairs 64 gate features with their 64 up features and weight_map's
  // box is 64 rows. Only launch_linear_gated takes such a plan.
  int gated_width{0};
};

// Returns 0 or a negative error; `error` (may be null) receives a static message.
// requested_splits <= 0 picks the split factor automatically.
// element_bytes = 2 plans the same linear for bf16 input and weight (input_width a multiple of 8);
// the launch functions then take null scales and multiply by one.
int make_linear_plan(LinearPlan *plan, const void *fp8_input, const void *fp8_weight, int rows,
                     int input_width, int output_width, int requested_splits, const char **error,
                     int element_bytes = 1);

// The gate_up linear with GeGLU in its epilogue. `fp8_weight` is [2 * gated_width, input_width]
// with the gate rows first; gated_width must be a multiple of 64.
int make_gated_linear_plan(LinearPlan *plan, const void *fp8_input, const void *fp8_weight,
                           int rows, int input_width, int gated_width, const char **error,
                           int element_bytes = 1);

// activated[row, j] = bf16(gelu_tanh(g) * u) with g = bf16(acc_gate[row, j] * x_scale * w_scale)
// and u likewise from the up rows: the values launch_linear_bf16 followed by the GeGLU kernel
// produce (cuda/ops.cu:228-284), without the [rows, 2 * gated_width] round trip. The largest
// |activated| is folded into *amax_bits with atomicMax (float bits; the caller zeroes it).
// With `fp8_output` set the launch also does the activation quantisation that follows in the
// reference (cuda/layer_runner.cu:331-347): *scale_out = max / 448 (1 when 0) and
// fp8_output[rows, gated_width] = e4m3(activated / scale).
// `tail_partial` (linear_tail_bytes(plan) bytes; may be null, the plan's K-cut tail is then not
// used) holds the pieces of the tail tiles between the kernel's phases. `grid_counter` is one word
// that is zero on entry and zero again on return; the kernel's grid-wide barriers count on it.
// The grid is one CTA per SM at most, so every CTA is resident; the waits are bounded.
int launch_linear_gated(const LinearPlan &plan, const float *input_scale,
                        const float *weight_scale, void *bf16_activated, unsigned int *amax_bits,
                        void *fp8_output, float *scale_out, float *tail_partial,
                        unsigned int *grid_counter, int *device_error, cudaStream_t stream);

// Bytes of fp32 scratch a plan needs when it splits K (0 when splits == 1):
// [splits, rows, output_width].
std::size_t linear_partial_bytes(const LinearPlan &plan);

// The schedule alone (tiles, K pieces, tail) for a shape: no tensor maps, usable without a device.
void schedule_linear_shape(LinearPlan *plan, int rows, int input_width, int output_width,
                           int requested_splits, int element_bytes = 1);

// The same figure from the shape alone (no tensor maps, usable without a device).
std::size_t linear_partial_bytes_for(int rows, int input_width, int output_width,
                                     int element_bytes = 1);

// y[row, n] = bf16(acc * x_scale * w_scale). When plan.splits > 1 the kernel writes fp32 partial
// sums into `partial` and a second kernel sums, scales and rounds them into `output`.
int launch_linear_bf16(const LinearPlan &plan, const float *input_scale, const float *weight_scale,
                       void *bf16_output, float *partial, int *device_error, cudaStream_t stream);

// bf16 epilogue for the whole tiles; the last plan.tail_tiles tiles leave unscaled fp32 partial sums
// [tail_splits, rows, tail_tiles * 128] in `tail_partial` for a consumer that sums, scales and
// rounds them (the values `bf16_output` would have held in those columns are not written).
int launch_linear_bf16_tail(const LinearPlan &plan, const float *input_scale,
                            const float *weight_scale, void *bf16_output, float *tail_partial,
                            int *device_error, cudaStream_t stream);
std::size_t linear_tail_bytes(const LinearPlan &plan);

// Leaves the unscaled fp32 partial sums [splits, rows, output_width] for a consumer that sums them.
int launch_linear_partial(const LinearPlan &plan, float *partial, int *device_error,
                          cudaStream_t stream);

// Argmax epilogue (always one piece per tile). `best` holds one packed 64-bit key per row and must
// be zero before the launch: (orderable bf16 logit << 32) | ~index, combined with atomicMax, so
// equal logits keep the lowest index. Unpack with best_index().
int launch_linear_argmax(const LinearPlan &plan, const float *input_scale,
                         const float *weight_scale, unsigned long long *best, int *device_error,
                         cudaStream_t stream);

// tokens[row] = index stored in best[row].
int launch_unpack_best(const unsigned long long *best, int *tokens, int rows, cudaStream_t stream);

// Plain one-thread-per-output kernel with the same contract as the bf16 epilogue. It exists so the
// tensor-core kernel can be cross-checked on the device at full size; nothing on the step path
// calls it.
int launch_linear_simt_check(const void *fp8_input, const float *input_scale,
                             const void *fp8_weight, const float *weight_scale, void *bf16_output,
                             int rows, int input_width, int output_width, cudaStream_t stream);

__host__ __device__ inline int best_index(unsigned long long key) {
  return static_cast<int>(~static_cast<unsigned int>(key & 0xFFFFFFFFULL));
}

} // namespace carat_b200
