// Host-side interface of the weight-only INT4 linear (W4A16): signed 4-bit weights in K-local
// groups with one bf16 scale per group, bf16 activations, fp32 accumulation, bf16 output.
//
// Quantiser rule (reference: cuda/int4_bf16_linear.cu:95-136): per output row and group of
// `group_width` consecutive K values, scale = bf16(max|w| / 7) (1.0 when the group is all zero),
// code = clamp(rint(w / float(scale)), -7, 7); two codes per byte, even K in the low nibble; scales
// stored group-major [K / group_width][output_width]. The value the linear multiplies with is
// bf16(code * scale) (reference: tests/cuda_ops_tests.cu:824-843).
#pragma once

#include "fp8_linear.cuh"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace carat_b200 {

// `schedule` reuses the item list of the e4m3 linear (128-feature tiles x K pieces of 128-element
// blocks); its weight_map covers the reordered nibbles, its input_map the bf16 activations.
struct Int4LinearPlan {
  LinearPlan schedule;
  CUtensorMap scale_map;
  int group_shift{0};   // log2(K blocks per scale group): 0 for groups of 128, 1 for 256
};

// codes/scales from a bf16 [output_width, input_width] weight, in the reference's layout.
int launch_int4_quantize(const void *bf16_weight, void *packed_row_major, void *bf16_scales,
                         int output_width, int input_width, int group_width, cudaStream_t stream);

// One-time reordering of the packed codes for the kernel: inside every 32-bit word (eight
// consecutive K values) nibble i holds K value 2i and nibble i + 4 holds K value 2i + 1, each as
// code + 8, so that one shift-and-mask yields a pair of neighbouring K values in the two halves of
// a register. Takes the place of the reference's cutlass::reorder_tensor step
// (cuda/int4_bf16_linear.cu:268-276). `bytes` must be a multiple of 4.
int launch_int4_reorder(const void *packed_row_major, void *reordered, std::size_t bytes,
                        cudaStream_t stream);

// rows <= 128, input_width a multiple of group_width (128 or 256), output_width a multiple of 8.
int make_int4_linear_plan(Int4LinearPlan *plan, const void *bf16_input, const void *reordered_weight,
                          const void *bf16_scales, int rows, int input_width, int output_width,
                          int group_width, int requested_splits, const char **error);

// fp32 scratch the plan needs (split-K pieces or the K-cut tail round), 0 when none.
std::size_t int4_linear_partial_bytes(const Int4LinearPlan &plan);
std::size_t int4_linear_partial_bytes_for(int rows, int input_width, int output_width);

// output[row, n] = bf16(sum_k input[row, k] * bf16(code[n, k] * scale[k / group, n])).
// Split plans leave fp32 pieces in `partial` and a second kernel sums and rounds them.
int launch_int4_linear_bf16(const Int4LinearPlan &plan, void *bf16_output, float *partial,
                            int *device_error, cudaStream_t stream);

// Whole tiles to bf16, the tail tiles as fp32 pieces [tail_splits, rows, tail_tiles * 128] for a
// consumer that sums and rounds them.
int launch_int4_linear_bf16_tail(const Int4LinearPlan &plan, void *bf16_output, float *tail_partial,
                                 int *device_error, cudaStream_t stream);

// fp32 pieces [splits, rows, output_width] for a consumer that sums and rounds them.
int launch_int4_linear_partial(const Int4LinearPlan &plan, float *partial, int *device_error,
                               cudaStream_t stream);

// One output per thread from the reference-layout codes; a device-side cross-check for tests.
int launch_int4_linear_simt_check(const void *bf16_input, const void *packed_row_major,
                                  const void *bf16_scales, void *bf16_output, int rows,
                                  int input_width, int output_width, int group_width,
                                  cudaStream_t stream);

} // namespace carat_b200
