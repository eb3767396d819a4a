// C entry points for the FP8 and INT4 linear kernels (declared in include/carat_b200.h).
#include "../../include/carat_b200.h"
#include "context.cuh"
#include "fp8_linear.cuh"
#include "int4_linear.cuh"

using namespace carat_b200;

namespace {

int plan_or_fail(LinearPlan *plan, const void *input, const void *weight, int rows, int input_width,
                 int output_width, int splits, int element_bytes = 1) {
  const char *message = "invalid FP8 linear shape";
  const int status = make_linear_plan(plan, input, weight, rows, input_width, output_width,
                                      splits, &message, element_bytes);
  if (status != 0)
    set_last_error(message);
  return status;
}

int launch_status(int status, const char *what) {
  if (status == 0)
    return 0;
  set_last_error(std::string(what) + " launch failed: " +
                 cudaGetErrorString(cudaGetLastError()));
  return status;
}

} // namespace

extern "C" const char *carat_b200_last_error(void) { return last_error_text(); }

extern "C" int carat_b200_abi_version(void) { return 1; }

extern "C" int carat_b200_device_error(int *code) { return read_and_clear_device_error(code); }

extern "C" size_t carat_b200_fp8_linear_workspace_bytes(int rows, int input_width,
                                                        int output_width) {
  return linear_partial_bytes_for(rows, input_width, output_width);
}

extern "C" int carat_b200_fp8_linear(const void *fp8_input, const float *device_input_scale,
                                     const void *fp8_weight, const float *device_weight_scale,
                                     void *bf16_output, int rows, int input_width,
                                     int output_width, void *workspace, size_t workspace_bytes,
                                     void *stream) {
  if (device_input_scale == nullptr || device_weight_scale == nullptr || bf16_output == nullptr) {
    set_last_error("invalid FP8 linear shape");
    return -1;
  }
  LinearPlan plan;
  int status = plan_or_fail(&plan, fp8_input, fp8_weight, rows, input_width, output_width, 0);
  if (status != 0)
    return status;
  const size_t needed = linear_partial_bytes(plan);
  if (needed > 0 && (workspace == nullptr || workspace_bytes < needed)) {
    set_last_error("FP8 linear workspace is too small");
    return -6;
  }
  int *error_word = device_error_word();
  if (error_word == nullptr) {
    set_last_error("device error word is unavailable");
    return -101;
  }
  status = launch_linear_bf16(plan, device_input_scale, device_weight_scale, bf16_output,
                              static_cast<float *>(workspace), error_word,
                              static_cast<cudaStream_t>(stream));
  return launch_status(status, "FP8 linear");
}

extern "C" int carat_b200_fp8_linear_argmax(const void *fp8_input, const float *device_input_scale,
                                            const void *fp8_weight,
                                            const float *device_weight_scale, int *device_tokens,
                                            void *device_keys, int rows, int input_width,
                                            int output_width, void *stream) {
  if (device_input_scale == nullptr || device_weight_scale == nullptr ||
      device_tokens == nullptr || device_keys == nullptr) {
    set_last_error("invalid FP8 linear shape");
    return -1;
  }
  LinearPlan plan;
  // One piece per tile: the LM head has thousands of tiles, the tail round needs no cutting.
  int status = plan_or_fail(&plan, fp8_input, fp8_weight, rows, input_width, output_width, 1);
  if (status != 0)
    return status;
  int *error_word = device_error_word();
  if (error_word == nullptr) {
    set_last_error("device error word is unavailable");
    return -101;
  }
  auto *keys = static_cast<unsigned long long *>(device_keys);
  const auto cuda_stream = static_cast<cudaStream_t>(stream);
  status = check_cuda(cudaMemsetAsync(keys, 0, sizeof(unsigned long long) * rows, cuda_stream),
                      "clear argmax keys");
  if (status != 0)
    return status;
  status = launch_linear_argmax(plan, device_input_scale, device_weight_scale, keys, error_word,
                                cuda_stream);
  if (status != 0)
    return launch_status(status, "FP8 LM head");
  return launch_status(launch_unpack_best(keys, device_tokens, rows, cuda_stream),
                       "argmax unpack");
}

// gate_up linear with GeGLU in the epilogue -----------------------------------------------------

namespace {
constexpr size_t gated_counter_bytes = 256;   // the grid barrier's word, on a line of its own

size_t gated_tail_bytes(int rows, int input_width, int gated_width, int element_bytes) {
  if (rows <= 0 || rows > 256 || input_width <= 0 || gated_width <= 0)
    return 0;
  LinearPlan plan{};
  schedule_linear_shape(&plan, rows, input_width, 2 * gated_width, 1, element_bytes);
  return (linear_tail_bytes(plan) + 255) / 256 * 256;
}
} // namespace

extern "C" size_t carat_b200_fp8_linear_geglu_workspace_bytes(int rows, int input_width,
                                                              int gated_width) {
  return gated_tail_bytes(rows, input_width, gated_width, 1) + gated_counter_bytes;
}

extern "C" int carat_b200_fp8_linear_geglu(const void *fp8_input, const float *device_input_scale,
                                           const void *fp8_weight,
                                           const float *device_weight_scale, void *bf16_activated,
                                           unsigned int *device_amax_bits, void *fp8_output,
                                           float *device_output_scale, int rows, int input_width,
                                           int gated_width, void *workspace,
                                           size_t workspace_bytes, void *stream) {
  if (device_input_scale == nullptr || device_weight_scale == nullptr ||
      bf16_activated == nullptr || device_amax_bits == nullptr ||
      (fp8_output != nullptr && device_output_scale == nullptr)) {
    set_last_error("invalid FP8 linear shape");
    return -1;
  }
  LinearPlan plan;
  const char *message = "invalid FP8 linear shape";
  int status = make_gated_linear_plan(&plan, fp8_input, fp8_weight, rows, input_width, gated_width,
                                      &message, 1);
  if (status != 0) {
    set_last_error(message);
    return status;
  }
  const size_t tail_bytes = gated_tail_bytes(rows, input_width, gated_width, 1);
  if (workspace == nullptr || workspace_bytes < tail_bytes + gated_counter_bytes) {
    set_last_error("FP8 linear workspace is too small");
    return -6;
  }
  int *error_word = device_error_word();
  if (error_word == nullptr) {
    set_last_error("device error word is unavailable");
    return -101;
  }
  const auto cuda_stream = static_cast<cudaStream_t>(stream);
  auto *counter =
      reinterpret_cast<unsigned int *>(static_cast<unsigned char *>(workspace) + tail_bytes);
  status = check_cuda(cudaMemsetAsync(counter, 0, gated_counter_bytes, cuda_stream),
                      "clear grid counter");
  if (status == 0)
    status = check_cuda(cudaMemsetAsync(device_amax_bits, 0, sizeof(unsigned int), cuda_stream),
                        "clear activation maximum");
  if (status != 0)
    return status;
  status = launch_linear_gated(plan, device_input_scale, device_weight_scale, bf16_activated,
                               device_amax_bits, fp8_output, device_output_scale,
                               static_cast<float *>(workspace), counter, error_word, cuda_stream);
  return launch_status(status, "FP8 gated linear");
}

extern "C" int carat_b200_fp8_linear_check(const void *fp8_input, const float *device_input_scale,
                                           const void *fp8_weight,
                                           const float *device_weight_scale, void *bf16_output,
                                           int rows, int input_width, int output_width,
                                           void *stream) {
  if (fp8_input == nullptr || fp8_weight == nullptr || device_input_scale == nullptr ||
      device_weight_scale == nullptr || bf16_output == nullptr || rows <= 0 || input_width <= 0 ||
      output_width <= 0) {
    set_last_error("invalid FP8 linear shape");
    return -1;
  }
  return launch_status(launch_linear_simt_check(fp8_input, device_input_scale, fp8_weight,
                                                device_weight_scale, bf16_output, rows,
                                                input_width, output_width,
                                                static_cast<cudaStream_t>(stream)),
                       "FP8 linear check");
}

// BF16 linear (the same weight-streaming kernel with 16-bit operands) ----------------------------

extern "C" size_t carat_b200_bf16_linear_workspace_bytes(int rows, int input_width,
                                                         int output_width) {
  return linear_partial_bytes_for(rows, input_width, output_width, 2);
}

extern "C" int carat_b200_bf16_linear(const void *bf16_input, const void *bf16_weight,
                                      void *bf16_output, int rows, int input_width,
                                      int output_width, void *workspace, size_t workspace_bytes,
                                      void *stream) {
  if (bf16_output == nullptr) {
    set_last_error("invalid BF16 linear shape");
    return -1;
  }
  LinearPlan plan;
  int status = plan_or_fail(&plan, bf16_input, bf16_weight, rows, input_width, output_width, 0, 2);
  if (status != 0) {
    set_last_error("invalid BF16 linear shape");
    return status;
  }
  const size_t needed = linear_partial_bytes(plan);
  if (needed > 0 && (workspace == nullptr || workspace_bytes < needed)) {
    set_last_error("BF16 linear workspace is too small");
    return -6;
  }
  int *error_word = device_error_word();
  if (error_word == nullptr) {
    set_last_error("device error word is unavailable");
    return -101;
  }
  status = launch_linear_bf16(plan, nullptr, nullptr, bf16_output, static_cast<float *>(workspace),
                              error_word, static_cast<cudaStream_t>(stream));
  return launch_status(status, "BF16 linear");
}

extern "C" int carat_b200_bf16_linear_argmax(const void *bf16_input, const void *bf16_weight,
                                             int *device_tokens, void *device_keys, int rows,
                                             int input_width, int output_width, void *stream) {
  if (device_tokens == nullptr || device_keys == nullptr) {
    set_last_error("invalid BF16 linear shape");
    return -1;
  }
  LinearPlan plan;
  int status = plan_or_fail(&plan, bf16_input, bf16_weight, rows, input_width, output_width, 1, 2);
  if (status != 0) {
    set_last_error("invalid BF16 linear shape");
    return status;
  }
  int *error_word = device_error_word();
  if (error_word == nullptr) {
    set_last_error("device error word is unavailable");
    return -101;
  }
  auto *keys = static_cast<unsigned long long *>(device_keys);
  const auto cuda_stream = static_cast<cudaStream_t>(stream);
  status = check_cuda(cudaMemsetAsync(keys, 0, sizeof(unsigned long long) * rows, cuda_stream),
                      "clear argmax keys");
  if (status != 0)
    return status;
  status = launch_linear_argmax(plan, nullptr, nullptr, keys, error_word, cuda_stream);
  if (status != 0)
    return launch_status(status, "BF16 LM head");
  return launch_status(launch_unpack_best(keys, device_tokens, rows, cuda_stream),
                       "argmax unpack");
}

// INT4 weight-only linear ---------------------------------------------------------------------

namespace {

bool int4_shape_ok(int output_width, int input_width, int group_width) {
  return output_width > 0 && input_width > 0 && (group_width == 128 || group_width == 256) &&
         input_width % group_width == 0;
}

} // namespace

extern "C" int carat_b200_int4_quantize_weight(const void *bf16_weight, void *packed_row_major,
                                               void *bf16_scales, int output_width,
                                               int input_width, int group_width, void *stream) {
  if (bf16_weight == nullptr || packed_row_major == nullptr || bf16_scales == nullptr ||
      !int4_shape_ok(output_width, input_width, group_width)) {
    set_last_error("invalid BF16 INT4 linear weight shape");
    return -1;
  }
  return launch_status(launch_int4_quantize(bf16_weight, packed_row_major, bf16_scales,
                                            output_width, input_width, group_width,
                                            static_cast<cudaStream_t>(stream)),
                       "INT4 weight quantization");
}

extern "C" int carat_b200_int4_reorder_weight(const void *packed_row_major, void *reordered,
                                              int output_width, int input_width, void *stream) {
  if (packed_row_major == nullptr || reordered == nullptr || output_width <= 0 ||
      input_width <= 0 || input_width % 8 != 0) {
    set_last_error("invalid BF16 INT4 linear weight shape");
    return -1;
  }
  const size_t bytes = static_cast<size_t>(output_width) * input_width / 2;
  return launch_status(launch_int4_reorder(packed_row_major, reordered, bytes,
                                           static_cast<cudaStream_t>(stream)),
                       "INT4 weight reordering");
}

extern "C" size_t carat_b200_int4_linear_workspace_bytes(int rows, int input_width,
                                                         int output_width) {
  return int4_linear_partial_bytes_for(rows, input_width, output_width);
}

extern "C" int carat_b200_int4_linear(const void *bf16_input, const void *reordered_weight,
                                      const void *bf16_scales, void *bf16_output, int rows,
                                      int input_width, int output_width, int group_width,
                                      void *workspace, size_t workspace_bytes, void *stream) {
  if (bf16_output == nullptr) {
    set_last_error("invalid BF16 INT4 linear activation shape");
    return -1;
  }
  Int4LinearPlan plan;
  const char *message = "invalid BF16 INT4 linear weight shape";
  int status = make_int4_linear_plan(&plan, bf16_input, reordered_weight, bf16_scales, rows,
                                     input_width, output_width, group_width, 0, &message);
  if (status != 0) {
    set_last_error(message);
    return status;
  }
  const size_t needed = int4_linear_partial_bytes(plan);
  if (needed > 0 && (workspace == nullptr || workspace_bytes < needed)) {
    set_last_error("BF16 INT4 linear workspace is too small");
    return -6;
  }
  int *error_word = device_error_word();
  if (error_word == nullptr) {
    set_last_error("device error word is unavailable");
    return -101;
  }
  status = launch_int4_linear_bf16(plan, bf16_output, static_cast<float *>(workspace), error_word,
                                   static_cast<cudaStream_t>(stream));
  return launch_status(status, "BF16 INT4 linear");
}

extern "C" int carat_b200_int4_linear_check(const void *bf16_input, const void *packed_row_major,
                                            const void *bf16_scales, void *bf16_output, int rows,
                                            int input_width, int output_width, int group_width,
                                            void *stream) {
  if (bf16_input == nullptr || packed_row_major == nullptr || bf16_scales == nullptr ||
      bf16_output == nullptr || rows <= 0 || !int4_shape_ok(output_width, input_width, group_width)) {
    set_last_error("invalid BF16 INT4 linear weight shape");
    return -1;
  }
  return launch_status(launch_int4_linear_simt_check(bf16_input, packed_row_major, bf16_scales,
                                                     bf16_output, rows, input_width, output_width,
                                                     group_width,
                                                     static_cast<cudaStream_t>(stream)),
                       "BF16 INT4 linear check");
}
