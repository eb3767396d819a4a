// FP8 linear for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a linear: a
// latency-critical serving loop whose allocator is frozen once the model is loaded, and plugins
// that are handed a fixed memory budget by their framework and are forbidden to grow it.
// carat_b200_fp8_linear needs a caller-provided workspace for its split-K partial sums; this
// variant keeps that workspace in a fixed array inside the library image instead, so the caller
// passes inputs and outputs only and the call performs no allocation of any kind.
#include "../../include/carat_b200.h"
#include "context.cuh"
#include "fp8_linear.cuh"

#include <mutex>

using namespace carat_b200;

namespace {

// 8 MiB of fp32 partial sums: [splits, rows, output_width]. Every GPU that loads the library
// holds this array until the process exits.
constexpr size_t static_partial_floats = 2U * 1024U * 1024U;

static __device__ __align__(256) float static_partials[static_partial_floats];
// The kernels record here when one of their bounded waits runs out (0 = healthy). Kept inside the
// image for the same reason as the partial sums. The launch path never reads it back (that would
// synchronise the device); carat_b200_device_error() reads and clears it together with the
// library's other error word.
static __device__ __align__(256) int static_error_word[64];

struct DeviceScratch {
  float *partials{nullptr};
  int *error_word{nullptr};
  bool ready{false};
};

std::mutex scratch_mutex;
DeviceScratch scratch_by_device[maximum_devices];

// In host code `static_partials` names a host-side stand-in for the device array, not a device
// address: the address a kernel can use has to be asked for, once per device, with that device
// current.
int scratch_for_current_device(DeviceScratch *result) {
  int device = 0;
  int status = check_cuda(cudaGetDevice(&device), "get current device");
  if (status != 0)
    return status;
  if (device < 0 || device >= maximum_devices) {
    set_last_error("device index is beyond what the no-allocation FP8 linear supports");
    return -20;
  }
  std::lock_guard<std::mutex> lock(scratch_mutex);
  DeviceScratch &entry = scratch_by_device[device];
  if (!entry.ready) {
    void *partials = nullptr;
    void *error_word = nullptr;
    status = check_cuda(cudaGetSymbolAddress(&partials, static_partials),
                        "look up the static split-K scratch");
    if (status != 0)
      return status;
    status = check_cuda(cudaGetSymbolAddress(&error_word, static_error_word),
                        "look up the static error word");
    if (status != 0)
      return status;
    entry.partials = static_cast<float *>(partials);
    entry.error_word = static_cast<int *>(error_word);
    entry.ready = true;
    register_extra_error_word(entry.error_word);
  }
  *result = entry;
  return 0;
}

} // namespace

static_assert(static_partial_floats * sizeof(float) == CARAT_B200_STATIC_SCRATCH_BYTES,
              "the header states the size of the built-in scratch");

extern "C" int carat_b200_fp8_linear_static(const void *fp8_input, const float *device_input_scale,
                                            const void *fp8_weight,
                                            const float *device_weight_scale, void *bf16_output,
                                            int rows, int input_width, int output_width,
                                            void *stream) {
  if (device_input_scale == nullptr || device_weight_scale == nullptr || bf16_output == nullptr) {
    set_last_error("invalid FP8 linear shape");
    return -1;
  }
  LinearPlan plan;
  const char *message = "invalid FP8 linear shape";
  int status = make_linear_plan(&plan, fp8_input, fp8_weight, rows, input_width, output_width, 0,
                                &message);
  if (status != 0) {
    set_last_error(message);
    return status;
  }
  if (linear_partial_bytes(plan) > static_partial_floats * sizeof(float)) {
    set_last_error("FP8 linear needs " + std::to_string(linear_partial_bytes(plan)) +
                   " bytes of split-K scratch, more than the " +
                   std::to_string(static_partial_floats * sizeof(float)) +
                   " bytes built into the library; use carat_b200_fp8_linear with a workspace");
    return -6;
  }
  DeviceScratch scratch;
  status = scratch_for_current_device(&scratch);
  if (status != 0)
    return status;
  status = launch_linear_bf16(plan, device_input_scale, device_weight_scale, bf16_output,
                              scratch.partials, scratch.error_word,
                              static_cast<cudaStream_t>(stream));
  if (status != 0) {
    set_last_error(std::string("FP8 linear launch failed: ") +
                   cudaGetErrorString(cudaGetLastError()));
  }
  return status;
}
