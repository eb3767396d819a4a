// Process-wide pieces shared by the C entry points: last-error text and the per-device error word
// that kernels with bounded waits write when a wait runs out.
#pragma once

#include <cuda_runtime.h>

#include <string>

namespace carat_b200 {

// Thread-local message returned by carat_b200_last_error().
void set_last_error(const std::string &message);
const char *last_error_text();

// Records `operation: cuda error string` and returns -100 when result is not cudaSuccess.
int check_cuda(cudaError_t result, const char *operation);

// Device pointer to a zero-initialised int for the current device (allocated on first use).
// Kernels write a non-zero code into it when a bounded wait gives up.
int *device_error_word();

// Reads the error word of the current device back (synchronises the device) and clears it.
int read_and_clear_device_error(int *value);

} // namespace carat_b200
