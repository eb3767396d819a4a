// Process-wide pieces shared by the C entry points: last-error text and the per-device error word
// that kernels with bounded waits write when a wait runs out.
#pragma once

#include <cuda_runtime.h>

#include <mutex>
#include <string>

namespace carat_b200 {

// Function attributes (dynamic shared memory), occupancy figures, multiprocessor counts and
// library-owned scratch are all per device, so everything cached lazily is keyed by the device
// that is current at the call, never once per process.
constexpr int maximum_devices = 64;

// Ordinal of the current device, or -1 when it cannot be read or is beyond maximum_devices.
int current_device();

// Multiprocessor count of the current device (cached per device); 148 when the query fails.
int device_multiprocessors();

// A configuration step that must run once per device: run(body) calls body() the first time it
// is reached with a given device current and returns that call's status ever after.
class PerDeviceOnce {
public:
  template <typename Body> cudaError_t run(Body &&body) {
    const int device = current_device();
    if (device < 0)
      return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mutex_);
    if (!done_[device]) {
      status_[device] = body();
      done_[device] = true;
    }
    return status_[device];
  }

private:
  std::mutex mutex_;
  bool done_[maximum_devices]{};
  cudaError_t status_[maximum_devices]{};
};

// One lazily-made value per device (a scratch pointer, an occupancy limit).
template <typename T> class PerDevice {
public:
  // Slot of the current device, or nullptr. The caller holds lock() while it reads or changes it.
  T *slot() {
    const int device = current_device();
    return device < 0 ? nullptr : &values_[device];
  }
  std::mutex &lock() { return mutex_; }

private:
  std::mutex mutex_;
  T values_[maximum_devices]{};
};

// Thread-local message returned by carat_b200_last_error().
void set_last_error(const std::string &message);
const char *last_error_text();

// Records `operation: cuda error string` and returns -100 when result is not cudaSuccess.
int check_cuda(cudaError_t result, const char *operation);

// Device pointer to a zero-initialised int for the current device (allocated on first use).
// Kernels write a non-zero code into it when a bounded wait gives up.
int *device_error_word();

// A second word on the current device that read_and_clear_device_error() also reads and clears
// (the no-allocation linear keeps its own inside the library image).
void register_extra_error_word(int *word);

// Reads the error words of the current device back (synchronises the device) and clears them;
// *value is the first non-zero code.
int read_and_clear_device_error(int *value);

} // namespace carat_b200
