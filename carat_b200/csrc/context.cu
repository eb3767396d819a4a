#include "context.cuh"

#include <map>
#include <mutex>

namespace carat_b200 {
namespace {

thread_local std::string last_error_storage;
std::mutex device_words_mutex;
std::map<int, int *> device_words;
std::map<int, int *> extra_words;
PerDevice<int> multiprocessor_counts;

} // namespace

void set_last_error(const std::string &message) { last_error_storage = message; }

const char *last_error_text() { return last_error_storage.c_str(); }

int check_cuda(cudaError_t result, const char *operation) {
  if (result == cudaSuccess)
    return 0;
  set_last_error(std::string(operation) + ": " + cudaGetErrorString(result));
  return -100;
}

int current_device() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= maximum_devices)
    return -1;
  return device;
}

int device_multiprocessors() {
  int *slot = multiprocessor_counts.slot();
  if (slot == nullptr)
    return 148;
  std::lock_guard<std::mutex> lock(multiprocessor_counts.lock());
  if (*slot <= 0) {
    int value = 0;
    if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, current_device()) !=
            cudaSuccess ||
        value <= 0) {
      return 148;
    }
    *slot = value;
  }
  return *slot;
}

void register_extra_error_word(int *word) {
  const int device = current_device();
  if (device < 0)
    return;
  std::lock_guard<std::mutex> lock(device_words_mutex);
  extra_words[device] = word;
}

int *device_error_word() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess)
    return nullptr;
  std::lock_guard<std::mutex> lock(device_words_mutex);
  const auto found = device_words.find(device);
  if (found != device_words.end())
    return found->second;
  int *word = nullptr;
  if (cudaMalloc(&word, sizeof(int)) != cudaSuccess)
    return nullptr;
  if (cudaMemset(word, 0, sizeof(int)) != cudaSuccess) {
    cudaFree(word);
    return nullptr;
  }
  device_words[device] = word;
  return word;
}

int read_and_clear_device_error(int *value) {
  int *word = device_error_word();
  if (word == nullptr) {
    set_last_error("device error word is unavailable");
    return -101;
  }
  int host = 0;
  int status = check_cuda(cudaMemcpy(&host, word, sizeof(int), cudaMemcpyDeviceToHost),
                          "read device error word");
  if (status != 0)
    return status;
  if (host != 0) {
    status = check_cuda(cudaMemset(word, 0, sizeof(int)), "clear device error word");
    if (status != 0)
      return status;
  }
  int *extra = nullptr;
  {
    std::lock_guard<std::mutex> lock(device_words_mutex);
    const auto found = extra_words.find(current_device());
    if (found != extra_words.end())
      extra = found->second;
  }
  if (extra != nullptr) {
    int extra_host = 0;
    status = check_cuda(cudaMemcpy(&extra_host, extra, sizeof(int), cudaMemcpyDeviceToHost),
                        "read static error word");
    if (status != 0)
      return status;
    if (extra_host != 0) {
      status = check_cuda(cudaMemset(extra, 0, sizeof(int)), "clear static error word");
      if (status != 0)
        return status;
      if (host == 0)
        host = extra_host;
    }
  }
  if (value != nullptr)
    *value = host;
  return 0;
}

} // namespace carat_b200
