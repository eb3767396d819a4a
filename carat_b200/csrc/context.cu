#include "context.cuh"

#include <map>
#include <mutex>

namespace carat_b200 {
namespace {

thread_local std::string last_error_storage;
std::mutex device_words_mutex;
std::map<int, int *> device_words;

} // namespace

void set_last_error(const std::string &message) { last_error_storage = message; }

const char *last_error_text() { return last_error_storage.c_str(); }

int check_cuda(cudaError_t result, const char *operation) {
  if (result == cudaSuccess)
    return 0;
  set_last_error(std::string(operation) + ": " + cudaGetErrorString(result));
  return -100;
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
  if (value != nullptr)
    *value = host;
  return 0;
}

} // namespace carat_b200
