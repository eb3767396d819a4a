#include "accept.cuh"
#include "fp8_linear.cuh"
#include "launch.cuh"

#include <cuda_bf16.h>
#include <math_constants.h>

namespace carat_b200 {
namespace {

__global__ void accept_kernel(AcceptArguments a) {
  __shared__ int shared_accepted;
  grid_dependency_launch();
  grid_dependency_wait();
  const int request = static_cast<int>(blockIdx.x);
  const int start = request * a.depth;
  if (threadIdx.x == 0) {
    int cap = a.depth;
    if (a.caps != nullptr)
      cap = min(max(a.caps[request], 0), a.depth);
    int accepted = 0;
    while (accepted < cap) {
      const int expected = accepted == 0 ? a.target_first[request]
                                         : best_index(a.best[start + accepted - 1]);
      if (!a.assume_match && a.proposals[start + accepted] != expected)
        break;
      ++accepted;
    }
    a.accepted[request] = accepted;
    a.next_tokens[request] =
        accepted == 0 ? a.target_first[request] : best_index(a.best[start + accepted - 1]);
    a.slot_positions[a.slots[request]] += accepted;
    shared_accepted = accepted;
  }
  for (int token = static_cast<int>(threadIdx.x); token < a.depth; token += blockDim.x)
    a.predictions[start + token] = best_index(a.best[start + token]);
  __syncthreads();
  const int accepted = shared_accepted;
  if (accepted == 0)
    return;
  const auto *source = static_cast<const __nv_bfloat16 *>(a.final_hidden) +
                       static_cast<size_t>(start + accepted - 1) * a.hidden;
  auto *destination =
      static_cast<__nv_bfloat16 *>(a.hidden_by_slot) + static_cast<size_t>(a.slots[request]) * a.hidden;
  for (int column = static_cast<int>(threadIdx.x) * 8; column < a.hidden; column += blockDim.x * 8)
    *reinterpret_cast<uint4 *>(destination + column) =
        *reinterpret_cast<const uint4 *>(source + column);
}

__global__ void commit_kernel(const CommitLayer *layers, const int *positions, const int *accepted,
                              const int *slots, int depth) {
  grid_dependency_launch();
  grid_dependency_wait();
  const CommitLayer layer = layers[blockIdx.y];
  const int request = static_cast<int>(blockIdx.x);
  const int limit = min(accepted[request], depth);
  const int chunks_per_row = layer.head_dim / 8;
  const int total = layer.kv_heads * limit * chunks_per_row;
  const int position = positions[request];
  const int slot = slots[request];
  for (int index = static_cast<int>(threadIdx.x); index < total; index += blockDim.x) {
    const int chunk = index % chunks_per_row;
    const int token = (index / chunks_per_row) % limit;
    const int head = index / (chunks_per_row * limit);
    const size_t source =
        ((static_cast<size_t>(request) * layer.kv_heads + head) * depth + token) * layer.head_dim +
        chunk * 8;
    const size_t destination = static_cast<size_t>(slot * layer.slot_stride + head * layer.head_stride) +
                               static_cast<size_t>((position + token) % layer.capacity) * layer.head_dim +
                               chunk * 8;
    *reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(layer.key_cache) + destination) =
        *reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(layer.staged_keys) + source);
    *reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(layer.value_cache) + destination) =
        *reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(layer.staged_values) + source);
  }
}

__global__ void backup_kernel(const __nv_bfloat16 *const *key_sources,
                              const __nv_bfloat16 *const *value_sources, __nv_bfloat16 *backup_keys,
                              __nv_bfloat16 *backup_values, const int *positions, int requests,
                              int heads, int tokens, int dimension, int capacity) {
  const long long index = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long request_elements = static_cast<long long>(heads) * tokens * dimension;
  if (index >= requests * request_elements)
    return;
  const int request = static_cast<int>(index / request_elements);
  const long long local = index % request_elements;
  const int component = static_cast<int>(local % dimension);
  const int token = static_cast<int>((local / dimension) % tokens);
  const int head = static_cast<int>(local / (static_cast<long long>(dimension) * tokens));
  const size_t source =
      (static_cast<size_t>(head) * capacity + (positions[request] + token) % capacity) * dimension +
      component;
  backup_keys[index] = key_sources[request][source];
  backup_values[index] = value_sources[request][source];
}

__global__ void restore_kernel(const __nv_bfloat16 *backup_keys, const __nv_bfloat16 *backup_values,
                               __nv_bfloat16 *const *key_destinations,
                               __nv_bfloat16 *const *value_destinations, const int *positions,
                               const int *accepted, int requests, int heads, int tokens,
                               int dimension, int capacity) {
  const long long index = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long request_elements = static_cast<long long>(heads) * tokens * dimension;
  if (index >= requests * request_elements)
    return;
  const int request = static_cast<int>(index / request_elements);
  const long long local = index % request_elements;
  const int component = static_cast<int>(local % dimension);
  const int token = static_cast<int>((local / dimension) % tokens);
  if (token < accepted[request])
    return;
  const int head = static_cast<int>(local / (static_cast<long long>(dimension) * tokens));
  const size_t destination =
      (static_cast<size_t>(head) * capacity + (positions[request] + token) % capacity) * dimension +
      component;
  key_destinations[request][destination] = backup_keys[index];
  value_destinations[request][destination] = backup_values[index];
}

struct Best {
  float value;
  int index;
};

__device__ __forceinline__ Best better(Best left, Best right) {
  return right.value > left.value || (right.value == left.value && right.index < left.index) ? right
                                                                                             : left;
}

__global__ void argmax_rows_kernel(const __nv_bfloat16 *values, int elements, int *output) {
  __shared__ Best reduction[256];
  const __nv_bfloat16 *row = values + static_cast<size_t>(blockIdx.x) * elements;
  Best current{-CUDART_INF_F, 0};
  for (int index = static_cast<int>(threadIdx.x); index < elements; index += 256)
    current = better(current, {__bfloat162float(row[index]), index});
  reduction[threadIdx.x] = current;
  __syncthreads();
  for (int stride = 128; stride > 0; stride >>= 1) {
    if (static_cast<int>(threadIdx.x) < stride)
      reduction[threadIdx.x] = better(reduction[threadIdx.x], reduction[threadIdx.x + stride]);
    __syncthreads();
  }
  if (threadIdx.x == 0)
    output[blockIdx.x] = reduction[0].index;
}

__global__ void move_rows_kernel(const __nv_bfloat16 *input, const int *indices,
                                 __nv_bfloat16 *output, int width, bool gather) {
  const int row = static_cast<int>(blockIdx.x);
  const size_t source = static_cast<size_t>(gather ? indices[row] : row) * width;
  const size_t destination = static_cast<size_t>(gather ? row : indices[row]) * width;
  for (int column = static_cast<int>(threadIdx.x); column < width; column += blockDim.x)
    output[destination + column] = input[source + column];
}

int launched() { return cudaPeekAtLastError() == cudaSuccess ? 0 : -11; }

} // namespace

int launch_accept(const AcceptArguments &a, cudaStream_t stream) {
  if (a.best == nullptr || a.proposals == nullptr || a.target_first == nullptr ||
      a.accepted == nullptr || a.next_tokens == nullptr || a.predictions == nullptr ||
      a.final_hidden == nullptr || a.hidden_by_slot == nullptr || a.slots == nullptr ||
      a.slot_positions == nullptr || a.requests <= 0 || a.depth <= 0 || a.hidden % 8 != 0) {
    return -1;
  }
  launch_chained(accept_kernel, dim3(static_cast<unsigned>(a.requests)), dim3(256), 0, stream, false, a);
  return launched();
}

int launch_commit(const CommitLayer *device_layers, int layers, const int *positions,
                  const int *accepted, const int *slots, int requests, int depth,
                  int max_row_elements, cudaStream_t stream) {
  (void)max_row_elements;
  if (layers == 0)
    return 0;
  if (device_layers == nullptr || positions == nullptr || accepted == nullptr || slots == nullptr ||
      requests <= 0 || depth <= 0)
    return -1;
  launch_chained(commit_kernel, dim3(static_cast<unsigned>(requests), static_cast<unsigned>(layers)),
                 dim3(256), 0, stream, false, device_layers, positions, accepted, slots, depth);
  return launched();
}

int launch_backup_kv_ring_spans(const void *const *key_sources, const void *const *value_sources,
                                void *backup_keys, void *backup_values, const int *positions,
                                int requests, int heads, int tokens, int head_dim, int capacity,
                                cudaStream_t stream) {
  if (key_sources == nullptr || value_sources == nullptr || backup_keys == nullptr ||
      backup_values == nullptr || positions == nullptr || requests <= 0 || heads <= 0 ||
      tokens <= 0 || head_dim <= 0 || capacity <= 0) {
    return -1;
  }
  const long long elements = static_cast<long long>(requests) * heads * tokens * head_dim;
  backup_kernel<<<static_cast<unsigned>((elements + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16 *const *>(key_sources),
      reinterpret_cast<const __nv_bfloat16 *const *>(value_sources),
      static_cast<__nv_bfloat16 *>(backup_keys), static_cast<__nv_bfloat16 *>(backup_values),
      positions, requests, heads, tokens, head_dim, capacity);
  return launched();
}

int launch_restore_kv_ring_suffixes(const void *backup_keys, const void *backup_values,
                                    void *const *key_destinations,
                                    void *const *value_destinations, const int *positions,
                                    const int *accepted, int requests, int heads, int tokens,
                                    int head_dim, int capacity, cudaStream_t stream) {
  if (backup_keys == nullptr || backup_values == nullptr || key_destinations == nullptr ||
      value_destinations == nullptr || positions == nullptr || accepted == nullptr ||
      requests <= 0 || heads <= 0 || tokens <= 0 || head_dim <= 0 || capacity <= 0) {
    return -1;
  }
  const long long elements = static_cast<long long>(requests) * heads * tokens * head_dim;
  restore_kernel<<<static_cast<unsigned>((elements + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16 *>(backup_keys),
      static_cast<const __nv_bfloat16 *>(backup_values),
      reinterpret_cast<__nv_bfloat16 *const *>(key_destinations),
      reinterpret_cast<__nv_bfloat16 *const *>(value_destinations), positions, accepted, requests,
      heads, tokens, head_dim, capacity);
  return launched();
}

int launch_argmax_bf16_rows(const void *values, int rows, int elements, int *output,
                            cudaStream_t stream) {
  if (values == nullptr || output == nullptr || rows <= 0 || elements <= 0)
    return -1;
  argmax_rows_kernel<<<rows, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(values),
                                               elements, output);
  return launched();
}

int launch_gather_rows(const void *input, const int *indices, void *output, int rows, int width,
                       cudaStream_t stream) {
  if (input == nullptr || indices == nullptr || output == nullptr || rows <= 0 || width <= 0)
    return -1;
  move_rows_kernel<<<rows, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(input), indices,
                                             static_cast<__nv_bfloat16 *>(output), width, true);
  return launched();
}

int launch_scatter_rows(const void *input, const int *indices, void *output, int rows, int width,
                        cudaStream_t stream) {
  if (input == nullptr || indices == nullptr || output == nullptr || rows <= 0 || width <= 0)
    return -1;
  move_rows_kernel<<<rows, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(input), indices,
                                             static_cast<__nv_bfloat16 *>(output), width, false);
  return launched();
}

} // namespace carat_b200
