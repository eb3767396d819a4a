#include "accept.cuh"
#include "fp8_linear.cuh"
#include "launch.cuh"

#include <cuda_bf16.h>

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

// Rollback primitive, both directions in one kernel: CTA (head, request) moves whole rows of
// `dimension` bf16 as 16-byte vectors between the ring rows (position + token) % capacity of that
// request's cache [heads, capacity, dimension] and the packed span [request][head][token]
// [dimension]. restore = false saves the span; restore = true writes back the tokens from
// accepted[request] on (the rejected suffix) and leaves accepted rows alone.
template <bool restore>
__global__ void ring_span_kernel(__nv_bfloat16 *const *key_caches,
                                 __nv_bfloat16 *const *value_caches, __nv_bfloat16 *span_keys,
                                 __nv_bfloat16 *span_values, const int *positions,
                                 const int *accepted, int heads, int tokens, int dimension,
                                 int capacity) {
  const int head = static_cast<int>(blockIdx.x);
  const int request = static_cast<int>(blockIdx.y);
  const int first_token = restore ? min(max(accepted[request], 0), tokens) : 0;
  const int vectors_per_row = dimension / 8;
  const int position = positions[request];
  const size_t span_base = (static_cast<size_t>(request) * heads + head) * tokens * dimension;
  const size_t cache_base = static_cast<size_t>(head) * capacity * dimension;
  uint4 *const span[2] = {reinterpret_cast<uint4 *>(span_keys + span_base),
                          reinterpret_cast<uint4 *>(span_values + span_base)};
  __nv_bfloat16 *const cache[2] = {key_caches[request] + cache_base,
                                   value_caches[request] + cache_base};
  const int vectors = (tokens - first_token) * vectors_per_row;
  for (int index = static_cast<int>(threadIdx.x); index < vectors; index += blockDim.x) {
    const int token = first_token + index / vectors_per_row;
    const int vector = index % vectors_per_row;
    const size_t ring_row = static_cast<size_t>((position + token) % capacity);
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      uint4 *ring = reinterpret_cast<uint4 *>(cache[which] + ring_row * dimension) + vector;
      uint4 *saved = span[which] + static_cast<size_t>(token) * vectors_per_row + vector;
      if constexpr (restore)
        *ring = *saved;
      else
        *saved = *ring;
    }
  }
}

// Row argmax with the LM head's packed keys: (orderable bf16 value << 32) | ~index, so one
// unsigned maximum picks the largest value and, among equals, the lowest index; NaN orders below
// every number and an all-NaN row yields index 0.
__device__ __forceinline__ unsigned long long argmax_key(__nv_bfloat16 value, int index) {
  const unsigned int bits = __bfloat16_as_ushort(value);
  unsigned int orderable = (bits & 0x8000U) ? (~bits & 0xFFFFU) : (bits | 0x8000U);
  if ((bits & 0x7FFFU) > 0x7F80U)
    orderable = 0U;
  return (static_cast<unsigned long long>(orderable) << 32) |
         static_cast<unsigned long long>(~static_cast<unsigned int>(index));
}

__global__ void argmax_rows_kernel(const __nv_bfloat16 *values, int elements, int *output) {
  __shared__ unsigned long long warp_best[32];
  const __nv_bfloat16 *row = values + static_cast<size_t>(blockIdx.x) * elements;
  unsigned long long best = 0ULL;
  for (int index = static_cast<int>(threadIdx.x); index < elements; index += blockDim.x)
    best = max(best, argmax_key(row[index], index));
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1)
    best = max(best, __shfl_xor_sync(0xFFFFFFFFU, best, offset));
  if ((threadIdx.x & 31U) == 0U)
    warp_best[threadIdx.x >> 5U] = best;
  __syncthreads();
  if (threadIdx.x < 32U) {
    best = threadIdx.x < (blockDim.x + 31U) / 32U ? warp_best[threadIdx.x] : 0ULL;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
      best = max(best, __shfl_xor_sync(0xFFFFFFFFU, best, offset));
    if (threadIdx.x == 0U)
      output[blockIdx.x] = best_index(best);
  }
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
      a.requests <= 0 || a.depth <= 0 || a.hidden % 8 != 0) {
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
  if (head_dim % 8 != 0)
    return -1;
  ring_span_kernel<false><<<dim3(static_cast<unsigned>(heads), static_cast<unsigned>(requests)),
                            128, 0, stream>>>(
      reinterpret_cast<__nv_bfloat16 *const *>(const_cast<void *const *>(key_sources)),
      reinterpret_cast<__nv_bfloat16 *const *>(const_cast<void *const *>(value_sources)),
      static_cast<__nv_bfloat16 *>(backup_keys), static_cast<__nv_bfloat16 *>(backup_values),
      positions, nullptr, heads, tokens, head_dim, capacity);
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
  if (head_dim % 8 != 0)
    return -1;
  ring_span_kernel<true><<<dim3(static_cast<unsigned>(heads), static_cast<unsigned>(requests)),
                           128, 0, stream>>>(
      reinterpret_cast<__nv_bfloat16 *const *>(key_destinations),
      reinterpret_cast<__nv_bfloat16 *const *>(value_destinations),
      static_cast<__nv_bfloat16 *>(const_cast<void *>(backup_keys)),
      static_cast<__nv_bfloat16 *>(const_cast<void *>(backup_values)), positions, accepted, heads,
      tokens, head_dim, capacity);
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
