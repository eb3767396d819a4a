#include "qkv_post.cuh"

#include "launch.cuh"

#include <cuda_bf16.h>

namespace carat_b200 {
namespace {

__global__ void rope_table_kernel(__nv_bfloat16 *cosine, __nv_bfloat16 *sine, int positions,
                                  int dimension, float theta, bool proportional) {
  const int index = static_cast<int>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (index >= positions * dimension)
    return;
  const int position = index / dimension;
  const int half_index = index % (dimension / 2);
  float frequency = 0.0F;
  if (!proportional || half_index < dimension / 8)
    frequency = powf(theta, -2.0F * static_cast<float>(half_index) / dimension);
  float sin_value = 0.0F;
  float cos_value = 0.0F;
  sincosf(static_cast<float>(position) * frequency, &sin_value, &cos_value);
  cosine[index] = __float2bfloat16_rn(cos_value);
  sine[index] = __float2bfloat16_rn(sin_value);
}

__device__ __forceinline__ float warp_sum(float value) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1)
    value += __shfl_xor_sync(0xFFFFFFFFU, value, offset);
  return value;
}

// One warp per (row, head). A lane owns `per` consecutive elements of the first half of the head
// vector and the elements at the same offsets of the second half, so rotate-half partners live in
// the same thread.
template <int per>
__device__ __forceinline__ void load_halves(const __nv_bfloat16 *vector, int lane, float (&low)[per],
                                            float (&high)[per]) {
  constexpr int dimension = per * 64;
#pragma unroll
  for (int index = 0; index < per; ++index) {
    low[index] = __bfloat162float(vector[lane * per + index]);
    high[index] = __bfloat162float(vector[dimension / 2 + lane * per + index]);
  }
}

template <int per>
__device__ __forceinline__ void norm_rope_store(const float (&low)[per], const float (&high)[per],
                                                float inverse_rms, const __nv_bfloat16 *weight,
                                                const __nv_bfloat16 *cosine,
                                                const __nv_bfloat16 *sine, int lane,
                                                __nv_bfloat16 *output) {
  constexpr int dimension = per * 64;
#pragma unroll
  for (int index = 0; index < per; ++index) {
    const int first = lane * per + index;
    const int second = dimension / 2 + first;
    const float low_normalized = __bfloat162float(
        __float2bfloat16_rn(low[index] * inverse_rms * __bfloat162float(weight[first])));
    const float high_normalized = __bfloat162float(
        __float2bfloat16_rn(high[index] * inverse_rms * __bfloat162float(weight[second])));
    output[first] = __float2bfloat16_rn(low_normalized * __bfloat162float(cosine[first]) +
                                        (-high_normalized) * __bfloat162float(sine[first]));
    output[second] = __float2bfloat16_rn(high_normalized * __bfloat162float(cosine[second]) +
                                         low_normalized * __bfloat162float(sine[second]));
  }
}

template <int per> __global__ void qkv_post_kernel(QkvPostArguments a) {
  constexpr int dimension = per * 64;
  grid_dependency_launch();
  grid_dependency_wait();
  const int warp = static_cast<int>(blockIdx.x) * (blockDim.x / 32) + (threadIdx.x / 32);
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int heads_per_row = a.query_heads + a.kv_heads;
  const int rows = a.requests * a.depth;
  if (warp >= rows * heads_per_row)
    return;
  const int row = warp / heads_per_row;
  const int head = warp % heads_per_row;
  const int request = row / a.depth;
  const int token = row % a.depth;
  const int position = a.positions[request] + token;
  if (position < 0 || position >= a.max_positions)
    return;
  const int query_width = a.query_heads * dimension;
  const int kv_width = a.kv_heads * dimension;
  const int packed_width = query_width + kv_width * (a.key_equals_value ? 1 : 2);
  const auto *packed_row =
      static_cast<const __nv_bfloat16 *>(a.packed) + static_cast<size_t>(row) * packed_width;
  const auto *cosine =
      static_cast<const __nv_bfloat16 *>(a.cosine) + static_cast<size_t>(position) * dimension;
  const auto *sine =
      static_cast<const __nv_bfloat16 *>(a.sine) + static_cast<size_t>(position) * dimension;
  float low[per];
  float high[per];
  if (head < a.query_heads) {
    load_halves<per>(packed_row + head * dimension, lane, low, high);
    float square_sum = 0.0F;
#pragma unroll
    for (int index = 0; index < per; ++index)
      square_sum += low[index] * low[index] + high[index] * high[index];
    const float inverse_rms = rsqrtf(warp_sum(square_sum) / dimension + a.epsilon);
    auto *output = static_cast<__nv_bfloat16 *>(a.queries) +
                   ((static_cast<size_t>(request) * a.query_heads + head) * a.depth + token) *
                       dimension;
    norm_rope_store<per>(low, high, inverse_rms, static_cast<const __nv_bfloat16 *>(a.query_norm),
                         cosine, sine, lane, output);
    return;
  }
  const int kv_head = head - a.query_heads;
  const long long owner = a.direct ? a.slots[request] : request;
  const int cache_row = a.direct ? position % a.capacity : token;
  const size_t destination = static_cast<size_t>(owner * a.slot_stride + kv_head * a.head_stride) +
                             static_cast<size_t>(cache_row) * dimension;
  load_halves<per>(packed_row + query_width + kv_head * dimension, lane, low, high);
  float key_square_sum = 0.0F;
#pragma unroll
  for (int index = 0; index < per; ++index)
    key_square_sum += low[index] * low[index] + high[index] * high[index];
  const float inverse_key_rms = rsqrtf(warp_sum(key_square_sum) / dimension + a.epsilon);
  norm_rope_store<per>(low, high, inverse_key_rms, static_cast<const __nv_bfloat16 *>(a.key_norm),
                       cosine, sine, lane, static_cast<__nv_bfloat16 *>(a.key_base) + destination);
  float inverse_value_rms = inverse_key_rms;
  if (!a.key_equals_value) {
    load_halves<per>(packed_row + query_width + kv_width + kv_head * dimension, lane, low, high);
    float value_square_sum = 0.0F;
#pragma unroll
    for (int index = 0; index < per; ++index)
      value_square_sum += low[index] * low[index] + high[index] * high[index];
    inverse_value_rms = rsqrtf(warp_sum(value_square_sum) / dimension + a.epsilon);
  }
  auto *value_output = static_cast<__nv_bfloat16 *>(a.value_base) + destination;
#pragma unroll
  for (int index = 0; index < per; ++index) {
    value_output[lane * per + index] = __float2bfloat16_rn(low[index] * inverse_value_rms);
    value_output[dimension / 2 + lane * per + index] =
        __float2bfloat16_rn(high[index] * inverse_value_rms);
  }
}

template <int per>
__global__ void query_post_kernel(const __nv_bfloat16 *projected, const __nv_bfloat16 *weight,
                                  const __nv_bfloat16 *cosine_table,
                                  const __nv_bfloat16 *sine_table, __nv_bfloat16 *queries,
                                  const int *positions, int position_offset, int requests,
                                  int query_heads, int max_positions, float epsilon) {
  constexpr int dimension = per * 64;
  grid_dependency_launch();
  grid_dependency_wait();
  const int warp = static_cast<int>(blockIdx.x) * (blockDim.x / 32) + (threadIdx.x / 32);
  const int lane = static_cast<int>(threadIdx.x) & 31;
  if (warp >= requests * query_heads)
    return;
  const int request = warp / query_heads;
  const int position = positions[request] + position_offset;
  if (position < 0 || position >= max_positions)
    return;
  float low[per];
  float high[per];
  load_halves<per>(projected + static_cast<size_t>(warp) * dimension, lane, low, high);
  float square_sum = 0.0F;
#pragma unroll
  for (int index = 0; index < per; ++index)
    square_sum += low[index] * low[index] + high[index] * high[index];
  const float inverse_rms = rsqrtf(warp_sum(square_sum) / dimension + epsilon);
  norm_rope_store<per>(low, high, inverse_rms, weight,
                       cosine_table + static_cast<size_t>(position) * dimension,
                       sine_table + static_cast<size_t>(position) * dimension, lane,
                       queries + static_cast<size_t>(warp) * dimension);
}

} // namespace

int launch_rope_tables(void *cosine, void *sine, int positions, int head_dim, float theta,
                       bool proportional, cudaStream_t stream) {
  if (cosine == nullptr || sine == nullptr || positions <= 0 || head_dim <= 0 || head_dim % 8 != 0)
    return -1;
  const int elements = positions * head_dim;
  rope_table_kernel<<<(elements + 255) / 256, 256, 0, stream>>>(
      static_cast<__nv_bfloat16 *>(cosine), static_cast<__nv_bfloat16 *>(sine), positions, head_dim,
      theta, proportional);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -11;
}

int launch_qkv_post(const QkvPostArguments &a, cudaStream_t stream) {
  if (a.packed == nullptr || a.query_norm == nullptr || a.key_norm == nullptr ||
      a.cosine == nullptr || a.sine == nullptr || a.queries == nullptr || a.key_base == nullptr ||
      a.value_base == nullptr || a.positions == nullptr || (a.direct && a.slots == nullptr) ||
      a.requests <= 0 || a.depth <= 0 || a.query_heads <= 0 || a.kv_heads <= 0 ||
      a.capacity <= 0) {
    return -1;
  }
  const int warps = a.requests * a.depth * (a.query_heads + a.kv_heads);
  const int blocks = (warps + 3) / 4;
  switch (a.head_dim) {
  case 64:
    launch_chained(qkv_post_kernel<1>, dim3(blocks), dim3(128), 0, stream, false, a);
    break;
  case 256:
    launch_chained(qkv_post_kernel<4>, dim3(blocks), dim3(128), 0, stream, false, a);
    break;
  case 512:
    launch_chained(qkv_post_kernel<8>, dim3(blocks), dim3(128), 0, stream, false, a);
    break;
  default:
    return -3;
  }
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -11;
}

int launch_query_post(const void *projected, const void *query_norm, const void *cosine,
                      const void *sine, void *queries, const int *positions, int position_offset,
                      int requests, int query_heads, int head_dim, int max_positions,
                      float epsilon, cudaStream_t stream) {
  if (projected == nullptr || query_norm == nullptr || cosine == nullptr || sine == nullptr ||
      queries == nullptr || positions == nullptr || requests <= 0 || query_heads <= 0) {
    return -1;
  }
  const int warps = requests * query_heads;
  const int blocks = (warps + 3) / 4;
  const auto *p = static_cast<const __nv_bfloat16 *>(projected);
  const auto *w = static_cast<const __nv_bfloat16 *>(query_norm);
  const auto *c = static_cast<const __nv_bfloat16 *>(cosine);
  const auto *s = static_cast<const __nv_bfloat16 *>(sine);
  auto *q = static_cast<__nv_bfloat16 *>(queries);
  switch (head_dim) {
  case 64:
    launch_chained(query_post_kernel<1>, dim3(blocks), dim3(128), 0, stream, false, p, w, c, s, q,
                   positions, position_offset, requests, query_heads, max_positions, epsilon);
    break;
  case 256:
    launch_chained(query_post_kernel<4>, dim3(blocks), dim3(128), 0, stream, false, p, w, c, s, q,
                   positions, position_offset, requests, query_heads, max_positions, epsilon);
    break;
  case 512:
    launch_chained(query_post_kernel<8>, dim3(blocks), dim3(128), 0, stream, false, p, w, c, s, q,
                   positions, position_offset, requests, query_heads, max_positions, epsilon);
    break;
  default:
    return -3;
  }
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -11;
}

} // namespace carat_b200
