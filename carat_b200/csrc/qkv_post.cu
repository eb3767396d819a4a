#include "qkv_post.cuh"

#include "launch.cuh"

#include <cuda_bf16.h>

#include <cstdint>
#include <type_traits>

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
// the same thread. Every vector a lane touches is `per` consecutive bf16 values, moved as one
// access (8 bytes for head_dim 256, 16 for 512), and every load of a warp's work is issued before
// its first store: the stores may alias the loads as far as the compiler knows, so a load placed
// after a store would wait for its own round trip to memory.
template <int per>
__device__ __forceinline__ void load_values(const __nv_bfloat16 *source, float (&values)[per]) {
  if constexpr (per == 8 || per == 4) {
    using Raw = typename std::conditional<per == 8, uint4, uint2>::type;
    const Raw raw = *reinterpret_cast<const Raw *>(source);
    const auto *pairs = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
    for (int index = 0; index < per / 2; ++index) {
      const float2 pair = __bfloat1622float2(pairs[index]);
      values[2 * index] = pair.x;
      values[2 * index + 1] = pair.y;
    }
  } else {
#pragma unroll
    for (int index = 0; index < per; ++index)
      values[index] = __bfloat162float(source[index]);
  }
}

template <int per>
__device__ __forceinline__ void store_values(__nv_bfloat16 *destination,
                                             const float (&values)[per]) {
  if constexpr (per == 8 || per == 4) {
    using Raw = typename std::conditional<per == 8, uint4, uint2>::type;
    Raw raw;
    auto *pairs = reinterpret_cast<__nv_bfloat162 *>(&raw);
#pragma unroll
    for (int index = 0; index < per / 2; ++index)
      pairs[index] = __floats2bfloat162_rn(values[2 * index], values[2 * index + 1]);
    *reinterpret_cast<Raw *>(destination) = raw;
  } else {
#pragma unroll
    for (int index = 0; index < per; ++index)
      destination[index] = __float2bfloat16_rn(values[index]);
  }
}

template <int per>
__device__ __forceinline__ void load_halves(const __nv_bfloat16 *vector, int lane, float (&low)[per],
                                            float (&high)[per]) {
  constexpr int dimension = per * 64;
  load_values<per>(vector + lane * per, low);
  load_values<per>(vector + dimension / 2 + lane * per, high);
}

template <int per>
__device__ __forceinline__ void store_halves(__nv_bfloat16 *vector, int lane,
                                             const float (&low)[per], const float (&high)[per]) {
  constexpr int dimension = per * 64;
  store_values<per>(vector + lane * per, low);
  store_values<per>(vector + dimension / 2 + lane * per, high);
}

template <int per> __device__ __forceinline__ float inverse_rms_of(const float (&low)[per],
                                                                   const float (&high)[per],
                                                                   float epsilon) {
  constexpr int dimension = per * 64;
  float square_sum = 0.0F;
#pragma unroll
  for (int index = 0; index < per; ++index)
    square_sum += low[index] * low[index] + high[index] * high[index];
  return rsqrtf(warp_sum(square_sum) / dimension + epsilon);
}

// RMS norm (bf16-rounded) followed by rotate-half RoPE, on values already in registers.
template <int per> struct RopeOperands {
  float weight_low[per], weight_high[per];
  float cosine_low[per], cosine_high[per];
  float sine_low[per], sine_high[per];
};

template <int per>
__device__ __forceinline__ void norm_rope(const float (&low)[per], const float (&high)[per],
                                          float inverse_rms, const RopeOperands<per> &with,
                                          float (&out_low)[per], float (&out_high)[per]) {
#pragma unroll
  for (int index = 0; index < per; ++index) {
    const float low_normalized = __bfloat162float(
        __float2bfloat16_rn(low[index] * inverse_rms * with.weight_low[index]));
    const float high_normalized = __bfloat162float(
        __float2bfloat16_rn(high[index] * inverse_rms * with.weight_high[index]));
    out_low[index] = low_normalized * with.cosine_low[index] +
                     (-high_normalized) * with.sine_low[index];
    out_high[index] = high_normalized * with.cosine_high[index] +
                      low_normalized * with.sine_high[index];
  }
}

template <int per> __global__ void qkv_post_kernel(QkvPostArguments a) {
  constexpr int dimension = per * 64;
  grid_dependency_launch();
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
  const bool is_query = head < a.query_heads;
  const int kv_head = head - a.query_heads;
  const int query_width = a.query_heads * dimension;
  const int kv_width = a.kv_heads * dimension;
  const int packed_width = query_width + kv_width * (a.key_equals_value ? 1 : 2);
  RopeOperands<per> with;
  // The norm weights are static: they are fetched while the projection still runs.
  load_halves<per>(static_cast<const __nv_bfloat16 *>(is_query ? a.query_norm : a.key_norm), lane,
                   with.weight_low, with.weight_high);
  // Position-dependent operands: before the wait when the positions are inputs of the step.
  int position = 0;
  bool in_table = false;
  long long owner = request;
  const auto fetch_rope = [&] {
    if (a.direct && !is_query)
      owner = a.slots[request];
    position = a.positions[request] + token;
    in_table = position >= 0 && position < a.max_positions;
    if (in_table) {
      load_halves<per>(static_cast<const __nv_bfloat16 *>(a.cosine) +
                           static_cast<size_t>(position) * dimension,
                       lane, with.cosine_low, with.cosine_high);
      load_halves<per>(static_cast<const __nv_bfloat16 *>(a.sine) +
                           static_cast<size_t>(position) * dimension,
                       lane, with.sine_low, with.sine_high);
    }
  };
  if (a.inputs_static != 0)
    fetch_rope();
  grid_dependency_wait();
  if (a.inputs_static == 0)
    fetch_rope();

  const auto *packed_row =
      static_cast<const __nv_bfloat16 *>(a.packed) + static_cast<size_t>(row) * packed_width;
  float low[per];
  float high[per];
  float value_low[per];
  float value_high[per];
  load_halves<per>(packed_row + (is_query ? head * dimension : query_width + kv_head * dimension),
                   lane, low, high);
  const bool separate_value = !is_query && !a.key_equals_value;
  if (separate_value)
    load_halves<per>(packed_row + query_width + kv_width + kv_head * dimension, lane, value_low,
                     value_high);
  if (!in_table)
    return;

  const float inverse_rms = inverse_rms_of<per>(low, high, a.epsilon);
  float out_low[per];
  float out_high[per];
  norm_rope<per>(low, high, inverse_rms, with, out_low, out_high);
  if (is_query) {
    auto *output = static_cast<__nv_bfloat16 *>(a.queries) +
                   ((static_cast<size_t>(request) * a.query_heads + head) * a.depth + token) *
                       dimension;
    store_halves<per>(output, lane, out_low, out_high);
    return;
  }
  float inverse_value_rms = inverse_rms;
  if (separate_value) {
    inverse_value_rms = inverse_rms_of<per>(value_low, value_high, a.epsilon);
  } else {
#pragma unroll
    for (int index = 0; index < per; ++index) {
      value_low[index] = low[index];
      value_high[index] = high[index];
    }
  }
#pragma unroll
  for (int index = 0; index < per; ++index) {
    value_low[index] *= inverse_value_rms;
    value_high[index] *= inverse_value_rms;
  }
  const int cache_row = a.direct ? position % a.capacity : token;
  const size_t destination = static_cast<size_t>(owner * a.slot_stride + kv_head * a.head_stride) +
                             static_cast<size_t>(cache_row) * dimension;
  store_halves<per>(static_cast<__nv_bfloat16 *>(a.key_base) + destination, lane, out_low,
                    out_high);
  store_halves<per>(static_cast<__nv_bfloat16 *>(a.value_base) + destination, lane, value_low,
                    value_high);
}

template <int per>
__global__ void query_post_kernel(const __nv_bfloat16 *projected, const __nv_bfloat16 *weight,
                                  const __nv_bfloat16 *cosine_table,
                                  const __nv_bfloat16 *sine_table, __nv_bfloat16 *queries,
                                  const int *positions, int position_offset, int requests,
                                  int query_heads, int max_positions, float epsilon,
                                  bool inputs_static) {
  constexpr int dimension = per * 64;
  grid_dependency_launch();
  const int warp = static_cast<int>(blockIdx.x) * (blockDim.x / 32) + (threadIdx.x / 32);
  const int lane = static_cast<int>(threadIdx.x) & 31;
  if (warp >= requests * query_heads)
    return;
  const int request = warp / query_heads;
  RopeOperands<per> with;
  load_halves<per>(weight, lane, with.weight_low, with.weight_high);
  bool in_table = false;
  const auto fetch_rope = [&] {
    const int position = positions[request] + position_offset;
    in_table = position >= 0 && position < max_positions;
    if (in_table) {
      load_halves<per>(cosine_table + static_cast<size_t>(position) * dimension, lane,
                       with.cosine_low, with.cosine_high);
      load_halves<per>(sine_table + static_cast<size_t>(position) * dimension, lane,
                       with.sine_low, with.sine_high);
    }
  };
  if (inputs_static)
    fetch_rope();
  grid_dependency_wait();
  if (!inputs_static)
    fetch_rope();
  float low[per];
  float high[per];
  load_halves<per>(projected + static_cast<size_t>(warp) * dimension, lane, low, high);
  if (!in_table)
    return;
  const float inverse_rms = inverse_rms_of<per>(low, high, epsilon);
  float out_low[per];
  float out_high[per];
  norm_rope<per>(low, high, inverse_rms, with, out_low, out_high);
  store_halves<per>(queries + static_cast<size_t>(warp) * dimension, lane, out_low, out_high);
}

// The kernels move head vectors in 8- and 16-byte pieces.
template <typename... Pointers> bool aligned16(Pointers... pointers) {
  return ((reinterpret_cast<uintptr_t>(pointers) % 16 == 0) && ...);
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
      a.capacity <= 0 || a.slot_stride % 8 != 0 || a.head_stride % 8 != 0 ||
      !aligned16(a.packed, a.query_norm, a.key_norm, a.cosine, a.sine, a.queries, a.key_base,
                 a.value_base)) {
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
                      float epsilon, cudaStream_t stream, bool inputs_static) {
  if (projected == nullptr || query_norm == nullptr || cosine == nullptr || sine == nullptr ||
      queries == nullptr || positions == nullptr || requests <= 0 || query_heads <= 0 ||
      !aligned16(projected, query_norm, cosine, sine, queries)) {
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
                   positions, position_offset, requests, query_heads, max_positions, epsilon,
                   inputs_static);
    break;
  case 256:
    launch_chained(query_post_kernel<4>, dim3(blocks), dim3(128), 0, stream, false, p, w, c, s, q,
                   positions, position_offset, requests, query_heads, max_positions, epsilon,
                   inputs_static);
    break;
  case 512:
    launch_chained(query_post_kernel<8>, dim3(blocks), dim3(128), 0, stream, false, p, w, c, s, q,
                   positions, position_offset, requests, query_heads, max_positions, epsilon,
                   inputs_static);
    break;
  default:
    return -3;
  }
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -11;
}

} // namespace carat_b200
