#include "attention.cuh"
#include "attention_geometry.cuh"
#include "context.cuh"
#include "launch.cuh"

#include <cuda_bf16.h>
#include <math_constants.h>

namespace carat_b200 {
namespace {

// Pointer to the key/value row behind score column `column` of (request, kv_head).
__device__ __forceinline__ const __nv_bfloat16 *row_pointer(const AttentionArguments &a,
                                                            const void *cache, const void *fresh,
                                                            int request, int kv_head, int column) {
  if (column < proposal_columns) {
    return static_cast<const __nv_bfloat16 *>(fresh) + request * a.new_request_stride +
           kv_head * a.new_head_stride + static_cast<size_t>(column) * a.head_dim;
  }
  const int slot = a.slots[request];
  return static_cast<const __nv_bfloat16 *>(cache) + slot * a.slot_stride +
         kv_head * a.head_stride + static_cast<size_t>(column - proposal_columns) * a.head_dim;
}

__device__ __forceinline__ bool column_has_row(const KeyGeometry &g, int column) {
  return column < proposal_columns ? column < g.proposals : column - proposal_columns < g.cache_rows;
}

// Phase 1: scores[row, column] = bf16(q_row . k_column). One thread per column, queries in
// shared memory.
template <int dimension>
__global__ void __launch_bounds__(128) scores_kernel(AttentionArguments a) {
  extern __shared__ __align__(16) unsigned char shared_raw[];
  auto *shared_queries = reinterpret_cast<__nv_bfloat16 *>(shared_raw);
  grid_dependency_launch();
  grid_dependency_wait();
  const int request = static_cast<int>(blockIdx.z);
  const int kv_head = static_cast<int>(blockIdx.y);
  const int group = a.query_heads / a.kv_heads;
  const int rows = group * a.depth;
  const KeyGeometry g = key_geometry(a, request);
  const int first_column = static_cast<int>(blockIdx.x) * 128;
  if (first_column >= g.columns())
    return;
  const auto *query_rows = static_cast<const __nv_bfloat16 *>(a.queries) +
                           (static_cast<size_t>(request) * a.query_heads + kv_head * group) *
                               a.depth * dimension;
  for (int index = static_cast<int>(threadIdx.x) * 8; index < rows * dimension; index += 128 * 8)
    *reinterpret_cast<uint4 *>(shared_queries + index) =
        *reinterpret_cast<const uint4 *>(query_rows + index);
  __syncthreads();
  const int column = first_column + static_cast<int>(threadIdx.x);
  if (column >= g.columns() || !column_has_row(g, column))
    return;
  const __nv_bfloat16 *key_row = row_pointer(a, a.key_cache, a.new_keys, request, kv_head, column);
  auto *score_rows = static_cast<__nv_bfloat16 *>(a.scores) +
                     (static_cast<size_t>(request) * a.query_heads + kv_head * group) * a.depth *
                         a.score_stride;
  for (int row_base = 0; row_base < rows; row_base += 8) {
    float sums[8] = {0.0F, 0.0F, 0.0F, 0.0F, 0.0F, 0.0F, 0.0F, 0.0F};
    for (int component = 0; component < dimension; component += 8) {
      const uint4 key_raw = *reinterpret_cast<const uint4 *>(key_row + component);
      const auto *key_pairs = reinterpret_cast<const __nv_bfloat162 *>(&key_raw);
      float key_values[8];
#pragma unroll
      for (int pair = 0; pair < 4; ++pair) {
        const float2 both = __bfloat1622float2(key_pairs[pair]);
        key_values[2 * pair] = both.x;
        key_values[2 * pair + 1] = both.y;
      }
#pragma unroll
      for (int row = 0; row < 8; ++row) {
        if (row_base + row < rows) {
          const uint4 query_raw = *reinterpret_cast<const uint4 *>(
              shared_queries + (row_base + row) * dimension + component);
          const auto *query_pairs = reinterpret_cast<const __nv_bfloat162 *>(&query_raw);
#pragma unroll
          for (int pair = 0; pair < 4; ++pair) {
            const float2 both = __bfloat1622float2(query_pairs[pair]);
            sums[row] = fmaf(both.x, key_values[2 * pair], sums[row]);
            sums[row] = fmaf(both.y, key_values[2 * pair + 1], sums[row]);
          }
        }
      }
    }
#pragma unroll
    for (int row = 0; row < 8; ++row) {
      if (row_base + row < rows)
        score_rows[static_cast<size_t>(row_base + row) * a.score_stride + column] =
            __float2bfloat16_rn(sums[row]);
    }
  }
}

// Phase 2: in-place softmax of one score row; masked and padding columns become exact zeros.
// Visibility is evaluated without a division per element: for a ring row r the distance
// m = (position - 1 - r) mod capacity back from the newest resident position is one compare and
// add, and the row is inside query t's window iff m <= window - 2 - t.
struct RowVisibility {
  int proposals;
  int cache_rows;
  int token;
  int mode;          // 0 everything, 1 causal over a linear cache, 2 ring window
  int causal_last;   // mode 1: last visible cache row
  int newest_row;    // mode 2: (position - 1) % capacity
  int capacity;
  int reach;         // mode 2: window - 2 - token
  __device__ __forceinline__ bool operator()(int column) const {
    if (column < proposal_columns)
      return column < proposals && column <= token;
    const int row = column - proposal_columns;
    if (row >= cache_rows)
      return false;
    if (mode == 0)
      return true;
    if (mode == 1)
      return row <= causal_last;
    int distance = newest_row - row;
    if (distance < 0)
      distance += capacity;
    return distance <= reach;
  }
};

constexpr int softmax_threads = 128;

__global__ void __launch_bounds__(softmax_threads) softmax_kernel(AttentionArguments a) {
  __shared__ float scratch[softmax_threads / 32];
  grid_dependency_launch();
  grid_dependency_wait();
  const int row_index = static_cast<int>(blockIdx.x);
  const int token = row_index % a.depth;
  const int request = row_index / (a.depth * a.query_heads);
  const KeyGeometry g = key_geometry(a, request);
  const int position = a.positions[request];
  RowVisibility visible;
  visible.proposals = g.proposals;
  visible.cache_rows = g.cache_rows;
  visible.token = token;
  visible.capacity = a.capacity;
  visible.causal_last = position + token;
  visible.newest_row = position > 0 ? (position - 1) % a.capacity : 0;
  visible.reach = a.window - 2 - token;
  visible.mode = a.draft ? 0 : a.new_keys == nullptr ? 1 : a.window > 0 ? 2 : 0;
  auto *row = static_cast<__nv_bfloat16 *>(a.scores) + static_cast<size_t>(row_index) * a.score_stride;
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int warp = static_cast<int>(threadIdx.x) >> 5;
  // Whole 128-row cache tiles: the P.V phase multiplies complete tiles, so padding must be zero.
  const int padded = min(a.score_stride, score_columns(g.cache_rows));

  float maximum = -CUDART_INF_F;
  for (int base = static_cast<int>(threadIdx.x) * 8; base < padded; base += softmax_threads * 8) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(row + base);
    const auto *values = reinterpret_cast<const __nv_bfloat16 *>(&raw);
#pragma unroll
    for (int index = 0; index < 8; ++index) {
      if (visible(base + index))
        maximum = fmaxf(maximum, __bfloat162float(values[index]));
    }
  }
  for (int offset = 16; offset > 0; offset >>= 1)
    maximum = fmaxf(maximum, __shfl_xor_sync(0xFFFFFFFFU, maximum, offset));
  if (lane == 0)
    scratch[warp] = maximum;
  __syncthreads();
  maximum = fmaxf(fmaxf(scratch[0], scratch[1]), fmaxf(scratch[2], scratch[3]));
  __syncthreads();

  float sum = 0.0F;
  for (int base = static_cast<int>(threadIdx.x) * 8; base < padded; base += softmax_threads * 8) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(row + base);
    const auto *values = reinterpret_cast<const __nv_bfloat16 *>(&raw);
#pragma unroll
    for (int index = 0; index < 8; ++index) {
      if (visible(base + index))
        sum += expf(__bfloat162float(values[index]) - maximum);
    }
  }
  for (int offset = 16; offset > 0; offset >>= 1)
    sum += __shfl_xor_sync(0xFFFFFFFFU, sum, offset);
  if (lane == 0)
    scratch[warp] = sum;
  __syncthreads();
  const float inverse_sum = 1.0F / (scratch[0] + scratch[1] + scratch[2] + scratch[3]);

  for (int base = static_cast<int>(threadIdx.x) * 8; base < padded; base += softmax_threads * 8) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(row + base);
    const auto *values = reinterpret_cast<const __nv_bfloat16 *>(&raw);
    __align__(16) __nv_bfloat16 result[8];
#pragma unroll
    for (int index = 0; index < 8; ++index) {
      result[index] = visible(base + index)
                          ? __float2bfloat16_rn(expf(__bfloat162float(values[index]) - maximum) *
                                                inverse_sum)
                          : __float2bfloat16_rn(0.0F);
    }
    *reinterpret_cast<uint4 *>(row + base) = *reinterpret_cast<const uint4 *>(result);
  }
}

// Phase 3: out[row, :] = sum_column P[row, column] * V[column, :] over one chunk of cache rows
// (chunk 0 also takes the proposal columns). Each thread owns two adjacent components;
// probabilities are staged through shared memory 64 columns at a time.
template <int dimension, int max_rows>
__global__ void __launch_bounds__(dimension / 2) pv_kernel(AttentionArguments a) {
  __shared__ __nv_bfloat16 probabilities[max_rows][64];
  grid_dependency_launch();
  grid_dependency_wait();
  const int request = static_cast<int>(blockIdx.z);
  const int kv_head = static_cast<int>(blockIdx.y);
  const int chunk = static_cast<int>(blockIdx.x);
  const int group = a.query_heads / a.kv_heads;
  const int rows = group * a.depth;
  const KeyGeometry g = key_geometry(a, request);
  const int component = static_cast<int>(threadIdx.x) * 2;
  const auto *score_rows = static_cast<const __nv_bfloat16 *>(a.scores) +
                           (static_cast<size_t>(request) * a.query_heads + kv_head * group) *
                               a.depth * a.score_stride;
  float sums[max_rows][2];
#pragma unroll
  for (int row = 0; row < max_rows; ++row) {
    sums[row][0] = 0.0F;
    sums[row][1] = 0.0F;
  }
  // Two column ranges: the proposals (chunk 0 only) and this chunk's cache rows.
  for (int range = 0; range < 2; ++range) {
    int begin;
    int end;
    if (range == 0) {
      begin = 0;
      end = chunk == 0 ? g.proposals : 0;
    } else {
      begin = proposal_columns + chunk * a.chunk_keys;
      end = proposal_columns + min(g.cache_rows, (chunk + 1) * a.chunk_keys);
    }
    for (int tile = begin; tile < end; tile += 64) {
      __syncthreads();
      for (int index = static_cast<int>(threadIdx.x); index < rows * 64; index += dimension / 2) {
        const int row = index / 64;
        const int column = tile + index % 64;
        probabilities[row][index % 64] =
            column < end ? score_rows[static_cast<size_t>(row) * a.score_stride + column]
                         : __float2bfloat16_rn(0.0F);
      }
      __syncthreads();
      const int tile_columns = min(64, end - tile);
      for (int offset = 0; offset < tile_columns; ++offset) {
        const __nv_bfloat16 *value_row =
            row_pointer(a, a.value_cache, a.new_values, request, kv_head, tile + offset);
        const float2 value =
            __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(value_row + component));
#pragma unroll
        for (int row = 0; row < max_rows; ++row) {
          if (row < rows) {
            const float probability = __bfloat162float(probabilities[row][offset]);
            sums[row][0] = fmaf(probability, value.x, sums[row][0]);
            sums[row][1] = fmaf(probability, value.y, sums[row][1]);
          }
        }
      }
    }
  }
  const int width = a.query_heads * dimension;
#pragma unroll
  for (int row = 0; row < max_rows; ++row) {
    if (row < rows) {
      const int local_head = row / a.depth;
      const int token = row % a.depth;
      const size_t out_row = static_cast<size_t>(request) * a.depth + token;
      const size_t column = static_cast<size_t>(kv_head * group + local_head) * dimension + component;
      if (a.chunks > 1) {
        float *destination = a.chunk_partials +
                             (static_cast<size_t>(chunk) * a.requests * a.depth + out_row) * width +
                             column;
        *reinterpret_cast<float2 *>(destination) = make_float2(sums[row][0], sums[row][1]);
      } else {
        auto *destination = static_cast<__nv_bfloat16 *>(a.output) + out_row * width + column;
        *reinterpret_cast<__nv_bfloat162 *>(destination) =
            __halves2bfloat162(__float2bfloat16_rn(sums[row][0]), __float2bfloat16_rn(sums[row][1]));
      }
    }
  }
}

template <int dimension> int launch_phases(const AttentionArguments &a, cudaStream_t stream) {
  const int group = a.query_heads / a.kv_heads;
  const int rows = group * a.depth;
  const int columns = proposal_columns + a.max_cache_rows;
  const size_t query_bytes = static_cast<size_t>(rows) * dimension * sizeof(__nv_bfloat16);
  if (query_bytes > 96 * 1024 || rows > 80)
    return -2;
  static PerDeviceOnce configured;
  if (configured.run([] {
        return cudaFuncSetAttribute(scores_kernel<dimension>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
      }) != cudaSuccess) {
    return -10;
  }
  const dim3 score_grid(static_cast<unsigned>((columns + 127) / 128),
                        static_cast<unsigned>(a.kv_heads), static_cast<unsigned>(a.requests));
  launch_chained(scores_kernel<dimension>, score_grid, dim3(128), query_bytes, stream, false, a);
  launch_chained(softmax_kernel, dim3(static_cast<unsigned>(a.requests * a.query_heads * a.depth)),
                 dim3(softmax_threads), 0, stream, false, a);
  const dim3 pv_grid(static_cast<unsigned>(a.chunks), static_cast<unsigned>(a.kv_heads),
                     static_cast<unsigned>(a.requests));
  if (rows <= 16) {
    launch_chained(pv_kernel<dimension, 16>, pv_grid, dim3(dimension / 2), 0, stream, false, a);
  } else if (rows <= 40) {
    launch_chained(pv_kernel<dimension, 40>, pv_grid, dim3(dimension / 2), 0, stream, false, a);
  } else {
    launch_chained(pv_kernel<dimension, 80>, pv_grid, dim3(dimension / 2), 0, stream, false, a);
  }
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -11;
}

} // namespace

int validate_attention(const AttentionArguments &a) {
  if (a.queries == nullptr || a.key_cache == nullptr || a.value_cache == nullptr ||
      a.positions == nullptr || a.slots == nullptr || a.scores == nullptr || a.requests <= 0 ||
      a.depth <= 0 || a.depth > proposal_columns || a.query_heads <= 0 || a.kv_heads <= 0 ||
      a.query_heads % a.kv_heads != 0 || a.capacity <= 0 || a.chunks <= 0 || a.chunk_keys <= 0 ||
      a.chunk_keys % 128 != 0 || a.score_stride % 8 != 0 || a.max_cache_rows < 0 ||
      (a.chunks > 1 ? a.chunk_partials == nullptr : a.output == nullptr) ||
      (a.draft && (a.depth != 1 || a.new_keys != nullptr)) ||
      ((a.new_keys == nullptr) != (a.new_values == nullptr))) {
    return -1;
  }
  if (score_columns(a.max_cache_rows) > a.score_stride ||
      a.chunks * a.chunk_keys < a.max_cache_rows) {
    return -2;
  }
  return 0;
}

int launch_attention_softmax(const AttentionArguments &a, cudaStream_t stream) {
  launch_chained(softmax_kernel, dim3(static_cast<unsigned>(a.requests * a.query_heads * a.depth)),
                 dim3(softmax_threads), 0, stream, false, a);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -11;
}

int launch_attention_simt(const AttentionArguments &a, cudaStream_t stream) {
  const int status = validate_attention(a);
  if (status != 0)
    return status;
  switch (a.head_dim) {
  case 64:
    return launch_phases<64>(a, stream);
  case 256:
    return launch_phases<256>(a, stream);
  case 512:
    return launch_phases<512>(a, stream);
  default:
    return -3;
  }
}

} // namespace carat_b200
