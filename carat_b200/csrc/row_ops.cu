#include "row_ops.cuh"

#include "context.cuh"
#include "launch.cuh"

#include <cooperative_groups.h>
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace cg = cooperative_groups;

namespace carat_b200 {
namespace {

constexpr int row_threads = 512;
constexpr int row_warps = row_threads / 32;

enum class RowMode : int { embed_norm, norm, plain, post_attention, geglu, layer_output, embed_concat };

struct RowArguments {
  // sources
  const __nv_bfloat16 *input;        // bf16 [rows, width] (or [rows, 2*width] for geglu)
  const float *partial;              // fp32 [splits, rows, width] when splits > 0
  int splits;
  const float *input_scale;
  const float *weight_scale;
  const int *valid_splits;           // optional per-row-group piece counts (see PartialSource)
  int rows_per_group;
  const __nv_bfloat16 *embedding;
  const int *tokens;
  const int *row_indices;
  int vocabulary;
  const __nv_bfloat16 *norm_weight;
  const __nv_bfloat16 *residual;
  const __nv_bfloat16 *next_norm_weight;
  const __nv_bfloat16 *scalar;
  // bf16 outputs (any may be null)
  __nv_bfloat16 *first_out;
  __nv_bfloat16 *second_out;
  // quantised output
  unsigned char *fp8_output;
  float *scale;
  unsigned int *amax_bits;
  // geglu only: the up columns from packed column `tail_first_column` on come as fp32 partial
  // sums [tail_splits, rows, tail_width] of the linear (scaled by input_scale * weight_scale).
  const float *tail_partial;
  int tail_splits;
  int tail_first_column;
  int tail_width;
  int parts;                         // CTAs per row (GeGLU only; 0 or 1 = one)
  __nv_bfloat16 *pass_rows;          // two-launch form: bf16 rows [rows, width] between the launches
  unsigned int *clear_base;
  int clear_words;
  unsigned int *barrier_word;
  int *barrier_error;
  int width;
  float epsilon;
};

__device__ __forceinline__ float warp_sum(float value) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1)
    value += __shfl_xor_sync(0xFFFFFFFFU, value, offset);
  return value;
}

__device__ __forceinline__ float warp_max(float value) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1)
    value = fmaxf(value, __shfl_xor_sync(0xFFFFFFFFU, value, offset));
  return value;
}

// Every thread receives the block-wide result after a single barrier: each warp leaves its
// partial in shared memory and every thread adds up all of them (broadcast reads). `scratch`
// holds 2 * row_warps floats; consecutive reductions alternate between the halves (`parity`), so
// a warp that races ahead to the next reduction cannot overwrite partials others still read.
__device__ __forceinline__ float block_sum(float value, float *scratch, int &parity) {
  value = warp_sum(value);
  float *partials = scratch + parity * row_warps;
  if ((threadIdx.x & 31U) == 0U)
    partials[threadIdx.x >> 5U] = value;
  __syncthreads();
  float total = 0.0F;
#pragma unroll
  for (int warp = 0; warp < row_warps; ++warp)
    total += partials[warp];
  parity ^= 1;
  return total;
}

__device__ __forceinline__ float block_max(float value, float *scratch, int &parity) {
  value = warp_max(value);
  float *partials = scratch + parity * row_warps;
  if ((threadIdx.x & 31U) == 0U)
    partials[threadIdx.x >> 5U] = value;
  __syncthreads();
  float total = 0.0F;
#pragma unroll
  for (int warp = 0; warp < row_warps; ++warp)
    total = fmaxf(total, partials[warp]);
  parity ^= 1;
  return total;
}

struct Pack8 {
  float v[8];
};

__device__ __forceinline__ Pack8 load_bf16x8(const __nv_bfloat16 *pointer) {
  const uint4 raw = *reinterpret_cast<const uint4 *>(pointer);
  const __nv_bfloat162 *pairs = reinterpret_cast<const __nv_bfloat162 *>(&raw);
  Pack8 result;
#pragma unroll
  for (int pair = 0; pair < 4; ++pair) {
    const float2 both = __bfloat1622float2(pairs[pair]);
    result.v[2 * pair] = both.x;
    result.v[2 * pair + 1] = both.y;
  }
  return result;
}

__device__ __forceinline__ Pack8 unpack_bf16x8(const uint4 &raw) {
  const __nv_bfloat162 *pairs = reinterpret_cast<const __nv_bfloat162 *>(&raw);
  Pack8 result;
#pragma unroll
  for (int pair = 0; pair < 4; ++pair) {
    const float2 both = __bfloat1622float2(pairs[pair]);
    result.v[2 * pair] = both.x;
    result.v[2 * pair + 1] = both.y;
  }
  return result;
}

// Rounds to bf16, stores, and returns the rounded values as floats.
__device__ __forceinline__ Pack8 round_bf16x8(const Pack8 &values, uint4 *packed) {
  __nv_bfloat162 pairs[4];
  Pack8 rounded;
#pragma unroll
  for (int pair = 0; pair < 4; ++pair) {
    pairs[pair] = __halves2bfloat162(__float2bfloat16_rn(values.v[2 * pair]),
                                     __float2bfloat16_rn(values.v[2 * pair + 1]));
    const float2 both = __bfloat1622float2(pairs[pair]);
    rounded.v[2 * pair] = both.x;
    rounded.v[2 * pair + 1] = both.y;
  }
  *packed = *reinterpret_cast<const uint4 *>(pairs);
  return rounded;
}

// Loads a thread's `chunks` groups of eight values of the row's primary source: a bf16 tensor, or
// split-K / key-chunk partials summed in a fixed order (piece 0 first), scaled and rounded to bf16
// exactly like a separate finishing kernel. The loads of all groups are issued together, a few
// pieces at a time (as many as the registers hold): a loop that loads and adds group by group, or
// piece by piece, pays one L2 round trip per turn.
template <int chunks>
__device__ __forceinline__ void load_source(const RowArguments &a, size_t row, int column_base,
                                            int column_end, size_t rows, float partial_scale,
                                            Pack8 (&values)[chunks]) {
  if (a.splits <= 0) {
#pragma unroll
    for (int chunk = 0; chunk < chunks; ++chunk) {
      const int column = column_base + (chunk * row_threads + static_cast<int>(threadIdx.x)) * 8;
      if (column < column_end)
        values[chunk] = load_bf16x8(a.input + row * a.width + column);
    }
    return;
  }
  constexpr int batch = chunks <= 1 ? 8 : chunks <= 2 ? 4 : chunks <= 4 ? 2 : 1;
  int pieces = a.splits;
  if (a.valid_splits != nullptr)
    pieces = min(pieces, a.valid_splits[row / a.rows_per_group]);
  for (int first = 0; first < pieces; first += batch) {
    float4 low[chunks][batch];
    float4 high[chunks][batch];
#pragma unroll
    for (int chunk = 0; chunk < chunks; ++chunk) {
      const int column = column_base + (chunk * row_threads + static_cast<int>(threadIdx.x)) * 8;
#pragma unroll
      for (int offset = 0; offset < batch; ++offset) {
        low[chunk][offset] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
        high[chunk][offset] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
        if (column < column_end && first + offset < pieces) {
          const float *source =
              a.partial + (static_cast<size_t>(first + offset) * rows + row) * a.width + column;
          low[chunk][offset] = *reinterpret_cast<const float4 *>(source);
          high[chunk][offset] = *reinterpret_cast<const float4 *>(source + 4);
        }
      }
    }
#pragma unroll
    for (int chunk = 0; chunk < chunks; ++chunk) {
#pragma unroll
      for (int offset = 0; offset < batch; ++offset) {
        values[chunk].v[0] += low[chunk][offset].x;
        values[chunk].v[1] += low[chunk][offset].y;
        values[chunk].v[2] += low[chunk][offset].z;
        values[chunk].v[3] += low[chunk][offset].w;
        values[chunk].v[4] += high[chunk][offset].x;
        values[chunk].v[5] += high[chunk][offset].y;
        values[chunk].v[6] += high[chunk][offset].z;
        values[chunk].v[7] += high[chunk][offset].w;
      }
    }
  }
#pragma unroll
  for (int chunk = 0; chunk < chunks; ++chunk)
#pragma unroll
    for (int index = 0; index < 8; ++index)
      values[chunk].v[index] =
          __bfloat162float(__float2bfloat16_rn(values[chunk].v[index] * partial_scale));
}

// Every thread owns `chunks` groups of eight consecutive columns, group c at column
// (c * row_threads + thread) * 8, and keeps them in registers from the first load to the e4m3
// store: the row never goes through shared or global memory between the phases. Static operands
// (norm weights) are loaded before the wait on the previous grid, everything else right after it,
// so one global-memory round trip feeds the whole kernel.
//
// `two_launches` = false: cooperative launch, one grid barrier between the maximum and the e4m3
// store (needs every CTA resident at once). true: the kernel stops after the maximum, leaving the
// bf16 rows in a.pass_rows, and quantize_rows_kernel finishes; used when there are more rows than
// the device holds CTAs (the scratch words must then have been cleared by the caller).
template <RowMode mode, int chunks, bool two_launches>
__global__ void __launch_bounds__(row_threads, (mode == RowMode::geglu && chunks <= 4) ? 2 : 1)
row_kernel(RowArguments a) {
  __shared__ float scratch[2 * row_warps];
  int parity = 0;

  // Modes without a row-wide reduction (GeGLU) may cut a row into `parts` column ranges, one CTA
  // each, so that a wide row does not sit in a single CTA.
  const int parts = a.parts > 1 ? a.parts : 1;
  const size_t row = blockIdx.x / parts;
  const size_t rows = gridDim.x / parts;
  const int width = a.width;
  const int part = static_cast<int>(blockIdx.x) - static_cast<int>(row) * parts;
  const int column_base = part * (width / parts);
  const int column_end = part + 1 == parts ? width : column_base + width / parts;
  const float width_value = static_cast<float>(width);
  constexpr bool two_norms = mode == RowMode::post_attention || mode == RowMode::layer_output;
  constexpr bool one_norm = mode == RowMode::embed_norm || mode == RowMode::norm;

  grid_dependency_launch();
  uint4 weight_raw[chunks];
  uint4 next_weight_raw[chunks];
#pragma unroll
  for (int chunk = 0; chunk < chunks; ++chunk) {
    const int column = column_base + (chunk * row_threads + static_cast<int>(threadIdx.x)) * 8;
    weight_raw[chunk] = make_uint4(0, 0, 0, 0);
    next_weight_raw[chunk] = make_uint4(0, 0, 0, 0);
    if (column < column_end) {
      if constexpr (one_norm || two_norms)
        weight_raw[chunk] = *reinterpret_cast<const uint4 *>(a.norm_weight + column);
      if constexpr (two_norms)
        next_weight_raw[chunk] = *reinterpret_cast<const uint4 *>(a.next_norm_weight + column);
    }
  }
  // The layer scalar is a weight like the norm vectors: fetched before the wait as well.
  [[maybe_unused]] float layer_scale = 1.0F;
  if constexpr (mode == RowMode::layer_output)
    layer_scale = __bfloat162float(*a.scalar);
  grid_dependency_wait();

  if constexpr (mode == RowMode::embed_norm && !two_launches) {
    // When asked to, clear the per-step scratch words before the first atomic maximum of the
    // step; the barrier orders this against every later use, including this kernel's own.
    if (a.clear_words > 0) {
      for (int word = static_cast<int>(blockIdx.x) * row_threads + static_cast<int>(threadIdx.x);
           word < a.clear_words; word += static_cast<int>(gridDim.x) * row_threads)
        a.clear_base[word] = 0U;
      cg::this_grid().sync();
    }
  }

  float partial_scale = 1.0F;
  if (a.splits > 0 && a.input_scale != nullptr)
    partial_scale = a.input_scale[0] * a.weight_scale[0];

  // ---- load: the bf16-exact starting row (and the residual) into registers. No store happens
  // before the last load of this phase has been issued (a store could alias a later load as far
  // as the compiler knows, and would then hold that load back by a round trip to memory); the
  // rows some modes keep in bf16 are stored by the loop after it.
  Pack8 values[chunks];
  uint4 residual_raw[chunks];
#pragma unroll
  for (int chunk = 0; chunk < chunks; ++chunk) {
    residual_raw[chunk] = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int index = 0; index < 8; ++index)
      values[chunk].v[index] = 0.0F;
  }
  constexpr bool from_source = mode == RowMode::norm || mode == RowMode::plain || two_norms;
  if constexpr (from_source) {
    if constexpr (two_norms) {
#pragma unroll
      for (int chunk = 0; chunk < chunks; ++chunk) {
        const int column = column_base + (chunk * row_threads + static_cast<int>(threadIdx.x)) * 8;
        if (column < column_end)
          residual_raw[chunk] = *reinterpret_cast<const uint4 *>(a.residual + row * width + column);
      }
    }
    load_source<chunks>(a, row, column_base, column_end, rows, partial_scale, values);
  } else if constexpr (mode == RowMode::embed_norm || mode == RowMode::embed_concat) {
    // embed_concat: `width` is the concatenated width, scaled embedding row then the carried
    // hidden state.
    const int embedded = mode == RowMode::embed_norm ? width : width / 2;
    const int token = a.tokens[row];
    const float scale =
        __bfloat162float(__float2bfloat16_rn(sqrtf(static_cast<float>(embedded))));
    size_t source_row = row;
    if constexpr (mode == RowMode::embed_concat) {
      if (a.row_indices != nullptr)
        source_row = static_cast<size_t>(a.row_indices[row]);
    }
#pragma unroll
    for (int chunk = 0; chunk < chunks; ++chunk) {
      const int column = column_base + (chunk * row_threads + static_cast<int>(threadIdx.x)) * 8;
      if (column >= column_end)
        continue;
      if (column < embedded) {
        Pack8 raw = values[chunk];
        if (token >= 0 && token < a.vocabulary)
          raw = load_bf16x8(a.embedding + static_cast<size_t>(token) * embedded + column);
#pragma unroll
        for (int index = 0; index < 8; ++index)
          raw.v[index] *= scale;
        uint4 packed;
        values[chunk] = round_bf16x8(raw, &packed);
      } else {
        values[chunk] = load_bf16x8(a.input + source_row * embedded + (column - embedded));
      }
    }
  } else {   // GeGLU
    const __nv_bfloat16 *packed_row = a.input + row * 2 * width;
    float tail_scale = 1.0F;
    if (a.tail_partial != nullptr)
      tail_scale = a.input_scale[0] * a.weight_scale[0];
    // Gate and (outside the linear's K-cut tail tiles) up columns of every group first, in one
    // round trip; the tail columns, whose sums come from a loop over the pieces, after them.
    uint4 gate_raw[chunks];
    uint4 up_raw[chunks];
#pragma unroll
    for (int chunk = 0; chunk < chunks; ++chunk) {
      const int column = column_base + (chunk * row_threads + static_cast<int>(threadIdx.x)) * 8;
      gate_raw[chunk] = make_uint4(0, 0, 0, 0);
      up_raw[chunk] = make_uint4(0, 0, 0, 0);
      if (column < column_end) {
        gate_raw[chunk] = *reinterpret_cast<const uint4 *>(packed_row + column);
        if (!(a.tail_partial != nullptr && width + column >= a.tail_first_column))
          up_raw[chunk] = *reinterpret_cast<const uint4 *>(packed_row + width + column);
      }
    }
#pragma unroll
    for (int chunk = 0; chunk < chunks; ++chunk) {
      const int column = column_base + (chunk * row_threads + static_cast<int>(threadIdx.x)) * 8;
      if (column >= column_end)
        continue;
      const Pack8 gate = unpack_bf16x8(gate_raw[chunk]);
      Pack8 up = unpack_bf16x8(up_raw[chunk]);
      if (a.tail_partial != nullptr && width + column >= a.tail_first_column) {
        // Same finish as the linear's own epilogue: sum of the pieces, scaled, rounded to bf16.
        Pack8 sum;
#pragma unroll
        for (int index = 0; index < 8; ++index)
          sum.v[index] = 0.0F;
        for (int first = 0; first < a.tail_splits; first += 4) {
          float4 low[4];
          float4 high[4];
#pragma unroll
          for (int offset = 0; offset < 4; ++offset) {
            low[offset] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
            high[offset] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
            if (first + offset < a.tail_splits) {
              const float *source =
                  a.tail_partial +
                  (static_cast<size_t>(first + offset) * rows + row) * a.tail_width +
                  (width + column - a.tail_first_column);
              low[offset] = *reinterpret_cast<const float4 *>(source);
              high[offset] = *reinterpret_cast<const float4 *>(source + 4);
            }
          }
#pragma unroll
          for (int offset = 0; offset < 4; ++offset) {
            sum.v[0] += low[offset].x;
            sum.v[1] += low[offset].y;
            sum.v[2] += low[offset].z;
            sum.v[3] += low[offset].w;
            sum.v[4] += high[offset].x;
            sum.v[5] += high[offset].y;
            sum.v[6] += high[offset].z;
            sum.v[7] += high[offset].w;
          }
        }
#pragma unroll
        for (int index = 0; index < 8; ++index)
          sum.v[index] *= tail_scale;
        uint4 unused;
        up = round_bf16x8(sum, &unused);
      }
      Pack8 product;
#pragma unroll
      for (int index = 0; index < 8; ++index)
        product.v[index] = gelu_tanh(gate.v[index]) * up.v[index];
      uint4 packed;
      values[chunk] = round_bf16x8(product, &packed);
    }
  }
  {
    __nv_bfloat16 *rows_out = nullptr;
    if constexpr (mode == RowMode::embed_norm)
      rows_out = a.first_out;
    else if constexpr (mode == RowMode::embed_concat || mode == RowMode::geglu)
      rows_out = a.second_out;
    else if constexpr (mode == RowMode::plain)
      rows_out = a.first_out != nullptr ? a.first_out : a.second_out;
    if (rows_out != nullptr) {
#pragma unroll
      for (int chunk = 0; chunk < chunks; ++chunk) {
        const int column = column_base + (chunk * row_threads + static_cast<int>(threadIdx.x)) * 8;
        if (column >= column_end)
          continue;
        uint4 packed;
        (void)round_bf16x8(values[chunk], &packed);   // already bf16-exact: repack
        *reinterpret_cast<uint4 *>(rows_out + row * width + column) = packed;
      }
    }
  }

  // ---- first norm (+ residual, + layer scalar), rounded to bf16 exactly where the reference does
  if constexpr (one_norm || two_norms) {
    float square_sum = 0.0F;
#pragma unroll
    for (int chunk = 0; chunk < chunks; ++chunk)
#pragma unroll
      for (int index = 0; index < 8; ++index)
        square_sum += values[chunk].v[index] * values[chunk].v[index];
    const float inverse_rms = rsqrtf(block_sum(square_sum, scratch, parity) / width_value + a.epsilon);
#pragma unroll
    for (int chunk = 0; chunk < chunks; ++chunk) {
      const int column = column_base + (chunk * row_threads + static_cast<int>(threadIdx.x)) * 8;
      if (column >= column_end)
        continue;
      const Pack8 weights = unpack_bf16x8(weight_raw[chunk]);
      Pack8 result;
      if constexpr (two_norms) {
        const Pack8 residual = unpack_bf16x8(residual_raw[chunk]);
#pragma unroll
        for (int index = 0; index < 8; ++index)
          result.v[index] =
              values[chunk].v[index] * inverse_rms * weights.v[index] + residual.v[index];
      } else {
#pragma unroll
        for (int index = 0; index < 8; ++index)
          result.v[index] = values[chunk].v[index] * inverse_rms * weights.v[index];
      }
      uint4 packed;
      values[chunk] = round_bf16x8(result, &packed);
      if constexpr (mode == RowMode::layer_output) {
#pragma unroll
        for (int index = 0; index < 8; ++index)
          result.v[index] = values[chunk].v[index] * layer_scale;
        values[chunk] = round_bf16x8(result, &packed);
      }
      if constexpr (two_norms)
        *reinterpret_cast<uint4 *>(a.first_out + row * width + column) = packed;
      if constexpr (one_norm) {
        if (a.second_out != nullptr)
          *reinterpret_cast<uint4 *>(a.second_out + row * width + column) = packed;
      }
    }
  }

  // ---- second norm of the row just formed
  if constexpr (two_norms) {
    float square_sum = 0.0F;
#pragma unroll
    for (int chunk = 0; chunk < chunks; ++chunk)
#pragma unroll
      for (int index = 0; index < 8; ++index)
        square_sum += values[chunk].v[index] * values[chunk].v[index];
    const float inverse_rms = rsqrtf(block_sum(square_sum, scratch, parity) / width_value + a.epsilon);
#pragma unroll
    for (int chunk = 0; chunk < chunks; ++chunk) {
      const int column = column_base + (chunk * row_threads + static_cast<int>(threadIdx.x)) * 8;
      if (column >= column_end)
        continue;
      const Pack8 weights = unpack_bf16x8(next_weight_raw[chunk]);
      Pack8 result;
#pragma unroll
      for (int index = 0; index < 8; ++index)
        result.v[index] = values[chunk].v[index] * inverse_rms * weights.v[index];
      uint4 packed;
      values[chunk] = round_bf16x8(result, &packed);
      if (a.second_out != nullptr)
        *reinterpret_cast<uint4 *>(a.second_out + row * width + column) = packed;
    }
  }

  if (a.fp8_output == nullptr)
    return;   // bf16 consumer: the row is already stored (uniform over the grid)

  // ---- tensor-wide maximum, one barrier, e4m3 from registers
  float row_amax = 0.0F;
#pragma unroll
  for (int chunk = 0; chunk < chunks; ++chunk)
#pragma unroll
    for (int index = 0; index < 8; ++index)
      row_amax = fmaxf(row_amax, fabsf(values[chunk].v[index]));
  row_amax = block_max(row_amax, scratch, parity);
  if (threadIdx.x == 0U)
    atomicMax(a.amax_bits, __float_as_uint(row_amax));
  if constexpr (two_launches) {
#pragma unroll
    for (int chunk = 0; chunk < chunks; ++chunk) {
      const int column = column_base + (chunk * row_threads + static_cast<int>(threadIdx.x)) * 8;
      if (column >= column_end)
        continue;
      uint4 packed;
      (void)round_bf16x8(values[chunk], &packed);   // already bf16-exact: repack
      *reinterpret_cast<uint4 *>(a.pass_rows + row * width + column) = packed;
    }
    return;
  }
  float tensor_amax = 0.0F;
  if (a.barrier_word != nullptr) {
    // Every CTA of the grid is resident (the launcher checked the grid against the device's
    // capacity, and the grid that follows in the chain cannot start before all of these CTAs
    // have), so counting them in is a barrier. The count sits in the word after the maximum
    // (both zero on entry, eight-byte aligned as a pair): one thread a CTA publishes the CTA's
    // maximum, counts the CTA in, and polls both words with one load, so the value it sees with
    // the full count already holds every CTA's maximum. Nothing else crosses the barrier.
    if (threadIdx.x == 0U) {
      __threadfence();   // the atomicMax above is performed before the arrival below
      atomicAdd(a.barrier_word, 1U);
      const auto *pair = reinterpret_cast<volatile unsigned long long *>(a.amax_bits);
      const long long start = clock64();
      unsigned long long seen = *pair;
      while (static_cast<unsigned int>(seen >> 32) < gridDim.x) {
        if (clock64() - start > 4000000000LL) {   // about two seconds: give up, say so
          if (a.barrier_error != nullptr)
            atomicExch(a.barrier_error, 7);
          break;
        }
        seen = *pair;
      }
      scratch[parity * row_warps] = __uint_as_float(static_cast<unsigned int>(seen));
    }
    __syncthreads();
    tensor_amax = scratch[parity * row_warps];
  } else {
    cg::this_grid().sync();
    tensor_amax = __uint_as_float(*reinterpret_cast<volatile unsigned int *>(a.amax_bits));
  }
  const float scale = tensor_amax > 0.0F ? tensor_amax / 448.0F : 1.0F;
  const float inverse_scale = 1.0F / scale;
  if (blockIdx.x == 0U && threadIdx.x == 0U)
    *a.scale = scale;
#pragma unroll
  for (int chunk = 0; chunk < chunks; ++chunk) {
    const int column = column_base + (chunk * row_threads + static_cast<int>(threadIdx.x)) * 8;
    if (column >= column_end)
      continue;
    const Pack8 &v = values[chunk];
    __nv_fp8x4_e4m3 low(make_float4(v.v[0] * inverse_scale, v.v[1] * inverse_scale,
                                    v.v[2] * inverse_scale, v.v[3] * inverse_scale));
    __nv_fp8x4_e4m3 high(make_float4(v.v[4] * inverse_scale, v.v[5] * inverse_scale,
                                     v.v[6] * inverse_scale, v.v[7] * inverse_scale));
    uint2 packed;
    packed.x = low.__x;
    packed.y = high.__x;
    *reinterpret_cast<uint2 *>(a.fp8_output + row * width + column) = packed;
  }
}

// Second launch of the two-launch form: e4m3 = bf16 row / (maximum / 448), eight values a thread.
__global__ void quantize_rows_kernel(const __nv_bfloat16 *rows, const unsigned int *amax_bits,
                                     float *scale_out, unsigned char *fp8_output, size_t elements) {
  grid_dependency_launch();
  grid_dependency_wait();
  const float tensor_amax = __uint_as_float(*amax_bits);
  const float scale = tensor_amax > 0.0F ? tensor_amax / 448.0F : 1.0F;
  const float inverse_scale = 1.0F / scale;
  if (blockIdx.x == 0U && threadIdx.x == 0U)
    *scale_out = scale;
  const size_t index = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (index >= elements)
    return;
  const Pack8 v = load_bf16x8(rows + index);
  __nv_fp8x4_e4m3 low(make_float4(v.v[0] * inverse_scale, v.v[1] * inverse_scale,
                                  v.v[2] * inverse_scale, v.v[3] * inverse_scale));
  __nv_fp8x4_e4m3 high(make_float4(v.v[4] * inverse_scale, v.v[5] * inverse_scale,
                                   v.v[6] * inverse_scale, v.v[7] * inverse_scale));
  uint2 packed;
  packed.x = low.__x;
  packed.y = high.__x;
  *reinterpret_cast<uint2 *>(fp8_output + index) = packed;
}

// `ctas` = rows * parts. Returns -2 when the grid cannot be resident at once and no two-launch
// buffer was given.
template <RowMode mode, int chunks>
int launch_rows_chunks(const RowArguments &arguments, int ctas, cudaStream_t stream) {
  // CTAs of this variant the current device holds at once (the grid barrier needs them all).
  static PerDevice<int> resident_limits;
  int resident_limit = 0;
  {
    int *slot = resident_limits.slot();
    if (slot == nullptr)
      return -10;
    std::lock_guard<std::mutex> lock(resident_limits.lock());
    if (*slot <= 0) {
      int per_multiprocessor = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(
              &per_multiprocessor, row_kernel<mode, chunks, false>, row_threads, 0) !=
          cudaSuccess) {
        return -10;
      }
      *slot = device_multiprocessors() * per_multiprocessor;
    }
    resident_limit = *slot;
  }
  if (resident_limit <= 0)
    return -10;
  if (arguments.fp8_output == nullptr) {
    // No quantisation, so no grid barrier: any number of CTAs, plain launch.
    const cudaError_t status =
        launch_chained(row_kernel<mode, chunks, false>, dim3(static_cast<unsigned>(ctas)),
                       dim3(row_threads), 0, stream, false, arguments);
    return status == cudaSuccess ? 0 : -11;
  }
  if (ctas <= resident_limit) {
    const cudaError_t status =
        launch_chained(row_kernel<mode, chunks, false>, dim3(static_cast<unsigned>(ctas)),
                       dim3(row_threads), 0, stream, arguments.barrier_word == nullptr, arguments);
    return status == cudaSuccess ? 0 : -11;
  }
  if (arguments.pass_rows == nullptr)
    return -2;
  cudaError_t status =
      launch_chained(row_kernel<mode, chunks, true>, dim3(static_cast<unsigned>(ctas)),
                     dim3(row_threads), 0, stream, false, arguments);
  if (status != cudaSuccess)
    return -11;
  const int parts = arguments.parts > 1 ? arguments.parts : 1;
  const size_t elements = static_cast<size_t>(ctas / parts) * arguments.width;
  const unsigned blocks = static_cast<unsigned>((elements / 8 + 255) / 256);
  status = launch_chained(quantize_rows_kernel, dim3(blocks), dim3(256), 0, stream, false,
                          static_cast<const __nv_bfloat16 *>(arguments.pass_rows),
                          static_cast<const unsigned int *>(arguments.amax_bits), arguments.scale,
                          arguments.fp8_output, elements);
  return status == cudaSuccess ? 0 : -11;
}

template <RowMode mode> int launch_rows(RowArguments arguments, int rows, cudaStream_t stream) {
  const bool quantised = arguments.fp8_output != nullptr && arguments.scale != nullptr &&
                         arguments.amax_bits != nullptr;
  // Without an e4m3 target the call stops after the bf16 rows, which must then go somewhere.
  const bool bf16_only = arguments.fp8_output == nullptr &&
                         (arguments.second_out != nullptr || arguments.first_out != nullptr);
  if (rows <= 0 || arguments.width <= 0 || arguments.width % 8 != 0 || !(quantised || bf16_only))
    return -1;
  // The barrier count is read together with the maximum: one aligned eight-byte pair.
  if (arguments.barrier_word != nullptr &&
      (arguments.barrier_word != arguments.amax_bits + 1 ||
       reinterpret_cast<uintptr_t>(arguments.amax_bits) % 8 != 0)) {
    return -1;
  }
  int parts = 1;
  if constexpr (mode == RowMode::geglu) {
    // Wide rows: two CTAs a row when the halves stay multiples of eight columns and the grid
    // still fits the device at once (checked by launch_rows_chunks).
    if (arguments.width >= 8192 && arguments.width % 16 == 0 && rows <= 148)
      parts = 2;   // 2 * 148 CTAs of the two-per-SM variant fit
  }
  for (; parts >= 1; --parts) {
    arguments.parts = parts;
    const int span = arguments.width / parts;
    const int groups = (span / 8 + row_threads - 1) / row_threads;
    const int ctas = rows * parts;
    int status = -2;
    if (groups <= 1)
      status = launch_rows_chunks<mode, 1>(arguments, ctas, stream);
    else if (groups <= 2)
      status = launch_rows_chunks<mode, 2>(arguments, ctas, stream);
    else if (groups <= 4)
      status = launch_rows_chunks<mode, 4>(arguments, ctas, stream);
    else if (groups <= 8)
      status = launch_rows_chunks<mode, 8>(arguments, ctas, stream);
    // -2: the grid would not be resident at once; try again with one CTA a row.
    if (status != -2 || parts == 1)
      return status;
  }
  return -2;
}

// Large tensors (weights at load time): the reference's three-launch form, cuda/linear.cu:117-153.
__global__ void tensor_amax_kernel(const __nv_bfloat16 *input, size_t elements,
                                   unsigned int *maximum_bits) {
  __shared__ float scratch[2 * row_warps];
  int parity = 0;
  float maximum = 0.0F;
  for (size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; index < elements;
       index += static_cast<size_t>(blockDim.x) * gridDim.x)
    maximum = fmaxf(maximum, fabsf(__bfloat162float(input[index])));
  maximum = block_max(maximum, scratch, parity);
  if (threadIdx.x == 0U)
    atomicMax(maximum_bits, __float_as_uint(maximum));
}

__global__ void tensor_scale_kernel(const unsigned int *maximum_bits, float *scale) {
  const float maximum = __uint_as_float(*maximum_bits);
  *scale = maximum > 0.0F ? maximum / 448.0F : 1.0F;
}

__global__ void tensor_quantize_kernel(const __nv_bfloat16 *input, __nv_fp8_e4m3 *output,
                                       const float *scale, size_t elements) {
  const float inverse_scale = 1.0F / *scale;
  for (size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; index < elements;
       index += static_cast<size_t>(blockDim.x) * gridDim.x)
    output[index] = __nv_fp8_e4m3(__bfloat162float(input[index]) * inverse_scale);
}

RowArguments base_arguments(QuantTarget target, int width, float epsilon) {
  RowArguments arguments{};
  arguments.fp8_output = static_cast<unsigned char *>(target.fp8_output);
  arguments.scale = target.scale;
  arguments.amax_bits = target.amax_bits;
  arguments.pass_rows = static_cast<__nv_bfloat16 *>(target.two_launch_rows);
  arguments.barrier_word = target.barrier_word;
  arguments.barrier_error = target.barrier_error;
  arguments.second_out = static_cast<__nv_bfloat16 *>(target.bf16_output);
  arguments.width = width;
  arguments.epsilon = epsilon;
  return arguments;
}

void set_source(RowArguments &arguments, const void *input, const PartialSource &source) {
  arguments.input = static_cast<const __nv_bfloat16 *>(input);
  if (source.partial != nullptr && source.splits > 0) {
    arguments.partial = source.partial;
    arguments.splits = source.splits;
    arguments.input_scale = source.input_scale;
    arguments.weight_scale = source.weight_scale;
    arguments.valid_splits = source.valid_splits;
    arguments.rows_per_group = source.rows_per_group > 0 ? source.rows_per_group : 1;
  }
}

} // namespace

int launch_quant_tensor(const void *input, void *fp8_output, float *scale,
                        unsigned int *amax_bits, size_t elements, cudaStream_t stream) {
  if (input == nullptr || fp8_output == nullptr || scale == nullptr || amax_bits == nullptr ||
      elements == 0) {
    return -1;
  }
  const size_t wanted = (elements + row_threads - 1) / row_threads;
  const int blocks = static_cast<int>(wanted < 4096 ? wanted : 4096);
  tensor_amax_kernel<<<blocks, row_threads, 0, stream>>>(
      static_cast<const __nv_bfloat16 *>(input), elements, amax_bits);
  tensor_scale_kernel<<<1, 1, 0, stream>>>(amax_bits, scale);
  tensor_quantize_kernel<<<blocks, row_threads, 0, stream>>>(
      static_cast<const __nv_bfloat16 *>(input), static_cast<__nv_fp8_e4m3 *>(fp8_output), scale,
      elements);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -11;
}

int launch_quantize_rows(const void *bf16_rows, QuantTarget target, size_t elements,
                         cudaStream_t stream) {
  if (bf16_rows == nullptr || target.fp8_output == nullptr || target.scale == nullptr ||
      target.amax_bits == nullptr || elements == 0 || elements % 8 != 0) {
    return -1;
  }
  const unsigned blocks = static_cast<unsigned>((elements / 8 + 255) / 256);
  return launch_chained(quantize_rows_kernel, dim3(blocks), dim3(256), 0, stream, false,
                        static_cast<const __nv_bfloat16 *>(bf16_rows),
                        static_cast<const unsigned int *>(target.amax_bits), target.scale,
                        static_cast<unsigned char *>(target.fp8_output), elements) == cudaSuccess
             ? 0
             : -11;
}

int launch_embed_norm_quant(const void *embedding, const int *tokens, int vocabulary,
                            const void *norm_weight, void *hidden_out, QuantTarget target,
                            int rows, int width, float epsilon, unsigned int *clear_base,
                            int clear_words, cudaStream_t stream) {
  if (embedding == nullptr || tokens == nullptr || norm_weight == nullptr || hidden_out == nullptr)
    return -1;
  RowArguments arguments = base_arguments(target, width, epsilon);
  arguments.embedding = static_cast<const __nv_bfloat16 *>(embedding);
  arguments.tokens = tokens;
  arguments.vocabulary = vocabulary;
  arguments.norm_weight = static_cast<const __nv_bfloat16 *>(norm_weight);
  arguments.first_out = static_cast<__nv_bfloat16 *>(hidden_out);
  arguments.clear_base = clear_base;
  arguments.clear_words = clear_base == nullptr ? 0 : clear_words;
  return launch_rows<RowMode::embed_norm>(arguments, rows, stream);
}

int launch_embed_concat_quant(const void *embedding, const int *tokens, int vocabulary,
                              const void *hidden, const int *row_indices, QuantTarget target,
                              int rows, int width, cudaStream_t stream) {
  if (embedding == nullptr || tokens == nullptr || hidden == nullptr)
    return -1;
  RowArguments arguments = base_arguments(target, 2 * width, 0.0F);
  arguments.embedding = static_cast<const __nv_bfloat16 *>(embedding);
  arguments.tokens = tokens;
  arguments.vocabulary = vocabulary;
  arguments.input = static_cast<const __nv_bfloat16 *>(hidden);
  arguments.row_indices = row_indices;
  return launch_rows<RowMode::embed_concat>(arguments, rows, stream);
}

int launch_norm_quant(const void *input, const void *norm_weight, void *normalized_out,
                      QuantTarget target, int rows, int width, float epsilon,
                      cudaStream_t stream) {
  if (input == nullptr || norm_weight == nullptr)
    return -1;
  RowArguments arguments = base_arguments(target, width, epsilon);
  arguments.input = static_cast<const __nv_bfloat16 *>(input);
  arguments.norm_weight = static_cast<const __nv_bfloat16 *>(norm_weight);
  arguments.second_out = static_cast<__nv_bfloat16 *>(normalized_out);
  return launch_rows<RowMode::norm>(arguments, rows, stream);
}

int launch_quant(const void *input, const float *chunk_partials, int chunks,
                 const int *request_chunks, int rows_per_request, QuantTarget target, int rows,
                 int width, cudaStream_t stream) {
  if (input == nullptr && chunk_partials == nullptr)
    return -1;
  RowArguments arguments = base_arguments(target, width, 0.0F);
  arguments.input = static_cast<const __nv_bfloat16 *>(input);
  if (chunk_partials != nullptr && chunks > 0) {
    arguments.partial = chunk_partials;
    arguments.splits = chunks;
    arguments.valid_splits = request_chunks;
    arguments.rows_per_group = rows_per_request > 0 ? rows_per_request : 1;
  }
  return launch_rows<RowMode::plain>(arguments, rows, stream);
}

int launch_post_attention_norms_quant(const void *projected, PartialSource source,
                                      const void *norm_weight, const void *residual,
                                      const void *next_norm_weight, void *first_out,
                                      QuantTarget target, int rows, int width, float epsilon,
                                      cudaStream_t stream) {
  if ((projected == nullptr && source.partial == nullptr) || norm_weight == nullptr ||
      residual == nullptr || next_norm_weight == nullptr || first_out == nullptr) {
    return -1;
  }
  RowArguments arguments = base_arguments(target, width, epsilon);
  set_source(arguments, projected, source);
  arguments.norm_weight = static_cast<const __nv_bfloat16 *>(norm_weight);
  arguments.residual = static_cast<const __nv_bfloat16 *>(residual);
  arguments.next_norm_weight = static_cast<const __nv_bfloat16 *>(next_norm_weight);
  arguments.first_out = static_cast<__nv_bfloat16 *>(first_out);
  return launch_rows<RowMode::post_attention>(arguments, rows, stream);
}

int launch_geglu_quant(const void *packed_gate_up, TailSource tail, QuantTarget target, int rows,
                       int width, cudaStream_t stream) {
  if (packed_gate_up == nullptr)
    return -1;
  RowArguments arguments = base_arguments(target, width, 0.0F);
  arguments.input = static_cast<const __nv_bfloat16 *>(packed_gate_up);
  if (tail.partial != nullptr) {
    if (tail.splits <= 0 || tail.width <= 0 || tail.width % 8 != 0 || tail.first_column < width ||
        tail.first_column + tail.width != 2 * width || tail.input_scale == nullptr ||
        tail.weight_scale == nullptr) {
      return -1;
    }
    arguments.tail_partial = tail.partial;
    arguments.tail_splits = tail.splits;
    arguments.tail_first_column = tail.first_column;
    arguments.tail_width = tail.width;
    arguments.input_scale = tail.input_scale;
    arguments.weight_scale = tail.weight_scale;
  }
  return launch_rows<RowMode::geglu>(arguments, rows, stream);
}

int launch_layer_output_norm_quant(const void *down, PartialSource source, const void *norm_weight,
                                   const void *residual, const void *scalar, void *output,
                                   const void *next_norm_weight, void *next_out,
                                   QuantTarget target, int rows, int width, float epsilon,
                                   cudaStream_t stream) {
  if ((down == nullptr && source.partial == nullptr) || norm_weight == nullptr ||
      residual == nullptr || scalar == nullptr || output == nullptr ||
      next_norm_weight == nullptr) {
    return -1;
  }
  RowArguments arguments = base_arguments(target, width, epsilon);
  set_source(arguments, down, source);
  arguments.norm_weight = static_cast<const __nv_bfloat16 *>(norm_weight);
  arguments.residual = static_cast<const __nv_bfloat16 *>(residual);
  arguments.scalar = static_cast<const __nv_bfloat16 *>(scalar);
  arguments.first_out = static_cast<__nv_bfloat16 *>(output);
  arguments.next_norm_weight = static_cast<const __nv_bfloat16 *>(next_norm_weight);
  arguments.second_out = static_cast<__nv_bfloat16 *>(next_out);
  return launch_rows<RowMode::layer_output>(arguments, rows, stream);
}

} // namespace carat_b200
