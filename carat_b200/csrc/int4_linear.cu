// Weight-only INT4 linear (W4A16) for the verify step's small row counts.
//
// Contract (reference: Int4Bf16Linear, include/carat/linear.h:70-90, cuda/int4_bf16_linear.cu):
//   output[rows, N] = bf16( X_bf16[rows, K] . W[N, K]^T ),  W[n, k] = bf16(code[n, k] * scale[k / g, n]),
// fp32 accumulation.
//
// Same swapped-operand weight stream as the e4m3 linear (128 output features = UMMA M, padded
// activation rows = UMMA N, persistent CTAs walking tile x K-piece items), with one more stage
// between TMA and the tensor core: the 4-bit codes cannot feed tcgen05.mma together with bf16
// activations, so eight warps turn every [128 features x 128 K] tile of codes (8 KB, plus its 128
// group scales) into bf16 and store it into tensor memory (tcgen05.st), where the MMA warp takes
// it as the A operand (kind::f16, A in TMEM) against the bf16 activation boxes in shared memory.
// Keeping the converted weights out of shared memory matters: written there and read back by the
// tensor core they cost 64 KB of shared-memory traffic per K block on top of the 72 KB of TMA
// writes and B-operand reads, and the kernel was bound by shared-memory bandwidth (measured: no
// change when either TMA stream was switched off). Rings: codes + scales (TMA, deep, small),
// activations (TMA from L2), converted weights (four TMEM buffers of 64 columns, filled by two
// groups of four warps on alternate K blocks). The codes are read from HBM exactly once; that is
// half the bytes of the e4m3 weights, but the kernel is bound on the SM: at 128 padded rows the
// eight bf16 MMAs of a K block keep the tensor pipe busy about 700 cycles (an e4m3 MMA consumes 32
// bytes of a weight row, a bf16 MMA over 4-bit codes 8), and below 64 rows the conversion (shift,
// mask-or, bf16 subtract, bf16 multiply per pair of codes) is the limit.
#include "int4_linear.cuh"
#include "launch.cuh"
#include "linear_items.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>

#include <mutex>

namespace carat_b200 {
namespace {

constexpr int int4_threads = 480;        // warp 0 codes TMA, 1 MMA, 2 activations TMA, 3-6 epilogue,
constexpr int first_convert_warp = 7;    // 7-14 convert
constexpr int convert_warps = 8;
constexpr int code_tile_bytes = tile_features * 64;          // 128 features x 128 codes
constexpr int scale_tile_bytes = tile_features * 2;
constexpr int weight_buffers = 4;
constexpr int weight_columns = tile_k_elements / 2;          // TMEM columns of one converted K block

template <int padded_rows> struct Layout {
  static constexpr int input_box_bytes = padded_rows * 128;  // rows x 64 bf16
  static constexpr int input_stage_bytes = 2 * input_box_bytes;
  static constexpr int input_stages = padded_rows >= 128 ? 4 : 6;
  static constexpr int code_stages = 8;
  // Two accumulators, then the converted-weight buffers; allocations are powers of two.
  static constexpr int weight_column0 = 2 * padded_rows;
  static constexpr int used_columns = weight_column0 + weight_buffers * weight_columns;
  static constexpr int tmem_columns = used_columns <= 256 ? 256 : 512;
  static constexpr int dynamic_bytes = input_stages * input_stage_bytes +
                                       code_stages * (code_tile_bytes + scale_tile_bytes) + 1024;
};

template <int stages> struct Cursor {
  uint32_t stage{0};
  uint32_t phase{0};
  __device__ __forceinline__ void advance() {
    if (++stage == stages) {
      stage = 0;
      phase ^= 1U;
    }
  }
};

// Eight codes of one reordered word -> eight bf16 weights in K order. 0x4300 | c is the bf16 value
// 128 + c exactly (c < 16); minus 136 leaves the signed code; the product with the bf16 scale is
// rounded to bf16 once, which is the reference's bf16(code * scale).
__device__ __forceinline__ void convert_word(uint32_t word, __nv_bfloat162 scale_pair,
                                             uint32_t *out) {
  const uint32_t offset_bits = 0x43084308U;   // bf16 136.0 twice
  const __nv_bfloat162 offset = *reinterpret_cast<const __nv_bfloat162 *>(&offset_bits);
#pragma unroll
  for (int pair = 0; pair < 4; ++pair) {
    const uint32_t bits = ((word >> (4 * pair)) & 0x000F000FU) | 0x43004300U;
    __nv_bfloat162 value = *reinterpret_cast<const __nv_bfloat162 *>(&bits);
    value = __hmul2(__hsub2(value, offset), scale_pair);
    out[pair] = *reinterpret_cast<const uint32_t *>(&value);
  }
}

template <int padded_rows, int mode>
__global__ void __launch_bounds__(int4_threads, 1)
int4_linear_kernel(const __grid_constant__ CUtensorMap code_map,
                   const __grid_constant__ CUtensorMap scale_map,
                   const __grid_constant__ CUtensorMap input_map, const KernelArguments args,
                   const int group_shift) {
  using L = Layout<padded_rows>;
  constexpr uint32_t idesc = ptx::umma_idesc(1, 1, tile_features, padded_rows);
  constexpr uint32_t tmem_columns = L::tmem_columns;
  constexpr int barrier_count = 2 * L::code_stages + 2 * L::input_stages + 2 * weight_buffers + 4;

  extern __shared__ unsigned char shared_raw[];
  __shared__ __align__(8) unsigned long long barriers[barrier_count];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_word;

  const uint32_t raw_base = ptx::smem_u32(shared_raw);
  const uint32_t tiles_base = (raw_base + 1023U) & ~1023U;
  unsigned char *tiles_pointer = shared_raw + (tiles_base - raw_base);
  const uint32_t input_tiles = tiles_base;
  const uint32_t code_tiles = input_tiles + L::input_stages * L::input_stage_bytes;
  const uint32_t scale_tiles = code_tiles + L::code_stages * code_tile_bytes;

  const uint32_t code_full = ptx::smem_u32(&barriers[0]);
  const uint32_t code_empty = code_full + 8U * L::code_stages;
  const uint32_t input_full = code_empty + 8U * L::code_stages;
  const uint32_t input_empty = input_full + 8U * L::input_stages;
  const uint32_t weight_full = input_empty + 8U * L::input_stages;
  const uint32_t weight_empty = weight_full + 8U * weight_buffers;
  const uint32_t acc_full = weight_empty + 8U * weight_buffers;
  const uint32_t acc_empty = acc_full + 16U;

  const int warp = static_cast<int>(threadIdx.x) / 32;
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int items = item_count(args);
  const int first_item = static_cast<int>(blockIdx.x);
  const int item_stride = static_cast<int>(gridDim.x);
  volatile int *abort_flag = &abort_word;

  grid_dependency_launch();
  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int stage = 0; stage < L::code_stages; ++stage) {
      ptx::mbarrier_init(code_full + 8U * stage, 1);
      ptx::mbarrier_init(code_empty + 8U * stage, convert_warps / 2);
    }
    for (int stage = 0; stage < L::input_stages; ++stage) {
      ptx::mbarrier_init(input_full + 8U * stage, 1);
      ptx::mbarrier_init(input_empty + 8U * stage, 1);
    }
    for (int buffer = 0; buffer < weight_buffers; ++buffer) {
      ptx::mbarrier_init(weight_full + 8U * buffer, convert_warps / 2);
      ptx::mbarrier_init(weight_empty + 8U * buffer, 1);
    }
    for (int buffer = 0; buffer < 2; ++buffer) {
      ptx::mbarrier_init(acc_full + 8U * buffer, 1);
      ptx::mbarrier_init(acc_empty + 8U * buffer, 4);
    }
    ptx::fence_mbarrier_init();
    ptx::prefetch_tensormap(&code_map);
    ptx::prefetch_tensormap(&scale_map);
    ptx::prefetch_tensormap(&input_map);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&tmem_base_slot), tmem_columns);
    ptx::tmem_relinquish_alloc_permit();
  }
  ptx::tcgen05_fence_before_thread_sync();
  __syncthreads();
  ptx::tcgen05_fence_after_thread_sync();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // Codes and scales are static: this role never waits for the grid the launch depends on.
    if (lane == 0) {
      const uint64_t stream_policy = ptx::policy_evict_first();
      const uint64_t reuse_policy = ptx::policy_evict_last();
      Cursor<L::code_stages> cursor;
      bool healthy = true;
      for (int index = first_item; index < items && healthy; index += item_stride) {
        const WorkItem item = decode_item(args, index);
        const int feature0 = item.tile * tile_features;
        for (int block = item.k_begin; block < item.k_begin + item.k_count; ++block) {
          if (!ptx::mbarrier_wait_checked(code_empty + 8U * cursor.stage, cursor.phase ^ 1U, abort_flag,
                            args.device_error, 60)) {
            healthy = false;
            break;
          }
          const uint32_t full = code_full + 8U * cursor.stage;
          ptx::mbarrier_arrive_expect_tx(full, code_tile_bytes + scale_tile_bytes);
          ptx::tma_load_2d(code_tiles + cursor.stage * code_tile_bytes, &code_map, block * 64,
                           feature0, full, stream_policy);
          ptx::tma_load_2d(scale_tiles + cursor.stage * scale_tile_bytes, &scale_map, feature0,
                           block >> group_shift, full, reuse_policy);
          cursor.advance();
        }
      }
      if (!healthy) {
        // Copies already in flight must land before the CTA gives its shared memory back.
        for (uint32_t other = 0; other < static_cast<uint32_t>(L::code_stages); ++other)
          ptx::mbarrier_wait_bounded(code_full + 8U * other,
                                     other < cursor.stage ? cursor.phase : cursor.phase ^ 1U);
      }
    }
  } else if (warp == 2) {
    if (lane == 0) {
      const uint64_t reuse_policy = ptx::policy_evict_last();
      Cursor<L::input_stages> cursor;
      bool healthy = true;
      grid_dependency_wait();
      for (int index = first_item; index < items && healthy; index += item_stride) {
        const WorkItem item = decode_item(args, index);
        for (int block = item.k_begin; block < item.k_begin + item.k_count; ++block) {
          if (!ptx::mbarrier_wait_checked(input_empty + 8U * cursor.stage, cursor.phase ^ 1U, abort_flag,
                            args.device_error, 61)) {
            healthy = false;
            break;
          }
          const uint32_t full = input_full + 8U * cursor.stage;
          const uint32_t destination = input_tiles + cursor.stage * L::input_stage_bytes;
          ptx::mbarrier_arrive_expect_tx(full, L::input_stage_bytes);
          ptx::tma_load_2d(destination, &input_map, block * tile_k_elements, 0, full,
                           reuse_policy);
          ptx::tma_load_2d(destination + L::input_box_bytes, &input_map,
                           block * tile_k_elements + 64, 0, full, reuse_policy);
          cursor.advance();
        }
      }
      if (!healthy) {
        for (uint32_t other = 0; other < static_cast<uint32_t>(L::input_stages); ++other)
          ptx::mbarrier_wait_bounded(input_full + 8U * other,
                                     other < cursor.stage ? cursor.phase : cursor.phase ^ 1U);
      }
    }
  } else if (warp == 1) {
    // The whole warp walks the loop in lockstep and one elected lane issues: the loop state stays
    // warp-uniform, so descriptor and ring arithmetic can run on the uniform datapath instead of
    // competing with the converting warps for the integer pipe (with a single-lane loop the
    // issue cost per MMA was 70-90 cycles beside them).
    const uint64_t input_desc = ptx::umma_desc_k_major_sw128(input_tiles);
    const uint32_t desc_high = static_cast<uint32_t>(input_desc >> 32);
    const uint32_t input_low = static_cast<uint32_t>(input_desc);
    const uint32_t weight_base = tmem_base + L::weight_column0;
    Cursor<L::input_stages> input_cursor;
    Cursor<weight_buffers> weight_cursor;
    uint32_t buffer = 0;
    uint32_t buffer_phase = 0;
    bool healthy = true;
    for (int index = first_item; index < items && healthy; index += item_stride) {
      const WorkItem item = decode_item(args, index);
      const bool free_accumulator = ptx::mbarrier_wait_checked(acc_empty + 8U * buffer, buffer_phase ^ 1U,
                                                 abort_flag, args.device_error, 62);
      if (__all_sync(0xFFFFFFFFU, free_accumulator ? 1 : 0) == 0)
        break;
      ptx::tcgen05_fence_after_thread_sync();
      const uint32_t accumulator = tmem_base + buffer * padded_rows;
      for (int block = 0; block < item.k_count; ++block) {
        const bool ready =
            ptx::mbarrier_wait_checked(weight_full + 8U * weight_cursor.stage, weight_cursor.phase, abort_flag,
                         args.device_error, 63) &&
            ptx::mbarrier_wait_checked(input_full + 8U * input_cursor.stage, input_cursor.phase, abort_flag,
                         args.device_error, 64);
        if (__all_sync(0xFFFFFFFFU, ready ? 1 : 0) == 0) {
          healthy = false;
          break;
        }
        ptx::tcgen05_fence_after_thread_sync();
        const uint32_t a_columns = weight_base + weight_cursor.stage * weight_columns;
        const uint32_t b_low = input_low + input_cursor.stage * (L::input_stage_bytes >> 4);
        if (ptx::elect_one()) {
#pragma unroll
          for (int box = 0; box < 2; ++box) {
#pragma unroll
            for (int step = 0; step < 4; ++step) {
              // 16 bf16 along K: eight TMEM columns of A, 32 bytes inside B's swizzle atom (+2
              // in the address field).
              ptx::tcgen05_mma_f16_tmem_a(
                  accumulator, a_columns + (box * 4 + step) * 8,
                  b_low + box * (L::input_box_bytes >> 4) + 2 * step, desc_high, idesc,
                  (block > 0 || box > 0 || step > 0) ? 1U : 0U);
            }
          }
          ptx::tcgen05_commit(weight_empty + 8U * weight_cursor.stage);
          ptx::tcgen05_commit(input_empty + 8U * input_cursor.stage);
        }
        __syncwarp();
        weight_cursor.advance();
        input_cursor.advance();
      }
      if (healthy && ptx::elect_one())
        ptx::tcgen05_commit(acc_full + 8U * buffer);
      __syncwarp();
      buffer ^= 1U;
      if (buffer == 0)
        buffer_phase ^= 1U;
    }
  } else if (warp >= first_convert_warp) {
    // Thread -> feature row: a warp may touch only its own quarter of the TMEM lanes (warp index
    // mod 4), lane = feature row. The eight warps form two groups of four that take alternate K
    // blocks, so that on every scheduler one warp is converting while the other waits, loads or
    // stores (in lockstep all eight hit the integer and bf16 pipes at the same moment and leave
    // them idle the rest of the time). Code tiles arrive with the 64-byte swizzle (16-byte chunk
    // index xor bits 1-2 of the row), so the reads of a quarter warp touch eight bank groups.
    const int row = (warp & 3) * 32 + lane;
    const int group = (warp - first_convert_warp) >> 2;
    const uint32_t code_swizzle = static_cast<uint32_t>(row >> 1) & 3U;
    const unsigned char *code_row = tiles_pointer + (code_tiles - tiles_base) + row * 64;
    const unsigned char *scale_row = tiles_pointer + (scale_tiles - tiles_base) + row * 2;
    const uint32_t weight_lane =
        tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + L::weight_column0;
    int total_blocks = 0;
    for (int index = first_item; index < items; index += item_stride)
      total_blocks += decode_item(args, index).k_count;
    Cursor<L::code_stages> code_cursor;
    Cursor<weight_buffers> weight_cursor;
    if (group == 1) {
      code_cursor.advance();
      weight_cursor.advance();
    }
    for (int block = group; block < total_blocks; block += 2) {
      const bool ready =
          ptx::mbarrier_wait_checked(code_full + 8U * code_cursor.stage, code_cursor.phase, abort_flag,
                       args.device_error, 65) &&
          ptx::mbarrier_wait_checked(weight_empty + 8U * weight_cursor.stage, weight_cursor.phase ^ 1U,
                       abort_flag, args.device_error, 66);
      if (__all_sync(0xFFFFFFFFU, ready ? 1 : 0) == 0)
        break;
      const unsigned char *codes = code_row + code_cursor.stage * code_tile_bytes;
      uint4 raw[4];
#pragma unroll
      for (int chunk = 0; chunk < 4; ++chunk)
        raw[chunk] = *reinterpret_cast<const uint4 *>(
            codes + ((static_cast<uint32_t>(chunk) ^ code_swizzle) << 4));
      const __nv_bfloat16 scale = *reinterpret_cast<const __nv_bfloat16 *>(
          scale_row + code_cursor.stage * scale_tile_bytes);
      const __nv_bfloat162 scale_pair = __halves2bfloat162(scale, scale);
      ptx::tcgen05_fence_after_thread_sync();
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const uint32_t words[8] = {raw[2 * half].x,     raw[2 * half].y,     raw[2 * half].z,
                                   raw[2 * half].w,     raw[2 * half + 1].x, raw[2 * half + 1].y,
                                   raw[2 * half + 1].z, raw[2 * half + 1].w};
        uint32_t converted[32];
#pragma unroll
        for (int word = 0; word < 8; ++word)
          convert_word(words[word], scale_pair, converted + 4 * word);
        ptx::tmem_store_32x32b_x32(
            weight_lane + weight_cursor.stage * weight_columns + half * (weight_columns / 2),
            converted);
      }
      ptx::tmem_store_wait();
      ptx::tcgen05_fence_before_thread_sync();
      __syncwarp();
      if (lane == 0) {
        ptx::mbarrier_arrive(weight_full + 8U * weight_cursor.stage);
        ptx::mbarrier_arrive(code_empty + 8U * code_cursor.stage);
      }
      code_cursor.advance();
      code_cursor.advance();
      weight_cursor.advance();
      weight_cursor.advance();
    }
  } else {
    const int quarter = warp & 3;  // TMEM lane group this warp may read
    grid_dependency_wait();
    int local = 0;
    for (int index = first_item; index < items; index += item_stride, ++local) {
      const WorkItem item = decode_item(args, index);
      const int buffer = local & 1;
      const uint32_t use = static_cast<uint32_t>(local >> 1);
      const bool ready = ptx::mbarrier_wait_checked(acc_full + 8U * buffer, use & 1U, abort_flag,
                                      args.device_error, 67);
      if (__all_sync(0xFFFFFFFFU, ready ? 1 : 0) == 0)
        break;
      ptx::tcgen05_fence_after_thread_sync();
      const int feature = item.tile * tile_features + quarter * 32 + lane;
      const uint32_t lane_address =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buffer * padded_rows;
      // Where this item's values go: bf16 output, or fp32 pieces of a split / tail tile.
      float *pieces = nullptr;
      size_t piece_stride = 0;
      if constexpr (mode == 1) {
        pieces = args.partial + static_cast<size_t>(item.piece) * args.rows * args.output_width +
                 feature;
        piece_stride = static_cast<size_t>(args.output_width);
      } else if (item.tail) {
        const int tail_width = args.tail_tiles * tile_features;
        pieces = args.tail_partial + static_cast<size_t>(item.piece) * args.rows * tail_width +
                 (feature - (args.tiles - args.tail_tiles) * tile_features);
        piece_stride = static_cast<size_t>(tail_width);
      }
#pragma unroll
      for (int chunk = 0; chunk < padded_rows / 32; ++chunk) {
        if (chunk * 32 < args.rows) {  // warp-uniform
          uint32_t raw[32];
          ptx::tmem_load_32x32b_x32(lane_address + chunk * 32, raw);
          ptx::tmem_load_wait();
          if (feature < args.output_width) {
            if (pieces != nullptr) {
#pragma unroll
              for (int column = 0; column < 32; ++column) {
                const int row = chunk * 32 + column;
                if (row < args.rows)
                  pieces[static_cast<size_t>(row) * piece_stride] = __uint_as_float(raw[column]);
              }
            } else {
#pragma unroll
              for (int column = 0; column < 32; ++column) {
                const int row = chunk * 32 + column;
                if (row < args.rows)
                  args.output[static_cast<size_t>(row) * args.output_width + feature] =
                      __float2bfloat16_rn(__uint_as_float(raw[column]));
              }
            }
          }
        }
      }
      ptx::tcgen05_fence_before_thread_sync();
      __syncwarp();
      if (lane == 0)
        ptx::mbarrier_arrive(acc_empty + 8U * buffer);
    }
  }

  ptx::tcgen05_fence_before_thread_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tcgen05_fence_after_thread_sync();
    ptx::tmem_dealloc(tmem_base, tmem_columns);
  }
}

// output = bf16(sum of fp32 pieces); `first_column` / `piece_width` select a column range of the
// output rows (the whole row for split-K, the tail columns for the K-cut tail round).
__global__ void int4_finalize_kernel(const float *partial, __nv_bfloat16 *output, int pieces,
                                     int rows, int piece_width, int output_width,
                                     int first_column) {
  grid_dependency_launch();
  grid_dependency_wait();
  const size_t elements = static_cast<size_t>(rows) * piece_width;
  for (size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
       index < elements; index += static_cast<size_t>(blockDim.x) * gridDim.x) {
    float sum = 0.0F;
    for (int piece = 0; piece < pieces; ++piece)
      sum += partial[static_cast<size_t>(piece) * elements + index];
    const size_t row = index / piece_width;
    const size_t column = index - row * piece_width;
    output[row * output_width + first_column + column] = __float2bfloat16_rn(sum);
  }
}

__device__ __forceinline__ float block_max_256(float value, float *scratch) {
  for (int offset = 16; offset > 0; offset >>= 1)
    value = fmaxf(value, __shfl_xor_sync(0xFFFFFFFFU, value, offset));
  __syncthreads();   // the previous group's readers are done with scratch
  if ((threadIdx.x & 31U) == 0U)
    scratch[threadIdx.x >> 5U] = value;
  __syncthreads();
  float total = 0.0F;
  for (unsigned int warp = 0; warp < blockDim.x / 32U; ++warp)
    total = fmaxf(total, scratch[warp]);
  return total;
}

// One CTA per output row, one thread per K value of a group.
__global__ void int4_quantize_kernel(const __nv_bfloat16 *weight, unsigned char *packed,
                                     __nv_bfloat16 *scales, int output_width, int input_width,
                                     int group_width) {
  __shared__ float scratch[8];
  const int row = static_cast<int>(blockIdx.x);
  const size_t row_base = static_cast<size_t>(row) * input_width;
  const int groups = input_width / group_width;
  for (int group = 0; group < groups; ++group) {
    const int column = group * group_width + static_cast<int>(threadIdx.x);
    const float value = __bfloat162float(weight[row_base + column]);
    const float maximum = block_max_256(fabsf(value), scratch);
    const __nv_bfloat16 encoded =
        __float2bfloat16_rn(maximum > 0.0F ? __fdiv_rn(maximum, 7.0F) : 1.0F);
    const float scale = __bfloat162float(encoded);
    if (threadIdx.x == 0U)
      scales[static_cast<size_t>(group) * output_width + row] = encoded;
    const int code = max(-7, min(7, __float2int_rn(__fdiv_rn(value, scale))));
    const int neighbour = __shfl_down_sync(0xFFFFFFFFU, code, 1);
    if ((threadIdx.x & 1U) == 0U)
      packed[(row_base + column) / 2] =
          static_cast<unsigned char>((code & 0xF) | ((neighbour & 0xF) << 4));
  }
}

__global__ void int4_reorder_kernel(const uint32_t *packed, uint32_t *reordered, size_t words) {
  for (size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; index < words;
       index += static_cast<size_t>(blockDim.x) * gridDim.x) {
    const uint32_t word = packed[index] ^ 0x88888888U;   // two's complement -> code + 8
    uint32_t out = 0U;
#pragma unroll
    for (int pair = 0; pair < 4; ++pair) {
      out |= ((word >> (8 * pair)) & 0xFU) << (4 * pair);
      out |= ((word >> (8 * pair + 4)) & 0xFU) << (4 * pair + 16);
    }
    reordered[index] = out;
  }
}

__global__ void int4_simt_check_kernel(const __nv_bfloat16 *input, const unsigned char *packed,
                                       const __nv_bfloat16 *scales, __nv_bfloat16 *output, int rows,
                                       int input_width, int output_width, int group_width) {
  const int feature = static_cast<int>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int row = static_cast<int>(blockIdx.y);
  if (feature >= output_width || row >= rows)
    return;
  const __nv_bfloat16 *x = input + static_cast<size_t>(row) * input_width;
  const unsigned char *codes = packed + static_cast<size_t>(feature) * input_width / 2;
  float sum = 0.0F;
  for (int k = 0; k < input_width; ++k) {
    const int nibble = (codes[k / 2] >> (4 * (k & 1))) & 0xF;
    const int code = nibble >= 8 ? nibble - 16 : nibble;
    const float scale =
        __bfloat162float(scales[static_cast<size_t>(k / group_width) * output_width + feature]);
    const float weight = __bfloat162float(__float2bfloat16_rn(static_cast<float>(code) * scale));
    sum += __bfloat162float(x[k]) * weight;
  }
  output[static_cast<size_t>(row) * output_width + feature] = __float2bfloat16_rn(sum);
}

bool encode_map(CUtensorMap *map, CUtensorMapDataType type, const void *base, uint64_t inner,
                uint64_t outer, uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer,
                CUtensorMapSwizzle swizzle) {
  const EncodeTiled encode = encode_tiled_entry();
  if (encode == nullptr)
    return false;
  const cuuint64_t dimensions[2] = {inner, outer};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t element_strides[2] = {1, 1};
  return encode(map, type, 2, const_cast<void *>(base), dimensions, strides, box, element_strides,
                CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int padded_rows, int mode>
int launch_variant(const Int4LinearPlan &plan, const KernelArguments &arguments,
                   cudaStream_t stream) {
  constexpr int dynamic_bytes = Layout<padded_rows>::dynamic_bytes;
  static_assert(dynamic_bytes <= 227 * 1024, "shared memory budget");
  static PerDeviceOnce configured;
  if (configured.run([] {
        return cudaFuncSetAttribute(int4_linear_kernel<padded_rows, mode>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, dynamic_bytes);
      }) != cudaSuccess) {
    return -10;
  }
  const LinearPlan &schedule = plan.schedule;
  const int items = (schedule.tiles - arguments.tail_tiles) * arguments.splits +
                    arguments.tail_tiles * arguments.tail_splits;
  const int ctas = items < schedule.ctas ? items : schedule.ctas;
  return launch_chained(int4_linear_kernel<padded_rows, mode>, dim3(static_cast<unsigned>(ctas)),
                        dim3(int4_threads), dynamic_bytes, stream, false, schedule.weight_map,
                        plan.scale_map, schedule.input_map, arguments,
                        plan.group_shift) == cudaSuccess
             ? 0
             : -11;
}

template <int mode>
int launch_mode(const Int4LinearPlan &plan, const KernelArguments &arguments, cudaStream_t stream) {
  switch (plan.schedule.padded_rows) {
  case 32:
    return launch_variant<32, mode>(plan, arguments, stream);
  case 64:
    return launch_variant<64, mode>(plan, arguments, stream);
  case 128:
    return launch_variant<128, mode>(plan, arguments, stream);
  default:
    return -12;
  }
}

KernelArguments base_arguments(const LinearPlan &plan, int *device_error, bool split) {
  KernelArguments arguments{};
  arguments.device_error = device_error;
  arguments.rows = plan.rows;
  arguments.output_width = plan.output_width;
  arguments.tiles = plan.tiles;
  arguments.k_blocks = plan.k_blocks;
  arguments.splits = split ? plan.splits : 1;
  arguments.k_blocks_per_split = split ? plan.k_blocks_per_split : plan.k_blocks;
  arguments.tail_tiles = 0;
  arguments.tail_splits = 1;
  arguments.tail_k_blocks_per_split = plan.k_blocks;
  return arguments;
}

int launch_finalize(const float *partial, void *bf16_output, int pieces, int rows, int piece_width,
                    int output_width, int first_column, cudaStream_t stream) {
  const size_t elements = static_cast<size_t>(rows) * piece_width;
  const int blocks = static_cast<int>((elements + 255) / 256);
  return launch_chained(int4_finalize_kernel, dim3(blocks < 1184 ? blocks : 1184), dim3(256), 0,
                        stream, false, partial, static_cast<__nv_bfloat16 *>(bf16_output), pieces,
                        rows, piece_width, output_width, first_column) == cudaSuccess
             ? 0
             : -11;
}

std::size_t partial_bytes(const LinearPlan &plan) {
  if (plan.splits > 1)
    return sizeof(float) * static_cast<std::size_t>(plan.splits) * plan.rows * plan.output_width;
  return plan.tail_tiles <= 0 ? 0
                              : sizeof(float) * static_cast<std::size_t>(plan.tail_splits) *
                                    plan.rows * plan.tail_tiles * tile_features;
}

} // namespace

int launch_int4_quantize(const void *bf16_weight, void *packed_row_major, void *bf16_scales,
                         int output_width, int input_width, int group_width,
                         cudaStream_t stream) {
  if (bf16_weight == nullptr || packed_row_major == nullptr || bf16_scales == nullptr ||
      output_width <= 0 || input_width <= 0 || (group_width != 128 && group_width != 256) ||
      input_width % group_width != 0) {
    return -1;
  }
  int4_quantize_kernel<<<static_cast<unsigned>(output_width), static_cast<unsigned>(group_width),
                         0, stream>>>(static_cast<const __nv_bfloat16 *>(bf16_weight),
                                      static_cast<unsigned char *>(packed_row_major),
                                      static_cast<__nv_bfloat16 *>(bf16_scales), output_width,
                                      input_width, group_width);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -11;
}

int launch_int4_reorder(const void *packed_row_major, void *reordered, std::size_t bytes,
                        cudaStream_t stream) {
  if (packed_row_major == nullptr || reordered == nullptr || bytes == 0 || bytes % 4 != 0)
    return -1;
  const size_t words = bytes / 4;
  const size_t wanted = (words + 255) / 256;
  int4_reorder_kernel<<<static_cast<unsigned>(wanted < 4096 ? wanted : 4096), 256, 0, stream>>>(
      static_cast<const uint32_t *>(packed_row_major), static_cast<uint32_t *>(reordered), words);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -11;
}

std::size_t int4_linear_partial_bytes(const Int4LinearPlan &plan) {
  return partial_bytes(plan.schedule);
}

std::size_t int4_linear_partial_bytes_for(int rows, int input_width, int output_width) {
  if (rows <= 0 || rows > 128 || input_width <= 0 || output_width <= 0)
    return 0;
  LinearPlan plan{};
  schedule_linear(&plan, rows, input_width, output_width, 0);
  return partial_bytes(plan);
}

int make_int4_linear_plan(Int4LinearPlan *plan, const void *bf16_input,
                          const void *reordered_weight, const void *bf16_scales, int rows,
                          int input_width, int output_width, int group_width,
                          int requested_splits, const char **error) {
  const auto fail = [&](const char *message, int code) {
    if (error != nullptr)
      *error = message;
    return code;
  };
  if (plan == nullptr || bf16_input == nullptr || reordered_weight == nullptr ||
      bf16_scales == nullptr || rows <= 0 || input_width <= 0 || output_width <= 0) {
    return fail("invalid BF16 INT4 linear weight shape", -1);
  }
  if (rows > 128)
    return fail("invalid BF16 INT4 linear activation shape", -2);
  if ((group_width != 128 && group_width != 256) || input_width % group_width != 0 ||
      output_width % 8 != 0) {
    return fail("invalid BF16 INT4 linear weight shape", -3);
  }
  if ((reinterpret_cast<uintptr_t>(bf16_input) & 15U) != 0 ||
      (reinterpret_cast<uintptr_t>(reordered_weight) & 15U) != 0 ||
      (reinterpret_cast<uintptr_t>(bf16_scales) & 15U) != 0) {
    return fail("BF16 INT4 linear operands must be 16-byte aligned", -4);
  }
  Int4LinearPlan result{};
  schedule_linear(&result.schedule, rows, input_width, output_width, requested_splits);
  result.group_shift = group_width == 256 ? 1 : 0;
  const uint64_t k = static_cast<uint64_t>(input_width);
  const uint64_t n = static_cast<uint64_t>(output_width);
  if (!encode_map(&result.schedule.weight_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, reordered_weight,
                  k / 2, n, k / 2, 64, tile_features, CU_TENSOR_MAP_SWIZZLE_64B) ||
      !encode_map(&result.scale_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, bf16_scales, n,
                  k / static_cast<uint64_t>(group_width), n * 2, tile_features, 1,
                  CU_TENSOR_MAP_SWIZZLE_NONE) ||
      !encode_map(&result.schedule.input_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, bf16_input, k,
                  static_cast<uint64_t>(rows), k * 2, 64,
                  static_cast<uint32_t>(result.schedule.padded_rows),
                  CU_TENSOR_MAP_SWIZZLE_128B)) {
    return fail("cuTensorMapEncodeTiled failed", -5);
  }
  *plan = result;
  return 0;
}

int launch_int4_linear_partial(const Int4LinearPlan &plan, float *partial, int *device_error,
                               cudaStream_t stream) {
  if (partial == nullptr)
    return -13;
  KernelArguments arguments = base_arguments(plan.schedule, device_error, true);
  arguments.partial = partial;
  return launch_mode<1>(plan, arguments, stream);
}

int launch_int4_linear_bf16_tail(const Int4LinearPlan &plan, void *bf16_output, float *tail_partial,
                                 int *device_error, cudaStream_t stream) {
  const LinearPlan &schedule = plan.schedule;
  if (schedule.splits != 1 || schedule.tail_tiles <= 0 || tail_partial == nullptr)
    return -13;
  KernelArguments arguments = base_arguments(schedule, device_error, false);
  arguments.output = static_cast<__nv_bfloat16 *>(bf16_output);
  arguments.tail_partial = tail_partial;
  arguments.tail_tiles = schedule.tail_tiles;
  arguments.tail_splits = schedule.tail_splits;
  arguments.tail_k_blocks_per_split = schedule.tail_k_blocks_per_split;
  return launch_mode<0>(plan, arguments, stream);
}

int launch_int4_linear_bf16(const Int4LinearPlan &plan, void *bf16_output, float *partial,
                            int *device_error, cudaStream_t stream) {
  const LinearPlan &schedule = plan.schedule;
  if (schedule.splits == 1 && schedule.tail_tiles > 0 && partial != nullptr) {
    const int status = launch_int4_linear_bf16_tail(plan, bf16_output, partial, device_error, stream);
    if (status != 0)
      return status;
    const int tail_width = schedule.tail_tiles * tile_features;
    return launch_finalize(partial, bf16_output, schedule.tail_splits, schedule.rows, tail_width,
                           schedule.output_width, schedule.output_width - tail_width, stream);
  }
  if (schedule.splits == 1) {
    KernelArguments arguments = base_arguments(schedule, device_error, false);
    arguments.output = static_cast<__nv_bfloat16 *>(bf16_output);
    return launch_mode<0>(plan, arguments, stream);
  }
  const int status = launch_int4_linear_partial(plan, partial, device_error, stream);
  if (status != 0)
    return status;
  return launch_finalize(partial, bf16_output, schedule.splits, schedule.rows,
                         schedule.output_width, schedule.output_width, 0, stream);
}

int launch_int4_linear_simt_check(const void *bf16_input, const void *packed_row_major,
                                  const void *bf16_scales, void *bf16_output, int rows,
                                  int input_width, int output_width, int group_width,
                                  cudaStream_t stream) {
  const dim3 grid(static_cast<unsigned>((output_width + 127) / 128), static_cast<unsigned>(rows));
  int4_simt_check_kernel<<<grid, 128, 0, stream>>>(
      static_cast<const __nv_bfloat16 *>(bf16_input),
      static_cast<const unsigned char *>(packed_row_major),
      static_cast<const __nv_bfloat16 *>(bf16_scales), static_cast<__nv_bfloat16 *>(bf16_output),
      rows, input_width, output_width, group_width);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -11;
}

} // namespace carat_b200
