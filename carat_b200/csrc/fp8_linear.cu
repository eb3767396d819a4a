// Weight-streaming FP8 (e4m3 x e4m3 -> fp32 -> bf16) linear for the verify step's small row counts.
//
// Contract (reference: cuda/linear.cu:645-803 Fp8Linear::run, tensor scaling):
//   output[rows, N] = bf16( (x_scale * w_scale) * X_e4m3[rows, K] . W_e4m3[N, K]^T ), fp32 accumulate.
//
// The problem is HBM-bound (rows <= 256 means <= 512 FLOP per weight byte), so the design is a
// weight stream: the operands are swapped so that 128 output features form the UMMA M dimension
// and the (zero-padded) activation rows the UMMA N dimension. One CTA owns one 128-feature tile
// over one K range; a TMA producer warp keeps a multi-stage ring of 128-byte-swizzled
// [128 x 128 B] weight tiles and [rows x 128 B] activation tiles in flight, a single thread issues
// tcgen05.mma (kind::f8f6f4, K = 32) into a TMEM accumulator, and four epilogue warps read the
// accumulator with tcgen05.ld. Weights are read exactly once with an evict-first policy; the
// activation matrix is re-read from L2 by every tile with an evict-last policy.
#include "fp8_linear.cuh"
#include "context.cuh"
#include "launch.cuh"
#include "linear_items.cuh"
#include "ptx.cuh"
#include "row_ops.cuh"

#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace carat_b200 {
namespace {

constexpr int tile_k_bytes = 128;   // one 128B swizzle atom of e4m3 per row
constexpr int umma_k = 32;
constexpr int linear_threads = 192; // warp 0 TMA, warp 1 MMA + TMEM, warps 2-5 epilogue
constexpr int weight_tile_bytes = tile_features * tile_k_bytes;
constexpr int shared_budget = 200 * 1024;

__host__ __device__ constexpr int stages_for(int padded_rows) {
  const int per_stage = weight_tile_bytes + padded_rows * tile_k_bytes;
  const int fit = shared_budget / per_stage;
  return fit > 8 ? 8 : fit;
}

__device__ __forceinline__ unsigned int orderable_bf16(float rounded) {
  // Monotonic map of a bf16-representable float to 16 bits; NaN sorts below everything, matching
  // a comparison chain that never selects NaN.
  if (rounded != rounded)
    return 0U;
  const unsigned int bits = __float_as_uint(rounded) >> 16;
  return (bits & 0x8000U) ? (~bits & 0xFFFFU) : (bits | 0x8000U);
}

// Finishes 32 accumulator columns (activation rows chunk*32 ..) of one feature.
template <int mode>
__device__ __forceinline__ void finish_chunk(const KernelArguments &args, const float (&values)[32],
                                             int chunk, int feature, int feature_base, int lane,
                                             float scale, unsigned long long *row_best) {
  if constexpr (mode == 0) {
    if (feature < args.output_width) {
#pragma unroll
      for (int column = 0; column < 32; ++column) {
        const int row = chunk * 32 + column;
        if (row < args.rows)
          args.output[static_cast<size_t>(row) * args.output_width + feature] =
              __float2bfloat16_rn(values[column] * scale);
      }
    }
  } else {
    unsigned long long chunk_best = 0ULL;
#pragma unroll
    for (int column = 0; column < 32; ++column) {
      const float rounded = __bfloat162float(__float2bfloat16_rn(values[column] * scale));
      // Out-of-range features lose to everything; ties inside the warp go to the lowest lane,
      // which is the lowest feature index.
      const unsigned int key =
          feature < args.output_width
              ? ((orderable_bf16(rounded) + 1U) << 8) | static_cast<unsigned int>(31 - lane)
              : 0U;
      const unsigned int winner = __reduce_max_sync(0xFFFFFFFFU, key);
      if (lane == column && winner != 0U) {
        const unsigned int winner_feature =
            static_cast<unsigned int>(feature_base) + (31U - (winner & 31U));
        chunk_best = (static_cast<unsigned long long>(winner >> 8) << 32) |
                     static_cast<unsigned long long>(~winner_feature);
      }
    }
    const int row = chunk * 32 + lane;
    if (row < args.rows && chunk_best != 0ULL)
      atomicMax(&row_best[row], chunk_best);
  }
}

// Gated epilogue for 32 accumulator columns (activation rows chunk*32 ..). Thread t of the 128
// epilogue threads holds gate feature t (t < 64) or up feature t - 64 of the tile; the pair
// (t, t ^ 64) belongs to one activated column. Both round their sums to bf16 like the plain
// epilogue, hand each other half of the rows through shared memory, and each finishes sixteen
// rows: bf16(gelu(gate) * up), the arithmetic of the stand-alone GeGLU kernel.
__device__ __forceinline__ void gated_chunk(const KernelArguments &args, const float (&values)[32],
                                            int chunk, int tile, int quarter, int lane, float scale,
                                            __nv_bfloat16 *exchange, float &amax) {
  const bool gate_side = quarter < 2;
  const int thread = quarter * 32 + lane;
  // The gate side finishes rows 0..15 of the chunk and hands over its rows 16..31; the up side
  // the other way round. Static indices throughout, so everything stays in registers.
  __nv_bfloat16 kept[16];
  __align__(16) __nv_bfloat16 given[16];
#pragma unroll
  for (int column = 0; column < 16; ++column) {
    const __nv_bfloat16 low = __float2bfloat16_rn(values[column] * scale);
    const __nv_bfloat16 high = __float2bfloat16_rn(values[16 + column] * scale);
    kept[column] = gate_side ? low : high;
    given[column] = gate_side ? high : low;
  }
  uint4 *mine = reinterpret_cast<uint4 *>(exchange + thread * 16);
  mine[0] = *reinterpret_cast<const uint4 *>(&given[0]);
  mine[1] = *reinterpret_cast<const uint4 *>(&given[8]);
  asm volatile("bar.sync 1, 128;" ::: "memory");
  __align__(16) __nv_bfloat16 other[16];
  const uint4 *theirs = reinterpret_cast<const uint4 *>(exchange + (thread ^ 64) * 16);
  *reinterpret_cast<uint4 *>(&other[0]) = theirs[0];
  *reinterpret_cast<uint4 *>(&other[8]) = theirs[1];
  __nv_bfloat16 *destination =
      args.output + static_cast<size_t>(tile) * 64 + (quarter & 1) * 32 + lane;
  const int first_row = chunk * 32 + (gate_side ? 0 : 16);
#pragma unroll
  for (int column = 0; column < 16; ++column) {
    const float gate = __bfloat162float(gate_side ? kept[column] : other[column]);
    const float up = __bfloat162float(gate_side ? other[column] : kept[column]);
    const __nv_bfloat16 activated = __float2bfloat16_rn(gelu_tanh(gate) * up);
    const int row = first_row + column;
    if (row < args.rows) {
      destination[static_cast<size_t>(row) * args.gated_width] = activated;
      amax = fmaxf(amax, fabsf(__bfloat162float(activated)));
    }
  }
}

// `wide` = bf16 operands (kind::f16, 64 K elements per 128-byte block) instead of e4m3
// (kind::f8f6f4, 128 per block). Everything else is shared: both consume one 128-byte swizzle atom
// per row and block in four MMAs of 32 bytes of K.
template <int padded_rows, int mode, bool wide>
__global__ void __launch_bounds__(linear_threads, 1)
fp8_linear_kernel(const __grid_constant__ CUtensorMap weight_map,
                  const __grid_constant__ CUtensorMap input_map, const KernelArguments args) {
  constexpr int stages = stages_for(padded_rows);
  constexpr int input_tile_bytes = padded_rows * tile_k_bytes;
  constexpr uint32_t stage_bytes = weight_tile_bytes + input_tile_bytes;
  constexpr uint32_t idesc = wide ? ptx::umma_idesc(1, 1, tile_features, padded_rows)
                                  : ptx::umma_idesc(0, 0, tile_features, padded_rows);
  // Two accumulators; tensor-memory allocations are powers of two (192 padded rows take 512).
  constexpr uint32_t tmem_columns = 2 * padded_rows < 32 ? 32 : 2 * padded_rows > 256 ? 512 : 2 * padded_rows;

  extern __shared__ unsigned char shared_raw[];
  __shared__ __align__(8) unsigned long long barriers[2 * stages + 4];
  __shared__ uint32_t tmem_base_slot;
  __shared__ unsigned long long row_best[mode == 2 ? padded_rows : 1];
  __shared__ int epilogue_gave_up;   // modes 2, 3: set by an epilogue warp whose wait ran out
  __shared__ int tail_is_last;       // mode 3: this CTA finished the last K piece of a tail tile
  __shared__ __align__(16) __nv_bfloat16 exchange[mode == 3 ? 2 * 128 * 16 : 8];

  const uint32_t tiles_base = (ptx::smem_u32(shared_raw) + 1023U) & ~1023U;
  const uint32_t weight_tiles = tiles_base;
  const uint32_t input_tiles = tiles_base + stages * weight_tile_bytes;
  const uint32_t full_bar = ptx::smem_u32(&barriers[0]);
  const uint32_t empty_bar = ptx::smem_u32(&barriers[stages]);
  const uint32_t acc_full_bar = ptx::smem_u32(&barriers[2 * stages]);
  const uint32_t acc_empty_bar = ptx::smem_u32(&barriers[2 * stages + 2]);

  const int warp = static_cast<int>(threadIdx.x) / 32;
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int items = item_count(args);
  const int first_item = static_cast<int>(blockIdx.x);
  const int item_stride = static_cast<int>(gridDim.x);

  grid_dependency_launch();
  if (threadIdx.x == 0) {
    for (int stage = 0; stage < stages; ++stage) {
      ptx::mbarrier_init(full_bar + 8U * stage, 1);
      ptx::mbarrier_init(empty_bar + 8U * stage, 1);
    }
    for (int buffer = 0; buffer < 2; ++buffer) {
      ptx::mbarrier_init(acc_full_bar + 8U * buffer, 1);
      ptx::mbarrier_init(acc_empty_bar + 8U * buffer, 4);
    }
    ptx::fence_mbarrier_init();
    ptx::prefetch_tensormap(&weight_map);
    ptx::prefetch_tensormap(&input_map);
  }
  if constexpr (mode == 2) {
    for (int row = static_cast<int>(threadIdx.x); row < padded_rows; row += linear_threads)
      row_best[row] = 0ULL;
  }
  if (threadIdx.x == 0)
    epilogue_gave_up = 0;
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&tmem_base_slot), tmem_columns);
    ptx::tmem_relinquish_alloc_permit();
  }
  ptx::tcgen05_fence_before_thread_sync();
  __syncthreads();
  ptx::tcgen05_fence_after_thread_sync();
  const uint32_t tmem_base = tmem_base_slot;

  // The TMA and MMA roles are single threads whose loop bodies are the critical path (a dependent
  // instruction costs several cycles and nothing hides it), so both keep a running ring cursor and
  // precomputed descriptor words instead of dividing and rebuilding descriptors per K block.
  if (warp == 0) {
    if (lane == 0) {
      const uint64_t stream_policy = ptx::policy_evict_first();
      const uint64_t reuse_policy = ptx::policy_evict_last();
      uint32_t stage = 0;
      uint32_t phase = 0;
      bool healthy = true;
      // The weights are static: the first ring of weight tiles is requested before the grid this
      // launch depends on has finished. The activation tiles of those stages follow once it has.
      // Plain tiles are one [128 x 128 B] box; a gated tile is two [64 x 128 B] boxes, its gate
      // rows and the up rows gated_width further down, stacked in the same stage.
      const auto load_weights = [&](uint32_t destination, int k_byte, int tile, uint32_t bar) {
        if constexpr (mode == 3) {
          ptx::tma_load_2d(destination, &weight_map, k_byte, tile * (tile_features / 2), bar,
                           stream_policy);
          ptx::tma_load_2d(destination + weight_tile_bytes / 2, &weight_map, k_byte,
                           args.gated_width + tile * (tile_features / 2), bar, stream_policy);
        } else {
          ptx::tma_load_2d(destination, &weight_map, k_byte, tile * tile_features, bar,
                           stream_policy);
        }
      };
      int early = 0;
      if (first_item < items) {
        const WorkItem item = decode_item(args, first_item);
        early = min(item.k_count, stages);
        for (int block = 0; block < early; ++block) {
          ptx::mbarrier_arrive_expect_tx(full_bar + 8U * block, stage_bytes);
          load_weights(weight_tiles + block * weight_tile_bytes,
                       (item.k_begin + block) * tile_k_bytes, item.tile, full_bar + 8U * block);
        }
      }
      grid_dependency_wait();
      for (int index = first_item; index < items && healthy; index += item_stride) {
        const WorkItem item = decode_item(args, index);
        int k_byte = item.k_begin * tile_k_bytes;
        for (int block = 0; block < item.k_count; ++block, k_byte += tile_k_bytes) {
          const uint32_t full = full_bar + 8U * stage;
          if (early > 0) {
            --early;     // this stage's weight tile is already on its way
          } else {
            if (!ptx::mbarrier_wait_fast(empty_bar + 8U * stage, phase ^ 1U)) {
              healthy = false;
              atomicExch(args.device_error, 1);
              break;
            }
            ptx::mbarrier_arrive_expect_tx(full, stage_bytes);
            load_weights(weight_tiles + stage * weight_tile_bytes, k_byte, item.tile, full);
          }
          ptx::tma_load_2d(input_tiles + stage * input_tile_bytes, &input_map, k_byte, 0, full,
                           reuse_policy);
          if (++stage == stages) {
            stage = 0;
            phase ^= 1U;
          }
        }
      }
      if (!healthy) {
        // Let copies already in flight land before the CTA gives its shared memory back: wait
        // for the phase each stage was last armed for.
        for (uint32_t other = 0; other < static_cast<uint32_t>(stages); ++other)
          ptx::mbarrier_wait_bounded(full_bar + 8U * other, other < stage ? phase : phase ^ 1U);
      }
    }
  } else if (warp == 1) {
    // The whole warp walks the loop in lockstep and one elected lane issues, so the loop state
    // stays warp-uniform (descriptor and ring arithmetic on the uniform datapath).
    const uint64_t weight_desc = ptx::umma_desc_k_major_sw128(weight_tiles);
    const uint64_t input_desc = ptx::umma_desc_k_major_sw128(input_tiles);
    const uint32_t desc_high = static_cast<uint32_t>(weight_desc >> 32);
    const uint32_t weight_low = static_cast<uint32_t>(weight_desc);
    const uint32_t input_low = static_cast<uint32_t>(input_desc);
    uint32_t stage = 0;
    uint32_t phase = 0;
    uint32_t buffer = 0;
    uint32_t buffer_phase = 0;
    bool healthy = true;
    for (int index = first_item; index < items && healthy; index += item_stride) {
      const WorkItem item = decode_item(args, index);
      const bool free_accumulator =
          ptx::mbarrier_wait_fast(acc_empty_bar + 8U * buffer, buffer_phase ^ 1U);
      if (__all_sync(0xFFFFFFFFU, free_accumulator ? 1 : 0) == 0) {
        if (lane == 0)
          atomicExch(args.device_error, 4);
        break;
      }
      ptx::tcgen05_fence_after_thread_sync();
      const uint32_t accumulator = tmem_base + buffer * padded_rows;
      for (int block = 0; block < item.k_count; ++block) {
        const bool ready = ptx::mbarrier_wait_fast(full_bar + 8U * stage, phase);
        if (__all_sync(0xFFFFFFFFU, ready ? 1 : 0) == 0) {
          healthy = false;
          if (lane == 0)
            atomicExch(args.device_error, 2);
          break;
        }
        ptx::tcgen05_fence_after_thread_sync();
        const uint32_t a_low = weight_low + stage * (weight_tile_bytes >> 4);
        const uint32_t b_low = input_low + stage * (input_tile_bytes >> 4);
        if (ptx::elect_one()) {
          // +32 bytes along K inside the swizzle atom = +2 in the 16-byte address field.
          if constexpr (wide) {
            ptx::tcgen05_mma_f16_split(accumulator, a_low, desc_high, b_low, desc_high, idesc,
                                       block > 0 ? 1U : 0U);
#pragma unroll
            for (int step = 1; step < tile_k_bytes / umma_k; ++step)
              ptx::tcgen05_mma_f16_split(accumulator, a_low + 2 * step, desc_high,
                                         b_low + 2 * step, desc_high, idesc, 1U);
          } else {
            ptx::tcgen05_mma_f8f6f4_split(accumulator, a_low, desc_high, b_low, desc_high, idesc,
                                          block > 0 ? 1U : 0U);
#pragma unroll
            for (int step = 1; step < tile_k_bytes / umma_k; ++step)
              ptx::tcgen05_mma_f8f6f4_split(accumulator, a_low + 2 * step, desc_high,
                                            b_low + 2 * step, desc_high, idesc, 1U);
          }
          ptx::tcgen05_commit(empty_bar + 8U * stage);
        }
        __syncwarp();
        if (++stage == stages) {
          stage = 0;
          phase ^= 1U;
        }
      }
      if (healthy && ptx::elect_one())
        ptx::tcgen05_commit(acc_full_bar + 8U * buffer);
      __syncwarp();
      buffer ^= 1U;
      if (buffer == 0)
        buffer_phase ^= 1U;
    }
  } else {
    const int quarter = warp & 3;  // TMEM lane group this warp may read
    [[maybe_unused]] const int epilogue_thread = (warp - 2) * 32 + lane;
    grid_dependency_wait();
    float scale = 1.0F;
    if constexpr (mode != 1 && !wide)
      scale = args.input_scale[0] * args.weight_scale[0];
    int local = 0;
    [[maybe_unused]] int exchange_parity = 0;
    [[maybe_unused]] float gated_amax = 0.0F;
    for (int index = first_item; index < items; index += item_stride, ++local) {
      const WorkItem item = decode_item(args, index);
      const int buffer = local & 1;
      const uint32_t use = static_cast<uint32_t>(local >> 1);
      const bool ready =
          __all_sync(0xFFFFFFFFU,
                     ptx::mbarrier_wait_bounded(acc_full_bar + 8U * buffer, use & 1U) ? 1 : 0) != 0;
      if (!ready && lane == 0) {
        atomicExch(args.device_error, 3);
        epilogue_gave_up = 1;
      }
      if constexpr (mode == 2 || mode == 3) {
        // The four epilogue warps meet at a named barrier further down, so they must leave the
        // loop together: each one's wait is bounded, all reach this barrier, and all read the
        // same flag after it.
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*reinterpret_cast<volatile int *>(&epilogue_gave_up) != 0)
          break;
      } else {
        if (!ready)
          break;
      }
      ptx::tcgen05_fence_after_thread_sync();
      const int feature = item.tile * tile_features + quarter * 32 + lane;
      const int feature_base = item.tile * tile_features + quarter * 32;
      const uint32_t lane_address =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buffer * padded_rows;
      if constexpr (mode == 3) {
        const int tail_width = args.tail_tiles * tile_features;
        const int tail_tile = item.tile - (args.tiles - args.tail_tiles);
        const int tail_feature = tail_tile * tile_features + quarter * 32 + lane;
        if (item.tail) {    // uniform over the four warps
          // Park this piece's sums; every CTA takes a share of finishing them after the loop.
          float *destination = args.tail_partial +
                               static_cast<size_t>(item.piece) * args.rows * tail_width +
                               tail_feature;
#pragma unroll 1
          for (int chunk = 0; chunk < padded_rows / 32; ++chunk) {
            if (chunk * 32 < args.rows) {
              uint32_t raw[32];
              ptx::tmem_load_32x32b_x32(lane_address + chunk * 32, raw);
              ptx::tmem_load_wait();
#pragma unroll
              for (int column = 0; column < 32; ++column) {
                const int row = chunk * 32 + column;
                if (row < args.rows)
                  destination[static_cast<size_t>(row) * tail_width] = __uint_as_float(raw[column]);
              }
            }
          }
        } else {
#pragma unroll 1
          for (int chunk = 0; chunk < padded_rows / 32; ++chunk) {
            if (chunk * 32 < args.rows) {
              uint32_t raw[32];
              ptx::tmem_load_32x32b_x32(lane_address + chunk * 32, raw);
              ptx::tmem_load_wait();
              float values[32];
#pragma unroll
              for (int column = 0; column < 32; ++column)
                values[column] = __uint_as_float(raw[column]);
              gated_chunk(args, values, chunk, item.tile, quarter, lane, scale,
                          exchange + exchange_parity * (128 * 16), gated_amax);
              exchange_parity ^= 1;
            }
          }
        }
        {
          ptx::tcgen05_fence_before_thread_sync();
          __syncwarp();
          if (lane == 0)
            ptx::mbarrier_arrive(acc_empty_bar + 8U * buffer);
        }
      } else {
#pragma unroll
      for (int chunk = 0; chunk < padded_rows / 32; ++chunk) {
        if (chunk * 32 < args.rows) {  // warp-uniform
          uint32_t raw[32];
          ptx::tmem_load_32x32b_x32(lane_address + chunk * 32, raw);
          ptx::tmem_load_wait();
          if constexpr (mode == 1) {
            if (feature < args.output_width) {
              float *destination = args.partial +
                                   static_cast<size_t>(item.piece) * args.rows * args.output_width +
                                   feature;
#pragma unroll
              for (int column = 0; column < 32; ++column) {
                const int row = chunk * 32 + column;
                if (row < args.rows)
                  destination[static_cast<size_t>(row) * args.output_width] =
                      __uint_as_float(raw[column]);
              }
            }
          } else {
            bool finished = false;
            if constexpr (mode == 0) {
              if (item.tail) {    // warp-uniform
                const int tail_width = args.tail_tiles * tile_features;
                const int tail_feature = feature - (args.tiles - args.tail_tiles) * tile_features;
                float *destination = args.tail_partial +
                                     static_cast<size_t>(item.piece) * args.rows * tail_width +
                                     tail_feature;
#pragma unroll
                for (int column = 0; column < 32; ++column) {
                  const int row = chunk * 32 + column;
                  if (row < args.rows)
                    destination[static_cast<size_t>(row) * tail_width] =
                        __uint_as_float(raw[column]);
                }
                finished = true;
              }
            }
            if (!finished) {
              float values[32];
#pragma unroll
              for (int column = 0; column < 32; ++column)
                values[column] = __uint_as_float(raw[column]);
              finish_chunk<mode>(args, values, chunk, feature, feature_base, lane, scale,
                                 row_best);
            }
          }
        }
      }
      // The accumulator buffer is free again as soon as its values are in registers.
      ptx::tcgen05_fence_before_thread_sync();
      __syncwarp();
      if (lane == 0)
        ptx::mbarrier_arrive(acc_empty_bar + 8U * buffer);
      }

      if constexpr (mode == 2) {
        {
          // Combine the four feature quarters in shared memory, then one global atomic per row.
          asm volatile("bar.sync 1, 128;" ::: "memory");
          for (int row = epilogue_thread; row < args.rows && row < padded_rows; row += 128) {
            const unsigned long long candidate = row_best[row];
            if (candidate != 0ULL)
              atomicMax(args.best + row, candidate);
            row_best[row] = 0ULL;
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      }
    }
    if constexpr (mode == 3) {
      // Grid-wide phases after the item loop. Every CTA of the launch is resident (the grid is
      // at most one CTA per SM) and comes here, so a counter barrier is safe; its wait is bounded
      // like every other wait of the kernel.
      const unsigned int grid = gridDim.x;
      const bool has_tail = args.tail_tiles > 0;
      const bool quantises = args.fp8_output != nullptr;
      const unsigned int barriers = (has_tail ? 1U : 0U) + (quantises ? 1U : 0U);
      unsigned int passed = 0;
      bool alive = *reinterpret_cast<volatile int *>(&epilogue_gave_up) == 0;
      const auto grid_barrier = [&]() -> bool {
        ++passed;
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (epilogue_thread == 0) {
          // (barriers + 1) * grid increments a launch, the last of which wraps the word to zero.
          atomicInc(args.grid_counter, (barriers + 1U) * grid - 1U);
          const long long start = clock64();
          bool arrived = true;
          while (*reinterpret_cast<volatile unsigned int *>(args.grid_counter) < passed * grid) {
            if (clock64() - start > ptx::wait_cycle_limit) {
              arrived = false;
              atomicExch(args.device_error, 6);
              break;
            }
          }
          __threadfence();
          tail_is_last = arrived ? 1 : 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        return *reinterpret_cast<volatile int *>(&tail_is_last) != 0;
      };
      if (has_tail && alive) {
        alive = grid_barrier();
        if (alive) {
          // (tail tile, 32-row chunk) units dealt round the grid: sum the K pieces in piece
          // order and finish like a whole tile.
          const int tail_width = args.tail_tiles * tile_features;
          const int chunks = (args.rows + 31) / 32;
          const int units = args.tail_tiles * chunks;
          for (int unit = static_cast<int>(blockIdx.x); unit < units; unit += static_cast<int>(grid)) {
            const int tail_tile = unit / chunks;
            const int chunk = unit - tail_tile * chunks;
            const int tail_feature = tail_tile * tile_features + quarter * 32 + lane;
            float values[32];
#pragma unroll
            for (int column = 0; column < 32; ++column)
              values[column] = 0.0F;
            // Rows past the end read the last row again (and are dropped at the store), so the
            // 32 loads of a piece are unconditional and all in flight together.
            // Three pieces' loads are issued before the first add (one L2 round trip for all of
            // them); the adds stay in piece order.
            for (int first_piece = 0; first_piece < args.tail_splits; first_piece += 3) {
              float fetched[3][32];
#pragma unroll
              for (int offset = 0; offset < 3; ++offset) {
                if (first_piece + offset < args.tail_splits) {    // uniform
                  const float *source =
                      args.tail_partial +
                      static_cast<size_t>(first_piece + offset) * args.rows * tail_width +
                      tail_feature;
#pragma unroll
                  for (int column = 0; column < 32; ++column) {
                    const int row = min(chunk * 32 + column, args.rows - 1);
                    fetched[offset][column] =
                        __ldcg(source + static_cast<size_t>(row) * tail_width);
                  }
                }
              }
#pragma unroll
              for (int offset = 0; offset < 3; ++offset) {
                if (first_piece + offset < args.tail_splits) {
#pragma unroll
                  for (int column = 0; column < 32; ++column)
                    values[column] += fetched[offset][column];
                }
              }
            }
            gated_chunk(args, values, chunk, args.tiles - args.tail_tiles + tail_tile, quarter,
                        lane, scale, exchange + exchange_parity * (128 * 16), gated_amax);
            exchange_parity ^= 1;
          }
        }
      }
      // One atomic per warp and launch: the largest magnitude this warp wrote.
#pragma unroll
      for (int offset = 16; offset > 0; offset >>= 1)
        gated_amax = fmaxf(gated_amax, __shfl_xor_sync(0xFFFFFFFFU, gated_amax, offset));
      if (lane == 0 && gated_amax > 0.0F)
        atomicMax(args.amax_bits, __float_as_uint(gated_amax));
      if (quantises && alive) {
        alive = grid_barrier();
        if (alive) {
          const float tensor_amax =
              __uint_as_float(*reinterpret_cast<volatile unsigned int *>(args.amax_bits));
          const float quant_scale = tensor_amax > 0.0F ? tensor_amax / 448.0F : 1.0F;
          const float inverse_scale = 1.0F / quant_scale;
          if (blockIdx.x == 0 && epilogue_thread == 0)
            *args.scale_out = quant_scale;
          const size_t groups = static_cast<size_t>(args.rows) * args.gated_width / 8;
          const size_t share = (groups + grid - 1) / grid;
          const size_t first = share * blockIdx.x;
          const size_t last = first + share < groups ? first + share : groups;
          // Eight 16-byte loads in flight per thread: the rows come from L2, and a loop of
          // dependent load-convert-store steps would pay its latency once per step.
          const uint4 *source = reinterpret_cast<const uint4 *>(args.output);
          uint2 *destination = reinterpret_cast<uint2 *>(args.fp8_output);
          for (size_t base = first; base < last; base += 8 * 128) {
            uint4 raw[8];
#pragma unroll
            for (int step = 0; step < 8; ++step) {
              const size_t group = base + step * 128 + epilogue_thread;
              raw[step] = make_uint4(0, 0, 0, 0);
              if (group < last)
                raw[step] = __ldcg(source + group);
            }
#pragma unroll
            for (int step = 0; step < 8; ++step) {
              const size_t group = base + step * 128 + epilogue_thread;
              if (group < last) {
                const __nv_bfloat162 *pairs = reinterpret_cast<const __nv_bfloat162 *>(&raw[step]);
                const float2 a = __bfloat1622float2(pairs[0]);
                const float2 b = __bfloat1622float2(pairs[1]);
                const float2 c = __bfloat1622float2(pairs[2]);
                const float2 d = __bfloat1622float2(pairs[3]);
                __nv_fp8x4_e4m3 low(make_float4(a.x * inverse_scale, a.y * inverse_scale,
                                                b.x * inverse_scale, b.y * inverse_scale));
                __nv_fp8x4_e4m3 high(make_float4(c.x * inverse_scale, c.y * inverse_scale,
                                                 d.x * inverse_scale, d.y * inverse_scale));
                uint2 packed;
                packed.x = low.__x;
                packed.y = high.__x;
                destination[group] = packed;
              }
            }
          }
        }
      }
      if (barriers > 0 && epilogue_thread == 0 && passed == barriers)
        atomicInc(args.grid_counter, (barriers + 1U) * grid - 1U);   // the round that wraps to zero
    }
  }

  ptx::tcgen05_fence_before_thread_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tcgen05_fence_after_thread_sync();
    ptx::tmem_dealloc(tmem_base, tmem_columns);
  }
}

__global__ void finalize_split_k_kernel(const float *partial, const float *input_scale,
                                        const float *weight_scale, __nv_bfloat16 *output,
                                        int splits, size_t elements) {
  grid_dependency_launch();
  grid_dependency_wait();
  const float scale = input_scale != nullptr ? input_scale[0] * weight_scale[0] : 1.0F;
  for (size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
       index < elements; index += static_cast<size_t>(blockDim.x) * gridDim.x) {
    // Four pieces a round trip, added in piece order.
    float sum = 0.0F;
    for (int first = 0; first < splits; first += 4) {
      float piece[4];
#pragma unroll
      for (int offset = 0; offset < 4; ++offset)
        piece[offset] = first + offset < splits
                            ? partial[static_cast<size_t>(first + offset) * elements + index]
                            : 0.0F;
#pragma unroll
      for (int offset = 0; offset < 4; ++offset)
        if (first + offset < splits)
          sum += piece[offset];
    }
    output[index] = __float2bfloat16_rn(sum * scale);
  }
}

// output[row, first_column + c] = bf16(scale * sum over pieces of partial[piece, row, c]).
__global__ void finalize_tail_kernel(const float *partial, const float *input_scale,
                                     const float *weight_scale, __nv_bfloat16 *output, int pieces,
                                     int rows, int tail_width, int output_width, int first_column) {
  grid_dependency_launch();
  grid_dependency_wait();
  const float scale = input_scale != nullptr ? input_scale[0] * weight_scale[0] : 1.0F;
  const size_t elements = static_cast<size_t>(rows) * tail_width;
  for (size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
       index < elements; index += static_cast<size_t>(blockDim.x) * gridDim.x) {
    float sum = 0.0F;
    for (int first = 0; first < pieces; first += 4) {
      float piece[4];
#pragma unroll
      for (int offset = 0; offset < 4; ++offset)
        piece[offset] = first + offset < pieces
                            ? partial[static_cast<size_t>(first + offset) * elements + index]
                            : 0.0F;
#pragma unroll
      for (int offset = 0; offset < 4; ++offset)
        if (first + offset < pieces)
          sum += piece[offset];
    }
    const size_t row = index / tail_width;
    const size_t column = index - row * tail_width;
    output[row * output_width + first_column + column] = __float2bfloat16_rn(sum * scale);
  }
}

__global__ void unpack_best_kernel(const unsigned long long *best, int *tokens, int rows) {
  const int row = static_cast<int>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (row < rows)
    tokens[row] = best_index(best[row]);
}

__global__ void linear_simt_check_kernel(const __nv_fp8_e4m3 *input, const float *input_scale,
                                         const __nv_fp8_e4m3 *weight, const float *weight_scale,
                                         __nv_bfloat16 *output, int rows, int input_width,
                                         int output_width) {
  const int feature = static_cast<int>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int row = static_cast<int>(blockIdx.y);
  if (feature >= output_width || row >= rows)
    return;
  const __nv_fp8_e4m3 *x = input + static_cast<size_t>(row) * input_width;
  const __nv_fp8_e4m3 *w = weight + static_cast<size_t>(feature) * input_width;
  float sum = 0.0F;
  for (int k = 0; k < input_width; ++k)
    sum += static_cast<float>(x[k]) * static_cast<float>(w[k]);
  output[static_cast<size_t>(row) * output_width + feature] =
      __float2bfloat16_rn(sum * (input_scale[0] * weight_scale[0]));
}

// [outer, inner] row-major bytes, box [box_outer, 128] with the 128-byte swizzle; out-of-range
// rows and K tails read as zero.
bool encode_byte_matrix(CUtensorMap *map, const void *base, uint64_t inner, uint64_t outer,
                        uint32_t box_outer) {
  const EncodeTiled encode = encode_tiled_entry();
  if (encode == nullptr)
    return false;
  const cuuint64_t dimensions[2] = {inner, outer};
  const cuuint64_t strides[1] = {inner};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(tile_k_bytes), box_outer};
  const cuuint32_t element_strides[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dimensions,
                strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int padded_rows, int mode, bool wide>
int launch_variant(const LinearPlan &plan, const KernelArguments &arguments, cudaStream_t stream) {
  constexpr int stages = stages_for(padded_rows);
  constexpr int dynamic_bytes = stages * (weight_tile_bytes + padded_rows * tile_k_bytes) + 1024;
  static PerDeviceOnce configured;
  if (configured.run([] {
        return cudaFuncSetAttribute(fp8_linear_kernel<padded_rows, mode, wide>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, dynamic_bytes);
      }) != cudaSuccess) {
    return -10;
  }
  const int items = (plan.tiles - arguments.tail_tiles) * arguments.splits +
                    arguments.tail_tiles * arguments.tail_splits;
  const int ctas = items < plan.ctas ? items : plan.ctas;
  return launch_chained(fp8_linear_kernel<padded_rows, mode, wide>,
                        dim3(static_cast<unsigned>(ctas)),
                        dim3(linear_threads), dynamic_bytes, stream, false, plan.weight_map,
                        plan.input_map, arguments) == cudaSuccess
             ? 0
             : -11;
}

template <int mode, bool wide>
int launch_rows_bucket(const LinearPlan &plan, const KernelArguments &arguments,
                       cudaStream_t stream) {
  switch (plan.padded_rows) {
  case 32:
    return launch_variant<32, mode, wide>(plan, arguments, stream);
  case 64:
    return launch_variant<64, mode, wide>(plan, arguments, stream);
  case 128:
    return launch_variant<128, mode, wide>(plan, arguments, stream);
  case 192:
    return launch_variant<192, mode, wide>(plan, arguments, stream);
  case 256:
    return launch_variant<256, mode, wide>(plan, arguments, stream);
  default:
    return -12;
  }
}

template <int mode>
int launch_mode(const LinearPlan &plan, const KernelArguments &arguments, cudaStream_t stream) {
  return plan.element_bytes == 2 ? launch_rows_bucket<mode, true>(plan, arguments, stream)
                                 : launch_rows_bucket<mode, false>(plan, arguments, stream);
}

// `split` false: one piece per tile whatever the plan says (bf16 store and argmax epilogues).
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

} // namespace

void schedule_linear_shape(LinearPlan *plan, int rows, int input_width, int output_width,
                           int requested_splits, int element_bytes) {
  schedule_linear(plan, rows, input_width, output_width, requested_splits, element_bytes);
}

std::size_t linear_partial_bytes_for(int rows, int input_width, int output_width,
                                     int element_bytes) {
  if (rows <= 0 || rows > 256 || input_width <= 0 || output_width <= 0)
    return 0;
  LinearPlan plan{};
  schedule_linear(&plan, rows, input_width, output_width, 0, element_bytes);
  return linear_partial_bytes(plan);
}

int make_linear_plan(LinearPlan *plan, const void *fp8_input, const void *fp8_weight, int rows,
                     int input_width, int output_width, int requested_splits, const char **error,
                     int element_bytes) {
  const auto fail = [&](const char *message, int code) {
    if (error != nullptr)
      *error = message;
    return code;
  };
  if (plan == nullptr || fp8_input == nullptr || fp8_weight == nullptr || rows <= 0 ||
      input_width <= 0 || output_width <= 0) {
    return fail("invalid FP8 linear shape", -1);
  }
  if (element_bytes != 1 && element_bytes != 2)
    return fail("invalid FP8 linear shape", -1);
  if (rows > 256)
    return fail("FP8 linear supports at most 256 rows", -2);
  if (input_width * element_bytes % 16 != 0)
    return fail("FP8 linear input width must be a multiple of 16", -3);
  if ((reinterpret_cast<uintptr_t>(fp8_input) & 15U) != 0 ||
      (reinterpret_cast<uintptr_t>(fp8_weight) & 15U) != 0) {
    return fail("FP8 linear operands must be 16-byte aligned", -4);
  }
  LinearPlan result{};
  schedule_linear(&result, rows, input_width, output_width, requested_splits, element_bytes);
  const uint64_t row_bytes = static_cast<uint64_t>(input_width) * element_bytes;
  if (!encode_byte_matrix(&result.weight_map, fp8_weight, row_bytes,
                          static_cast<uint64_t>(output_width), tile_features) ||
      !encode_byte_matrix(&result.input_map, fp8_input, row_bytes, static_cast<uint64_t>(rows),
                          static_cast<uint32_t>(result.padded_rows))) {
    return fail("cuTensorMapEncodeTiled failed", -5);
  }
  *plan = result;
  return 0;
}

int make_gated_linear_plan(LinearPlan *plan, const void *fp8_input, const void *fp8_weight,
                           int rows, int input_width, int gated_width, const char **error,
                           int element_bytes) {
  if (gated_width <= 0 || gated_width % (tile_features / 2) != 0) {
    if (error != nullptr)
      *error = "gated linear width must be a multiple of 64";
    return -7;
  }
  LinearPlan result{};
  const int status = make_linear_plan(&result, fp8_input, fp8_weight, rows, input_width,
                                      2 * gated_width, 1, error, element_bytes);
  if (status != 0)
    return status;
  const uint64_t row_bytes = static_cast<uint64_t>(input_width) * element_bytes;
  if (!encode_byte_matrix(&result.weight_map, fp8_weight, row_bytes,
                          static_cast<uint64_t>(2) * gated_width, tile_features / 2)) {
    if (error != nullptr)
      *error = "cuTensorMapEncodeTiled failed";
    return -5;
  }
  result.gated_width = gated_width;
  *plan = result;
  return 0;
}

int launch_linear_gated(const LinearPlan &plan, const float *input_scale,
                        const float *weight_scale, void *bf16_activated, unsigned int *amax_bits,
                        void *fp8_output, float *scale_out, float *tail_partial,
                        unsigned int *grid_counter, int *device_error, cudaStream_t stream) {
  if (plan.gated_width <= 0 || bf16_activated == nullptr || amax_bits == nullptr ||
      grid_counter == nullptr || (fp8_output != nullptr && scale_out == nullptr)) {
    return -13;
  }
  KernelArguments arguments = base_arguments(plan, device_error, false);
  arguments.input_scale = input_scale;
  arguments.weight_scale = weight_scale;
  arguments.output = static_cast<__nv_bfloat16 *>(bf16_activated);
  arguments.amax_bits = amax_bits;
  arguments.grid_counter = grid_counter;
  arguments.fp8_output = static_cast<unsigned char *>(fp8_output);
  arguments.scale_out = scale_out;
  arguments.gated_width = plan.gated_width;
  if (plan.tail_tiles > 0 && tail_partial != nullptr) {
    arguments.tail_partial = tail_partial;
    arguments.tail_tiles = plan.tail_tiles;
    arguments.tail_splits = plan.tail_splits;
    arguments.tail_k_blocks_per_split = plan.tail_k_blocks_per_split;
  }
  return launch_mode<3>(plan, arguments, stream);
}

std::size_t linear_partial_bytes(const LinearPlan &plan) {
  if (plan.splits <= 1)
    return linear_tail_bytes(plan);
  return sizeof(float) * static_cast<std::size_t>(plan.splits) * plan.rows * plan.output_width;
}

int launch_linear_bf16(const LinearPlan &plan, const float *input_scale, const float *weight_scale,
                       void *bf16_output, float *partial, int *device_error, cudaStream_t stream) {
  if (plan.gated_width != 0)
    return -13;   // a gated plan's weight map has 64-row boxes
  if (plan.splits == 1 && plan.tail_tiles > 0 && partial != nullptr) {
    const int status = launch_linear_bf16_tail(plan, input_scale, weight_scale, bf16_output,
                                               partial, device_error, stream);
    if (status != 0)
      return status;
    const int tail_width = plan.tail_tiles * tile_features;
    const size_t elements = static_cast<size_t>(plan.rows) * tail_width;
    const int blocks = static_cast<int>((elements + 255) / 256);
    return launch_chained(finalize_tail_kernel, dim3(blocks < 1184 ? blocks : 1184), dim3(256), 0,
                          stream, false, static_cast<const float *>(partial), input_scale,
                          weight_scale, static_cast<__nv_bfloat16 *>(bf16_output),
                          plan.tail_splits, plan.rows, tail_width, plan.output_width,
                          plan.output_width - tail_width) == cudaSuccess
               ? 0
               : -11;
  }
  if (plan.splits == 1) {
    KernelArguments arguments = base_arguments(plan, device_error, false);
    arguments.input_scale = input_scale;
    arguments.weight_scale = weight_scale;
    arguments.output = static_cast<__nv_bfloat16 *>(bf16_output);
    return launch_mode<0>(plan, arguments, stream);
  }
  const int status = launch_linear_partial(plan, partial, device_error, stream);
  if (status != 0)
    return status;
  const size_t elements = static_cast<size_t>(plan.rows) * plan.output_width;
  const int blocks = static_cast<int>((elements + 255) / 256);
  return launch_chained(finalize_split_k_kernel, dim3(blocks < 1184 ? blocks : 1184), dim3(256), 0,
                        stream, false, static_cast<const float *>(partial), input_scale,
                        weight_scale, static_cast<__nv_bfloat16 *>(bf16_output), plan.splits,
                        elements) == cudaSuccess
             ? 0
             : -11;
}

int launch_linear_bf16_tail(const LinearPlan &plan, const float *input_scale,
                            const float *weight_scale, void *bf16_output, float *tail_partial,
                            int *device_error, cudaStream_t stream) {
  if (plan.splits != 1 || plan.tail_tiles <= 0 || tail_partial == nullptr)
    return -13;
  KernelArguments arguments = base_arguments(plan, device_error, false);
  arguments.input_scale = input_scale;
  arguments.weight_scale = weight_scale;
  arguments.output = static_cast<__nv_bfloat16 *>(bf16_output);
  arguments.tail_partial = tail_partial;
  arguments.tail_tiles = plan.tail_tiles;
  arguments.tail_splits = plan.tail_splits;
  arguments.tail_k_blocks_per_split = plan.tail_k_blocks_per_split;
  return launch_mode<0>(plan, arguments, stream);
}

std::size_t linear_tail_bytes(const LinearPlan &plan) {
  return plan.tail_tiles <= 0 ? 0
                              : sizeof(float) * static_cast<std::size_t>(plan.tail_splits) *
                                    plan.rows * plan.tail_tiles * tile_features;
}

int launch_linear_partial(const LinearPlan &plan, float *partial, int *device_error,
                          cudaStream_t stream) {
  if (partial == nullptr)
    return -13;
  KernelArguments arguments = base_arguments(plan, device_error, true);
  arguments.partial = partial;
  return launch_mode<1>(plan, arguments, stream);
}

int launch_linear_argmax(const LinearPlan &plan, const float *input_scale,
                         const float *weight_scale, unsigned long long *best, int *device_error,
                         cudaStream_t stream) {
  if (best == nullptr)
    return -14;
  KernelArguments arguments = base_arguments(plan, device_error, false);
  arguments.input_scale = input_scale;
  arguments.weight_scale = weight_scale;
  arguments.best = best;
  return launch_mode<2>(plan, arguments, stream);
}

int launch_unpack_best(const unsigned long long *best, int *tokens, int rows,
                       cudaStream_t stream) {
  unpack_best_kernel<<<(rows + 127) / 128, 128, 0, stream>>>(best, tokens, rows);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -11;
}

int launch_linear_simt_check(const void *fp8_input, const float *input_scale,
                             const void *fp8_weight, const float *weight_scale, void *bf16_output,
                             int rows, int input_width, int output_width, cudaStream_t stream) {
  const dim3 grid(static_cast<unsigned>((output_width + 127) / 128), static_cast<unsigned>(rows));
  linear_simt_check_kernel<<<grid, 128, 0, stream>>>(
      static_cast<const __nv_fp8_e4m3 *>(fp8_input), input_scale,
      static_cast<const __nv_fp8_e4m3 *>(fp8_weight), weight_scale,
      static_cast<__nv_bfloat16 *>(bf16_output), rows, input_width, output_width);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -11;
}

} // namespace carat_b200
