// One-kernel attention for head_dim 256 when the whole key range of a (request, kv head) fits one
// CTA: at most 1024 cache rows plus the proposal rows, at most 16 query rows per KV head. That is
// every sliding-window layer of the verify step and of the drafter.
//
// The three phases of the reference (QK GEMM -> softmax -> PV GEMM, bf16 scores, fp32 softmax, bf16
// probabilities, fp32 P.V) run back to back inside the CTA with the reference's rounding points,
// but the scores never leave the SM:
//   1. K streams through a TMA ring; S[key, row] accumulates in TMEM (two buffers); the epilogue
//      warps round S to bf16, replace masked entries by -inf and park the tile in shared memory,
//      already in the swizzled K-major layout the P.V instruction wants for its B operand. Each
//      thread also keeps a running (maximum, sum of exp) pair per row over the keys it has seen.
//   2. The pairs are merged across the CTA and the epilogue warps turn S into P in place:
//      P = bf16(exp(S - max) / sum); exp(-inf) is exactly 0, so masked keys need no second test.
//   3. V streams through the same ring as the MN-major A operand; O[d, row] accumulates in TMEM and
//      is rounded to bf16 once.
// K and V rows are read from HBM exactly once and nothing else touches HBM except the output.
//
// The kernel is persistent: one CTA per SM walks the (request, kv head) items, the TMA warp runs
// ahead across phase and item boundaries (the V tiles of an item are in flight while its softmax
// runs, the next item's K tiles while its output is written), and the ring is deep enough
// (10 x 16 KB) for one SM to keep far more than its share of HBM bandwidth in flight, so SMs that
// still have an item left absorb the bandwidth of those that are done.
// Every wait is bounded; a wait that runs out records a code in the device error word and raises a
// CTA-wide flag that makes every later wait return at once.
#include "attention.cuh"
#include "attention_geometry.cuh"
#include "attention_tc.cuh"
#include "context.cuh"
#include "launch.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>
#include <math_constants.h>

namespace carat_b200 {
namespace {

constexpr int fused_epilogue_warps = 8;
constexpr int fused_epilogue_threads = fused_epilogue_warps * 32;
constexpr int fused_threads = 64 + fused_epilogue_threads;   // warp 0 TMA, warp 1 MMA + TMEM
constexpr int fused_dimension = 256;
constexpr int fused_rows = 16;           // UMMA N: query rows of one KV head, padded
constexpr int fused_tile_keys = 128;     // cache rows per score tile (UMMA M)
constexpr int fused_max_tiles = 8;       // 1024 cache rows
constexpr int fused_stage_bytes = 16 * 1024;
constexpr int fused_stages = 10;
constexpr int fused_value_keys = 32;     // cache rows per V stage: [32 keys x 256 components]
constexpr int fused_query_bytes = 4 * fused_rows * 128;                      // 8 KB, two buffers
constexpr int fused_box_bytes = fused_rows * 128;                            // P box: 16 x 64 keys
constexpr int fused_boxes = 1 + fused_max_tiles * 2;                         // proposals + cache
constexpr int fused_shared_bytes = 2 * fused_query_bytes + fused_boxes * fused_box_bytes +
                                   fused_stages * fused_stage_bytes + 1024;

struct FusedArguments {
  AttentionArguments a;
  int *device_error;
  int items;               // requests * kv_heads
};

// What one (request, kv head) item needs, derived the same way by every role.
struct FusedItem {
  int request;
  int kv_head;
  int position;
  int cache_rows;
  int proposals;
  int cache_tiles;
  int score_items;
  int value_items;
  int query_row0;
  int staged_row0;
  long long cache_row0;
};

__device__ __forceinline__ FusedItem fused_item(const AttentionArguments &a, int index) {
  FusedItem item;
  item.request = index / a.kv_heads;
  item.kv_head = index - item.request * a.kv_heads;
  const KeyGeometry g = key_geometry(a, item.request);
  const int group = a.query_heads / a.kv_heads;
  item.position = a.positions[item.request];
  item.cache_rows = g.cache_rows;
  item.proposals = g.proposals;
  item.cache_tiles = (g.cache_rows + fused_tile_keys - 1) / fused_tile_keys;
  item.score_items = (g.proposals > 0 ? 1 : 0) + item.cache_tiles;
  item.value_items =
      (g.proposals > 0 ? 1 : 0) + (g.cache_rows + fused_value_keys - 1) / fused_value_keys;
  item.query_row0 = (item.request * a.query_heads + item.kv_head * group) * a.depth;
  item.staged_row0 = (item.request * a.kv_heads + item.kv_head) * a.depth;
  item.cache_row0 =
      (static_cast<long long>(a.slots[item.request]) * a.kv_heads + item.kv_head) * a.capacity;
  return item;
}

// Position in the TMA ring; advancing is two instructions instead of a division.
struct RingCursor {
  uint32_t stage{0};
  uint32_t phase{0};
  __device__ __forceinline__ void advance() {
    if (++stage == fused_stages) {
      stage = 0;
      phase ^= 1U;
    }
  }
};

// Byte offset of the 16-byte chunk (row, chunk) inside a [16 rows x 64 keys] bf16 box laid out
// like a TMA tile with the 128-byte swizzle: the chunk index is XORed with the row index modulo 8.
__device__ __forceinline__ uint32_t box_chunk_offset(int row, int chunk) {
  return static_cast<uint32_t>(row * 128 + ((chunk ^ (row & 7)) << 4));
}

__device__ __forceinline__ void epilogue_barrier() {
  asm volatile("bar.sync 1, %0;" ::"n"(fused_epilogue_threads) : "memory");
}

__device__ __forceinline__ float warp_max(float value) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1)
    value = fmaxf(value, __shfl_xor_sync(0xFFFFFFFFU, value, offset));
  return value;
}

__device__ __forceinline__ float warp_sum(float value) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1)
    value += __shfl_xor_sync(0xFFFFFFFFU, value, offset);
  return value;
}

__global__ void __launch_bounds__(fused_threads, 1)
attention_fused_kernel(const __grid_constant__ CUtensorMap key_map,
                       const __grid_constant__ CUtensorMap new_key_map,
                       const __grid_constant__ CUtensorMap value_map,
                       const __grid_constant__ CUtensorMap new_value_map,
                       const __grid_constant__ CUtensorMap query_map, const FusedArguments args) {
  constexpr uint32_t score_idesc = ptx::umma_idesc(1, 1, fused_tile_keys, fused_rows);
  // bf16 x bf16 -> fp32, A (V^T) MN-major: bit 15.
  constexpr uint32_t value_idesc = ptx::umma_idesc(1, 1, 128, fused_rows) | (1U << 15);
  constexpr uint32_t tmem_columns = 64;    // S: 2 x 16, O: 2 x 16
  constexpr uint32_t value_box_bytes = fused_value_keys * 128;   // [32 keys x 64 components]
  const AttentionArguments &a = args.a;

  extern __shared__ unsigned char shared_raw[];
  // full[stages] empty[stages] acc_full[2] acc_empty[2] query_full[2] query_free[2]
  // probability output
  __shared__ __align__(8) unsigned long long barriers[2 * fused_stages + 10];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_word;
  __shared__ float warp_maxima[fused_epilogue_warps][fused_rows / 2];
  __shared__ float warp_sums[fused_epilogue_warps][fused_rows / 2];
  __shared__ float row_maximum[fused_rows];
  __shared__ float row_inverse_sum[fused_rows];
  volatile int *abort_flag = &abort_word;
  const uint32_t base = (ptx::smem_u32(shared_raw) + 1023U) & ~1023U;
  const uint32_t query_tiles = base;
  const uint32_t boxes = base + 2 * fused_query_bytes;
  const uint32_t ring = boxes + fused_boxes * fused_box_bytes;
  unsigned char *const boxes_generic = shared_raw + (boxes - ptx::smem_u32(shared_raw));
  const uint32_t full_bar = ptx::smem_u32(&barriers[0]);
  const uint32_t empty_bar = ptx::smem_u32(&barriers[fused_stages]);
  const uint32_t acc_full_bar = ptx::smem_u32(&barriers[2 * fused_stages]);
  const uint32_t acc_empty_bar = ptx::smem_u32(&barriers[2 * fused_stages + 2]);
  const uint32_t query_full_bar = ptx::smem_u32(&barriers[2 * fused_stages + 4]);
  const uint32_t query_free_bar = ptx::smem_u32(&barriers[2 * fused_stages + 6]);
  const uint32_t probability_bar = ptx::smem_u32(&barriers[2 * fused_stages + 8]);
  const uint32_t output_bar = ptx::smem_u32(&barriers[2 * fused_stages + 9]);

  const int warp = static_cast<int>(threadIdx.x) / 32;
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int group = a.query_heads / a.kv_heads;
  const int rows = group * a.depth;

  grid_dependency_launch();
  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int stage = 0; stage < fused_stages; ++stage) {
      ptx::mbarrier_init(full_bar + 8U * stage, 1);
      ptx::mbarrier_init(empty_bar + 8U * stage, 1);
    }
    for (int buffer = 0; buffer < 2; ++buffer) {
      ptx::mbarrier_init(acc_full_bar + 8U * buffer, 1);
      ptx::mbarrier_init(acc_empty_bar + 8U * buffer, fused_epilogue_warps);
      ptx::mbarrier_init(query_full_bar + 8U * buffer, 1);
      ptx::mbarrier_init(query_free_bar + 8U * buffer, 1);
    }
    ptx::mbarrier_init(probability_bar, fused_epilogue_threads);
    ptx::mbarrier_init(output_bar, 1);
    ptx::fence_mbarrier_init();
    ptx::prefetch_tensormap(&key_map);
    ptx::prefetch_tensormap(&value_map);
    ptx::prefetch_tensormap(&query_map);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&tmem_base_slot), tmem_columns);
    ptx::tmem_relinquish_alloc_permit();
  }
  ptx::tcgen05_fence_before_thread_sync();
  __syncthreads();
  ptx::tcgen05_fence_after_thread_sync();
  const uint32_t tmem_base = tmem_base_slot;
  const uint32_t tmem_output = tmem_base + 2 * fused_rows;
  // The producer thread waits further down, after its early loads; the rest of its warp has
  // nothing to wait for.
  if (warp != 0)
    grid_dependency_wait();

  // The TMA and MMA roles are single threads whose loop bodies are the critical path of the whole
  // kernel (a dependent instruction costs a handful of cycles and there is nothing to hide it), so
  // they keep running cursors and precomputed descriptor words instead of recomputing anything.
  if (warp == 0) {
    if (lane == 0) {
      const uint64_t stream_policy = ptx::policy_evict_first();
      const uint64_t reuse_policy = ptx::policy_evict_last();
      RingCursor cursor;
      bool healthy = true;
      int local = 0;
      // Cache rows that no grid of this chain writes can be on their way while the previous grid
      // still runs: the first item's key tiles, into the stages they will be consumed from (the
      // proposal keys, which the previous grid produces, keep the four stages before them).
      int early_stages = 0;
      if (a.inputs_static != 0 && a.cache_static != 0 &&
          static_cast<int>(blockIdx.x) < args.items) {
        const FusedItem item = fused_item(a, static_cast<int>(blockIdx.x));
        const int reserved = item.proposals > 0 ? 4 : 0;
        RingCursor ahead;
        for (int skip = 0; skip < reserved; ++skip)
          ahead.advance();
        early_stages = min(fused_stages - reserved, item.cache_tiles * 4);
        const int cache_row0 = static_cast<int>(item.cache_row0);
        for (int early = 0; early < early_stages; ++early) {
          ptx::mbarrier_arrive_expect_tx(full_bar + 8U * ahead.stage, fused_stage_bytes);
          ptx::tma_load_2d(ring + ahead.stage * fused_stage_bytes, &key_map, (early & 3) * 64,
                           cache_row0 + (early >> 2) * fused_tile_keys,
                           full_bar + 8U * ahead.stage, stream_policy);
          ahead.advance();
        }
      }
      grid_dependency_wait();
      for (int index = static_cast<int>(blockIdx.x); index < args.items && healthy;
           index += static_cast<int>(gridDim.x), ++local) {
        const FusedItem item = fused_item(a, index);
        const int proposal_items = item.proposals > 0 ? 1 : 0;
        const int buffer = local & 1;
        const uint32_t use = static_cast<uint32_t>(local >> 1);
        if (!ptx::mbarrier_wait_checked(query_free_bar + 8U * buffer, (use & 1U) ^ 1U, abort_flag,
                          args.device_error, 30)) {
          healthy = false;
          break;
        }
        ptx::mbarrier_arrive_expect_tx(query_full_bar + 8U * buffer, fused_query_bytes);
#pragma unroll
        for (int sub = 0; sub < 4; ++sub)
          ptx::tma_load_2d(query_tiles + buffer * fused_query_bytes + sub * fused_rows * 128,
                           &query_map, sub * 64, item.query_row0, query_full_bar + 8U * buffer,
                           reuse_policy);
        const int cache_row0 = static_cast<int>(item.cache_row0);
        // K: one stage per 64-component column block of a 128-key tile.
        if (proposal_items != 0) {
#pragma unroll
          for (int sub = 0; sub < 4; ++sub) {
            if (!ptx::mbarrier_wait_checked(empty_bar + 8U * cursor.stage, cursor.phase ^ 1U, abort_flag,
                              args.device_error, 31)) {
              healthy = false;
              break;
            }
            ptx::mbarrier_arrive_expect_tx(full_bar + 8U * cursor.stage, proposal_columns * 128);
            ptx::tma_load_2d(ring + cursor.stage * fused_stage_bytes, &new_key_map, sub * 64,
                             item.staged_row0, full_bar + 8U * cursor.stage, reuse_policy);
            cursor.advance();
          }
        }
        for (int tile = 0; tile < item.cache_tiles && healthy; ++tile) {
          const int row = cache_row0 + tile * fused_tile_keys;
#pragma unroll
          for (int sub = 0; sub < 4; ++sub) {
            if (early_stages > 0) {   // requested before the wait (first item only)
              --early_stages;
              cursor.advance();
              continue;
            }
            if (!ptx::mbarrier_wait_checked(empty_bar + 8U * cursor.stage, cursor.phase ^ 1U, abort_flag,
                              args.device_error, 31)) {
              healthy = false;
              break;
            }
            ptx::mbarrier_arrive_expect_tx(full_bar + 8U * cursor.stage, fused_stage_bytes);
            ptx::tma_load_2d(ring + cursor.stage * fused_stage_bytes, &key_map, sub * 64, row,
                             full_bar + 8U * cursor.stage, stream_policy);
            cursor.advance();
          }
        }
        // V: one stage per 32 keys, four [32 keys x 64 components] boxes.
        if (proposal_items != 0 && healthy) {
          if (!ptx::mbarrier_wait_checked(empty_bar + 8U * cursor.stage, cursor.phase ^ 1U, abort_flag,
                            args.device_error, 32)) {
            healthy = false;
            break;
          }
          const uint32_t destination = ring + cursor.stage * fused_stage_bytes;
          ptx::mbarrier_arrive_expect_tx(full_bar + 8U * cursor.stage,
                                         4 * proposal_columns * 128);
#pragma unroll
          for (int box = 0; box < 4; ++box)
            ptx::tma_load_2d(destination + box * value_box_bytes, &new_value_map, box * 64,
                             item.staged_row0, full_bar + 8U * cursor.stage, reuse_policy);
          cursor.advance();
        }
        const int value_groups = item.value_items - proposal_items;
        for (int key_group = 0; key_group < value_groups && healthy; ++key_group) {
          if (!ptx::mbarrier_wait_checked(empty_bar + 8U * cursor.stage, cursor.phase ^ 1U, abort_flag,
                            args.device_error, 32)) {
            healthy = false;
            break;
          }
          const uint32_t destination = ring + cursor.stage * fused_stage_bytes;
          const int row = cache_row0 + key_group * fused_value_keys;
          ptx::mbarrier_arrive_expect_tx(full_bar + 8U * cursor.stage, fused_stage_bytes);
#pragma unroll
          for (int box = 0; box < 4; ++box)
            ptx::tma_load_2d(destination + box * value_box_bytes, &value_map, box * 64, row,
                             full_bar + 8U * cursor.stage, stream_policy);
          cursor.advance();
        }
      }
      if (!healthy) {
        // Let the copies in flight land before the CTA exits: every stage's current phase.
        for (int stage = 0; stage < fused_stages; ++stage) {
          const uint32_t parity = static_cast<uint32_t>(stage) < cursor.stage ? cursor.phase
                                                                               : cursor.phase ^ 1U;
          ptx::mbarrier_wait_bounded(full_bar + 8U * stage, parity);
        }
      }
    }
  } else if (warp == 1) {
    {
      // The whole warp walks this role in lockstep and one elected lane issues, so the loop state
      // stays warp-uniform.
      // Descriptor words. High words carry SBO (1024 bytes), version and swizzle mode and are the
      // same for both layouts; the low words hold the start address (16-byte units) and, for the
      // MN-major V tiles, the byte distance between 64-component boxes.
      const uint64_t key_desc = ptx::umma_desc_k_major_sw128(ring);
      const uint64_t value_desc = ptx::umma_desc_mn_major_sw128(ring, value_box_bytes);
      const uint32_t desc_high = static_cast<uint32_t>(key_desc >> 32);
      const uint32_t key_low = static_cast<uint32_t>(key_desc);
      const uint32_t value_low = static_cast<uint32_t>(value_desc);
      const uint32_t query_low = static_cast<uint32_t>(ptx::umma_desc_k_major_sw128(query_tiles));
      const uint32_t box_low = static_cast<uint32_t>(ptx::umma_desc_k_major_sw128(boxes));
      constexpr uint32_t stage_step = fused_stage_bytes >> 4;
      RingCursor cursor;
      uint32_t accumulator = 0;          // score accumulator buffer of the next tile
      uint32_t accumulator_phase = 0;    // flips every second tile
      bool healthy = true;
      int local = 0;
      for (int index = static_cast<int>(blockIdx.x); index < args.items && healthy;
           index += static_cast<int>(gridDim.x), ++local) {
        const FusedItem item = fused_item(a, index);
        const int proposal_items = item.proposals > 0 ? 1 : 0;
        const int query_buffer = local & 1;
        const uint32_t item_parity = static_cast<uint32_t>(local) & 1U;
        const uint32_t item_query_low = query_low + query_buffer * (fused_query_bytes >> 4);
        if (__all_sync(0xFFFFFFFFU, ptx::mbarrier_wait_checked(query_full_bar + 8U * query_buffer,
                          static_cast<uint32_t>(local >> 1) & 1U, abort_flag, args.device_error,
                          33) ? 1 : 0) == 0) {
          healthy = false;
          break;
        }
        for (int tile_item = 0; tile_item < item.score_items && healthy; ++tile_item) {
          if (__all_sync(0xFFFFFFFFU, ptx::mbarrier_wait_checked(acc_empty_bar + 8U * accumulator, accumulator_phase ^ 1U, abort_flag,
                            args.device_error, 34) ? 1 : 0) == 0) {
            healthy = false;
            break;
          }
          ptx::tcgen05_fence_after_thread_sync();
          const uint32_t tmem_scores = tmem_base + accumulator * fused_rows;
#pragma unroll
          for (int sub = 0; sub < 4; ++sub) {
            if (__all_sync(0xFFFFFFFFU, ptx::mbarrier_wait_checked(full_bar + 8U * cursor.stage, cursor.phase, abort_flag,
                              args.device_error, 35) ? 1 : 0) == 0) {
              healthy = false;
              break;
            }
            ptx::tcgen05_fence_after_thread_sync();
            const uint32_t a_low = key_low + cursor.stage * stage_step;
            const uint32_t b_low = item_query_low + sub * ((fused_rows * 128) >> 4);
            if (ptx::elect_one()) {
#pragma unroll
              for (int step = 0; step < 4; ++step)
                ptx::tcgen05_mma_f16_split(tmem_scores, a_low + 2 * step, desc_high,
                                           b_low + 2 * step, desc_high, score_idesc,
                                           (sub > 0 || step > 0) ? 1U : 0U);
              ptx::tcgen05_commit(empty_bar + 8U * cursor.stage);
            }
            __syncwarp();
            cursor.advance();
          }
          if (healthy && ptx::elect_one())
            ptx::tcgen05_commit(acc_full_bar + 8U * accumulator);
          __syncwarp();
          accumulator ^= 1U;
          if (accumulator == 0)
            accumulator_phase ^= 1U;
        }
        if (!healthy)
          break;
        // The query tiles may be overwritten once every score instruction has completed.
        if (ptx::elect_one())
          ptx::tcgen05_commit(query_free_bar + 8U * query_buffer);
        __syncwarp();
        if (__all_sync(0xFFFFFFFFU, ptx::mbarrier_wait_checked(probability_bar, item_parity, abort_flag, args.device_error, 36) ? 1 : 0) == 0) {
          healthy = false;
          break;
        }
        ptx::tcgen05_fence_after_thread_sync();
        uint32_t accumulate = 0;
        if (proposal_items != 0) {
          if (__all_sync(0xFFFFFFFFU, ptx::mbarrier_wait_checked(full_bar + 8U * cursor.stage, cursor.phase, abort_flag,
                            args.device_error, 37) ? 1 : 0) == 0) {
            healthy = false;
            break;
          }
          ptx::tcgen05_fence_after_thread_sync();
          const uint32_t a_low = value_low + cursor.stage * stage_step;
          if (ptx::elect_one()) {
#pragma unroll
            for (int slice = 0; slice < 2; ++slice)
              ptx::tcgen05_mma_f16_split(tmem_output + slice * fused_rows,
                                         a_low + slice * ((2 * value_box_bytes) >> 4), desc_high,
                                         box_low, desc_high, value_idesc, 0U);
            ptx::tcgen05_commit(empty_bar + 8U * cursor.stage);
          }
          __syncwarp();
          accumulate = 1;
          cursor.advance();
        }
        const int value_groups = item.value_items - proposal_items;
        for (int key_group = 0; key_group < value_groups; ++key_group) {
          if (__all_sync(0xFFFFFFFFU, ptx::mbarrier_wait_checked(full_bar + 8U * cursor.stage, cursor.phase, abort_flag,
                            args.device_error, 37) ? 1 : 0) == 0) {
            healthy = false;
            break;
          }
          ptx::tcgen05_fence_after_thread_sync();
          const uint32_t a_low = value_low + cursor.stage * stage_step;
          // Probability box (64 keys) and the 32-byte step inside its 128-byte rows.
          const uint32_t b_low = box_low + (1 + (key_group >> 1)) * (fused_box_bytes >> 4) +
                                 (key_group & 1) * 4;
          if (ptx::elect_one()) {
#pragma unroll
          for (int step = 0; step < 2; ++step) {
#pragma unroll
            for (int slice = 0; slice < 2; ++slice) {
              // 16 keys per instruction = two 8-row swizzle atoms of a V box (2048 bytes); the
              // two 64-component halves of a 128-component slice are consecutive boxes.
              ptx::tcgen05_mma_f16_split(
                  tmem_output + slice * fused_rows,
                  a_low + slice * ((2 * value_box_bytes) >> 4) + step * (2048 >> 4), desc_high,
                  b_low + 2 * step, desc_high, value_idesc, step > 0 ? 1U : accumulate);
            }
          }
          ptx::tcgen05_commit(empty_bar + 8U * cursor.stage);
          }
          __syncwarp();
          accumulate = 1;
          cursor.advance();
        }
        if (healthy && ptx::elect_one())
          ptx::tcgen05_commit(output_bar);
        __syncwarp();
      }
    }
  } else {
    const int epilogue_warp = warp - 2;
    const int quarter = warp & 3;                 // TMEM lane quarter this warp may read
    const int half = epilogue_warp >> 2;          // rows with (row & 1) == half belong to this warp
    const int thread = quarter * 32 + lane;       // key inside a tile, component inside a slice
    const int epilogue_thread = epilogue_warp * 32 + lane;
    const int mode = a.draft ? 0 : a.window > 0 ? 2 : 0;
    const int width = a.query_heads * fused_dimension;
    auto *output = static_cast<__nv_bfloat16 *>(a.output);
    // Row slot s of this warp is query row 2 * s + half; its token decides what it may see.
    int slot_token[fused_rows / 2];
#pragma unroll
    for (int slot = 0; slot < fused_rows / 2; ++slot)
      slot_token[slot] = (slot * 2 + half) % a.depth;
    constexpr float masked_score = -1.0e30F;   // stands in for -inf in the running statistics
    int tiles_done = 0;
    int local = 0;
    for (int index = static_cast<int>(blockIdx.x); index < args.items;
         index += static_cast<int>(gridDim.x), ++local) {
      const FusedItem item = fused_item(a, index);
      const int proposal_items = item.proposals > 0 ? 1 : 0;
      const uint32_t item_parity = static_cast<uint32_t>(local) & 1U;
      const int newest_row = item.position > 0 ? (item.position - 1) % a.capacity : 0;

      // ---- phase 1: S tiles -> bf16 (masked: -inf) -> shared memory; running (max, sum) pairs.
      // The running sums use the fast exponential: they only feed the normaliser, whose rounding
      // already depends on the summation order; the probabilities themselves use expf below.
      float maxima[fused_rows / 2];
      float sums[fused_rows / 2];
#pragma unroll
      for (int slot = 0; slot < fused_rows / 2; ++slot) {
        maxima[slot] = masked_score;
        sums[slot] = 0.0F;
      }
      for (int tile_item = 0; tile_item < item.score_items; ++tile_item, ++tiles_done) {
        const int buffer = tiles_done & 1;
        const uint32_t use = static_cast<uint32_t>(tiles_done >> 1);
        const bool ready =
            __all_sync(0xFFFFFFFFU, ptx::mbarrier_wait_checked(acc_full_bar + 8U * buffer, use & 1U, abort_flag,
                                                 args.device_error, 38)
                                        ? 1
                                        : 0) != 0;
        if (!ready)
          continue;
        ptx::tcgen05_fence_after_thread_sync();
        uint32_t values[16];
        ptx::tmem_load_32x32b_x16(
            tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buffer * fused_rows, values);
        const bool proposal = tile_item < proposal_items;
        const int tile = tile_item - proposal_items;
        // Query token t sees this key iff first_token <= t <= last_token.
        int first_token = 1 << 30;
        int last_token = -1;
        unsigned char *cell = nullptr;     // this key's element of row 0 of its box
        int chunk = 0;
        if (proposal) {
          if (thread < proposal_columns) {
            cell = boxes_generic + ((thread & 7) << 1);
            chunk = thread >> 3;
            if (thread < item.proposals) {
              first_token = thread;
              last_token = 1 << 30;
            }
          }
        } else {
          const int cache_row = tile * fused_tile_keys + thread;
          cell = boxes_generic + (1 + tile * 2 + (thread >> 6)) * fused_box_bytes +
                 ((thread & 7) << 1);
          chunk = (thread & 63) >> 3;
          if (cache_row < item.cache_rows) {
            first_token = 0;
            if (mode == 0) {
              last_token = 1 << 30;
            } else {
              int distance = newest_row - cache_row;
              if (distance < 0)
                distance += a.capacity;
              last_token = a.window - 2 - distance;
            }
          }
        }
        ptx::tmem_load_wait();
        ptx::tcgen05_fence_before_thread_sync();
        __syncwarp();
        if (lane == 0)
          ptx::mbarrier_arrive(acc_empty_bar + 8U * buffer);
        if (cell != nullptr) {
#pragma unroll
          for (int slot = 0; slot < fused_rows / 2; ++slot) {
            if (slot * 2 + half < rows) {
              const int row = slot * 2 + half;
              const float raw = __uint_as_float(half != 0 ? values[slot * 2 + 1] : values[slot * 2]);
              const bool visible = slot_token[slot] >= first_token && slot_token[slot] <= last_token;
              const __nv_bfloat16 rounded =
                  __float2bfloat16_rn(visible ? raw : -CUDART_INF_F);
              *reinterpret_cast<__nv_bfloat16 *>(cell + row * 128 + ((chunk ^ (row & 7)) << 4)) =
                  rounded;
              const float score = visible ? __bfloat162float(rounded) : masked_score;
              // Running (maximum, sum of exp) with one exponential per score: whichever of the
              // two terms of sum * exp(max - new_max) + exp(score - new_max) has a zero exponent
              // is exactly 1, the other is exp(-|score - max|).
              const float difference = score - maxima[slot];
              const float decay = __expf(-fabsf(difference));
              sums[slot] = difference > 0.0F ? fmaf(sums[slot], decay, 1.0F)
                                             : sums[slot] + (visible ? decay : 0.0F);
              maxima[slot] = fmaxf(maxima[slot], score);
            }
          }
        }
      }

      // ---- phase 2: merge the pairs, then P = bf16(exp(S - max) / sum) in place
      {
        float warp_maximum[fused_rows / 2];
#pragma unroll
        for (int slot = 0; slot < fused_rows / 2; ++slot)
          warp_maximum[slot] = warp_max(maxima[slot]);
#pragma unroll
        for (int slot = 0; slot < fused_rows / 2; ++slot)
          sums[slot] = warp_sum(sums[slot] * __expf(maxima[slot] - warp_maximum[slot]));
        if (lane == 0) {
#pragma unroll
          for (int slot = 0; slot < fused_rows / 2; ++slot) {
            warp_maxima[epilogue_warp][slot] = warp_maximum[slot];
            warp_sums[epilogue_warp][slot] = sums[slot];
          }
        }
      }
      epilogue_barrier();
      if (epilogue_thread < rows) {
        const int row = epilogue_thread;
        const int slot = row >> 1;
        const int first_warp = (row & 1) * 4;
        float maximum = masked_score;
#pragma unroll
        for (int other = 0; other < 4; ++other)
          maximum = fmaxf(maximum, warp_maxima[first_warp + other][slot]);
        float total = 0.0F;
#pragma unroll
        for (int other = 0; other < 4; ++other)
          total += warp_sums[first_warp + other][slot] *
                   __expf(warp_maxima[first_warp + other][slot] - maximum);
        row_maximum[row] = maximum;
        row_inverse_sum[row] = 1.0F / total;
      }
      epilogue_barrier();
      {
        // 16-byte chunks of eight keys: first the proposal box (two chunks per row), then the
        // cache boxes (eight chunks per row).
        const int proposal_chunks = proposal_items * rows * 2;
        const int per_box = rows * 8;
        const int chunks = proposal_chunks + item.cache_tiles * 2 * per_box;
        for (int chunk_index = epilogue_thread; chunk_index < chunks;
             chunk_index += fused_epilogue_threads) {
          int box_index;
          int row;
          int chunk;
          if (chunk_index < proposal_chunks) {
            box_index = 0;
            row = chunk_index >> 1;
            chunk = chunk_index & 1;
          } else {
            const int cache_index = chunk_index - proposal_chunks;
            const int cache_box = cache_index / per_box;
            const int remainder = cache_index - cache_box * per_box;
            box_index = 1 + cache_box;
            row = remainder >> 3;
            chunk = remainder & 7;
          }
          auto *cell = reinterpret_cast<uint4 *>(boxes_generic + box_index * fused_box_bytes +
                                                 box_chunk_offset(row, chunk));
          const float maximum = row_maximum[row];
          const float inverse_sum = row_inverse_sum[row];
          uint4 raw = *cell;
          auto *pairs = reinterpret_cast<__nv_bfloat162 *>(&raw);
#pragma unroll
          for (int pair = 0; pair < 4; ++pair) {
            const float2 both = __bfloat1622float2(pairs[pair]);
            pairs[pair] = __halves2bfloat162(
                __float2bfloat16_rn(expf(both.x - maximum) * inverse_sum),
                __float2bfloat16_rn(expf(both.y - maximum) * inverse_sum));
          }
          *cell = raw;
        }
      }
      // Make the generic-proxy writes visible to the tensor core before signalling.
      ptx::fence_proxy_async();
      ptx::mbarrier_arrive(probability_bar);

      // ---- phase 3: O -> bf16 output
      const bool finished =
          __all_sync(0xFFFFFFFFU, ptx::mbarrier_wait_checked(output_bar, item_parity, abort_flag,
                                               args.device_error, 39)
                                      ? 1
                                      : 0) != 0;
      if (finished) {
        ptx::tcgen05_fence_after_thread_sync();
        // Warps of half 0 write slice 0 (components 0..127), warps of half 1 slice 1.
        uint32_t values[16];
        ptx::tmem_load_32x32b_x16(
            tmem_output + (static_cast<uint32_t>(quarter * 32) << 16) + half * fused_rows, values);
        ptx::tmem_load_wait();
        const int component = half * 128 + thread;
        int token = 0;
        int local_head = 0;
        float largest = 0.0F;
#pragma unroll
        for (int row = 0; row < fused_rows; ++row) {
          if (row < rows) {
            const size_t out_row = static_cast<size_t>(item.request) * a.depth + token;
            const size_t column =
                static_cast<size_t>(item.kv_head * group + local_head) * fused_dimension + component;
            const __nv_bfloat16 rounded = __float2bfloat16_rn(__uint_as_float(values[row]));
            output[out_row * width + column] = rounded;
            largest = fmaxf(largest, fabsf(__bfloat162float(rounded)));
            if (++token == a.depth) {
              token = 0;
              ++local_head;
            }
          }
        }
        if (a.amax_bits != nullptr) {
          // Non-negative floats order like their bit patterns.
          const unsigned int bits = __reduce_max_sync(0xFFFFFFFFU, __float_as_uint(largest));
          if (lane == 0)
            atomicMax(a.amax_bits, bits);
        }
        ptx::tcgen05_fence_before_thread_sync();
      }
    }
  }

  ptx::tcgen05_fence_before_thread_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tcgen05_fence_after_thread_sync();
    ptx::tmem_dealloc(tmem_base, tmem_columns);
  }
}
} // namespace

bool attention_fused_applies(const AttentionArguments &a) {
  return a.maps != nullptr && a.maps->has_fused && a.head_dim == fused_dimension &&
         a.kv_heads > 0 && a.query_heads / a.kv_heads * a.depth <= fused_rows &&
         a.max_cache_rows <= fused_max_tiles * fused_tile_keys && a.chunks == 1 &&
         a.capacity % fused_tile_keys == 0 && a.output != nullptr &&
         (a.new_keys != nullptr || a.draft != 0);
}

int launch_attention_fused(const AttentionArguments &a, int *device_error, cudaStream_t stream) {
  static PerDeviceOnce configured;
  if (configured.run([] {
        return cudaFuncSetAttribute(attention_fused_kernel,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    fused_shared_bytes);
      }) != cudaSuccess) {
    return -10;
  }
  const AttentionMaps &maps = *a.maps;
  const int multiprocessors = device_multiprocessors();
  const int items = a.requests * a.kv_heads;
  const FusedArguments arguments{a, device_error, items};
  const bool staged = a.new_keys != nullptr;
  const dim3 grid(static_cast<unsigned>(items < multiprocessors ? items : multiprocessors));
  const cudaError_t status = launch_chained(
      attention_fused_kernel, grid, dim3(fused_threads), fused_shared_bytes, stream, false,
      maps.keys, staged ? maps.new_keys : maps.keys, maps.values32,
      staged ? maps.new_values : maps.values32, maps.queries, arguments);
  return status == cudaSuccess ? 0 : -11;
}

} // namespace carat_b200
