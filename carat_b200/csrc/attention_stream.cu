// Two-kernel tensor-core attention for key ranges that do not fit one CTA (global layers: head_dim
// 512, contexts of thousands of rows) and for query-row counts above 16.
//
// Reference semantics (cuda/prefill_gemm_attention.cu:165-349,552-730): bf16 scores, fp32 max / exp
// / sum over the visible keys, bf16 probabilities, fp32 P.V rounded to bf16 once. The work is cut
// into items (request, kv head, chunk of `chunk_keys` cache rows); both kernels are persistent, one
// CTA per SM walking the items, with a deep TMA ring and single-thread issue loops that keep
// running cursors and precomputed descriptor words.
//   scores_stream_kernel : K streams through the ring, S[key, row] accumulates in TMEM; the
//     epilogue warps write bf16 scores (masked entries as -inf) to the score buffer and one
//     (maximum, sum of exp) pair per query row and chunk to the statistics buffer.
//   values_stream_kernel : V streams through the ring as the MN-major A operand. Builder warps
//     merge the chunk statistics of each row, read the bf16 scores back (L2), and write
//     P = bf16(exp(S - max) / sum) straight into shared memory in the swizzled K-major layout of
//     the B operand, one 64-key box at a time, a few boxes ahead of the MMA thread. No separate
//     softmax pass and no probability round trip through global memory.
// K and V rows are read from HBM exactly once. Every wait is bounded; a wait that runs out records
// a code in the device error word and raises a CTA-wide flag that ends every later wait at once.
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

constexpr int stream_tile_keys = 128;          // cache rows per score tile (UMMA M)
constexpr int stream_subtile_bytes = 16 * 1024; // one [128 keys x 64 components] K sub-tile
constexpr int stream_stage_bytes = 2 * stream_subtile_bytes;   // two sub-tiles per ring stage
constexpr int stream_value_keys = 32;          // cache rows per V stage
constexpr float masked_score = -1.0e30F;       // stands in for -inf in the running statistics

struct StreamArguments {
  AttentionArguments a;
  int *device_error;
  int items;               // chunks * requests * kv_heads, chunk-major
};

struct StreamItem {
  int request;
  int kv_head;
  int chunk;
  int position;
  int cache_rows;          // rows of the request's cache that take part at all
  int proposals;           // staged proposal rows (chunk 0 only)
  int first_row;           // first cache row of this chunk
  int rows_here;           // cache rows of this chunk
  int query_row0;
  int staged_row0;
  int cache_row0;          // row of the (slot, head) block in the cache matrix
  __device__ __forceinline__ bool empty() const { return rows_here <= 0 && proposals <= 0; }
};

__device__ __forceinline__ StreamItem stream_item(const AttentionArguments &a, int request,
                                                  int kv_head, int chunk) {
  StreamItem item;
  item.chunk = chunk;
  item.request = request;
  item.kv_head = kv_head;
  const KeyGeometry g = key_geometry(a, item.request);
  const int group = a.query_heads / a.kv_heads;
  item.position = a.positions[item.request];
  item.cache_rows = g.cache_rows;
  item.proposals = item.chunk == 0 ? g.proposals : 0;
  item.first_row = item.chunk * a.chunk_keys;
  const int remaining = g.cache_rows - item.first_row;
  item.rows_here = remaining < 0 ? 0 : remaining < a.chunk_keys ? remaining : a.chunk_keys;
  item.query_row0 = (item.request * a.query_heads + item.kv_head * group) * a.depth;
  item.staged_row0 = (item.request * a.kv_heads + item.kv_head) * a.depth;
  item.cache_row0 = static_cast<int>(
      (static_cast<long long>(a.slots[item.request]) * a.kv_heads + item.kv_head) * a.capacity);
  return item;
}

// Which items a CTA walks. Contexts are ragged, so dealing (chunk, request, head) triples out by
// index leaves some CTAs with three full chunks and others with one short one, and the kernel
// takes as long as its busiest CTA. Instead the items that exist are put in descending order of
// their cache rows (all full chunks first, then every request's last, partial chunk, longest
// first) and dealt out boustrophedon: the first G items to CTAs 0..G-1, the next G to G-1..0, and
// so on, so the CTA that got the larger item of one pass gets the smaller of the next. Every CTA computes
// the same order from the positions; every role of a CTA then walks the CTA's own short list.
constexpr int cached_items = 32;
constexpr int schedule_requests = 64;

struct StreamSchedule {
  int count;                              // items of this CTA
  int full_chunks[schedule_requests];     // whole chunks of each request
  int full_before[schedule_requests];     // whole chunks of the requests before it
  int by_rank[schedule_requests];         // requests that have a last partial chunk, longest first
  int partial_rows[schedule_requests];    // rows of that chunk, -1 = the request has none
  int total_full;
  int total_partial;
  StreamItem items[cached_items];
};

// Position `ordinal` of this CTA's list in the global order, or -1 past the end.
__device__ __forceinline__ int dealt_index(int ordinal, int total) {
  const int grid = static_cast<int>(gridDim.x);
  const int block = static_cast<int>(blockIdx.x);
  const int index = ordinal * grid + ((ordinal & 1) != 0 ? grid - 1 - block : block);
  return index < total ? index : -1;
}

__device__ __forceinline__ StreamItem scheduled_item(const AttentionArguments &a,
                                                     const StreamSchedule &schedule, int index) {
  const int whole = schedule.total_full * a.kv_heads;
  if (index < whole) {
    const int chunk_index = index / a.kv_heads;
    int request = 0;
    while (request + 1 < a.requests && schedule.full_before[request + 1] <= chunk_index)
      ++request;
    return stream_item(a, request, index - chunk_index * a.kv_heads,
                       chunk_index - schedule.full_before[request]);
  }
  const int rank = (index - whole) / a.kv_heads;
  const int request = schedule.by_rank[rank];
  return stream_item(a, request, index - whole - rank * a.kv_heads, schedule.full_chunks[request]);
}

// Called by the whole CTA, followed by __syncthreads().
__device__ __forceinline__ void build_schedule(const AttentionArguments &a,
                                               StreamSchedule &schedule) {
  const int thread = static_cast<int>(threadIdx.x);
  if (thread < a.requests) {
    const KeyGeometry g = key_geometry(a, thread);
    const int whole = g.cache_rows / a.chunk_keys;
    const int rest = g.cache_rows - whole * a.chunk_keys;
    schedule.full_chunks[thread] = whole;
    // Proposals ride with chunk 0, which therefore exists even when the cache is still empty.
    schedule.partial_rows[thread] = rest > 0 || (whole == 0 && g.proposals > 0) ? rest : -1;
  }
  __syncthreads();
  if (thread < a.requests) {
    int before = 0;
    int rank = 0;
    const int mine = schedule.partial_rows[thread];
    for (int other = 0; other < a.requests; ++other) {
      if (other < thread)
        before += schedule.full_chunks[other];
      const int theirs = schedule.partial_rows[other];
      if (theirs >= 0 && (theirs > mine || (theirs == mine && other < thread)))
        ++rank;
    }
    schedule.full_before[thread] = before;
    if (mine >= 0)
      schedule.by_rank[rank] = thread;
    if (thread == a.requests - 1)
      schedule.total_full = before + schedule.full_chunks[thread];
  }
  if (thread == 0) {
    int partial = 0;
    for (int request = 0; request < a.requests; ++request)
      partial += schedule.partial_rows[request] >= 0 ? 1 : 0;
    schedule.total_partial = partial;
  }
  __syncthreads();
  const int total = (schedule.total_full + schedule.total_partial) * a.kv_heads;
  if (thread < cached_items) {
    const int index = dealt_index(thread, total);
    if (index >= 0)
      schedule.items[thread] = scheduled_item(a, schedule, index);
  }
  if (thread == 0) {
    int count = 0;
    while (dealt_index(count, total) >= 0)
      ++count;
    schedule.count = count;
  }
}

__device__ __forceinline__ StreamItem cached_item(const AttentionArguments &a,
                                                  const StreamSchedule &schedule, int ordinal) {
  if (ordinal < cached_items)
    return schedule.items[ordinal];
  const int total = (schedule.total_full + schedule.total_partial) * a.kv_heads;
  return scheduled_item(a, schedule, dealt_index(ordinal, total));
}

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

__host__ __device__ constexpr uint32_t tmem_columns_for(int columns) {
  return columns <= 32 ? 32U : columns <= 64 ? 64U : columns <= 128 ? 128U
                                                  : columns <= 256 ? 256U : 512U;
}

// Visibility of one key for the query tokens: token t sees it iff first <= t <= last.
struct TokenRange {
  int first;
  int last;
};

__device__ __forceinline__ TokenRange proposal_range(int proposal, int proposals) {
  TokenRange range{1 << 30, -1};
  if (proposal < proposals) {
    range.first = proposal;
    range.last = 1 << 30;
  }
  return range;
}

// mode 0: everything in the cache is visible; 1: causal over a linear cache that already holds the
// proposals (row <= position + token); 2: sliding ring read in place.
__device__ __forceinline__ TokenRange cache_range(const AttentionArguments &a, int mode,
                                                  int cache_row, int cache_rows, int position,
                                                  int newest_row) {
  TokenRange range{1 << 30, -1};
  if (cache_row < cache_rows) {
    range.first = 0;
    range.last = 1 << 30;
    if (mode == 1) {
      range.first = cache_row - position;      // token >= row - position
    } else if (mode == 2) {
      int distance = newest_row - cache_row;
      if (distance < 0)
        distance += a.capacity;
      range.last = a.window - 2 - distance;
    }
  }
  return range;
}

// ------------------------------------------------------------------------------------ scores
constexpr int scores_row_groups = 4;            // epilogue warps per TMEM lane quarter
constexpr int scores_epilogue_warps = 4 * scores_row_groups;
constexpr int scores_epilogue_threads = scores_epilogue_warps * 32;
constexpr int scores_threads = 64 + scores_epilogue_threads;   // warp 0 TMA, warp 1 MMA + TMEM

template <int dimension, int padded_rows> struct ScoresShape {
  static constexpr int subtiles = dimension / 64;
  static constexpr int query_bytes = subtiles * padded_rows * 128;
  static constexpr int budget = 227 * 1024 - 1024 - 8192 - query_bytes;
  static constexpr int stages = budget / stream_stage_bytes > 5 ? 5 : budget / stream_stage_bytes;
  static constexpr int shared_bytes = query_bytes + stages * stream_stage_bytes + 1024;
};

template <int dimension, int padded_rows>
__global__ void __launch_bounds__(scores_threads, 1)
scores_stream_kernel(const __grid_constant__ CUtensorMap key_map,
                     const __grid_constant__ CUtensorMap new_key_map,
                     const __grid_constant__ CUtensorMap query_map, const StreamArguments args) {
  using Shape = ScoresShape<dimension, padded_rows>;
  constexpr int stages = Shape::stages;
  constexpr int subtiles = Shape::subtiles;
  // An epilogue warp owns a quarter of the query rows and reads them 16 TMEM columns at a time.
  constexpr int parts = (padded_rows / scores_row_groups + 15) / 16;
  constexpr int slots = parts * 16;
  constexpr uint32_t idesc = ptx::umma_idesc(1, 1, stream_tile_keys, padded_rows);
  // The last 16-column read of the second half may run past the second accumulator.
  constexpr uint32_t tmem_columns = tmem_columns_for(2 * padded_rows + 16);
  const AttentionArguments &a = args.a;

  extern __shared__ unsigned char shared_raw[];
  // full[stages] empty[stages] acc_full[2] acc_empty[2] query_full query_free
  __shared__ __align__(8) unsigned long long barriers[2 * stages + 6];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_word;
  __shared__ float warp_maxima[scores_epilogue_warps][slots];
  __shared__ float warp_sums[scores_epilogue_warps][slots];
  __shared__ uint32_t token_slots[scores_row_groups][proposal_columns];
  __shared__ StreamSchedule schedule;
  volatile int *abort_flag = &abort_word;
  const uint32_t base = (ptx::smem_u32(shared_raw) + 1023U) & ~1023U;
  const uint32_t query_tiles = base;
  const uint32_t ring = base + Shape::query_bytes;
  const uint32_t full_bar = ptx::smem_u32(&barriers[0]);
  const uint32_t empty_bar = ptx::smem_u32(&barriers[stages]);
  const uint32_t acc_full_bar = ptx::smem_u32(&barriers[2 * stages]);
  const uint32_t acc_empty_bar = ptx::smem_u32(&barriers[2 * stages + 2]);
  const uint32_t query_full_bar = ptx::smem_u32(&barriers[2 * stages + 4]);
  const uint32_t query_free_bar = ptx::smem_u32(&barriers[2 * stages + 5]);

  const int warp = static_cast<int>(threadIdx.x) / 32;
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int group = a.query_heads / a.kv_heads;
  const int rows = group * a.depth;

  grid_dependency_launch();
  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int stage = 0; stage < stages; ++stage) {
      ptx::mbarrier_init(full_bar + 8U * stage, 1);
      ptx::mbarrier_init(empty_bar + 8U * stage, 1);
    }
    for (int buffer = 0; buffer < 2; ++buffer) {
      ptx::mbarrier_init(acc_full_bar + 8U * buffer, 1);
      ptx::mbarrier_init(acc_empty_bar + 8U * buffer, scores_epilogue_warps);
    }
    ptx::mbarrier_init(query_full_bar, 1);
    ptx::mbarrier_init(query_free_bar, 1);
    ptx::fence_mbarrier_init();
    ptx::prefetch_tensormap(&key_map);
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
  // The schedule depends on the requests' positions only; when those are the step's inputs it is
  // laid out while the previous grid still runs.
  if (a.inputs_static != 0)
    build_schedule(a, schedule);
  grid_dependency_wait();
  if (a.inputs_static == 0)
    build_schedule(a, schedule);
  __syncthreads();

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t stream_policy = ptx::policy_evict_first();
      const uint64_t reuse_policy = ptx::policy_evict_last();
      Cursor<stages> cursor;
      bool healthy = true;
      uint32_t local = 0;
      for (int ordinal = 0; ordinal < schedule.count && healthy; ++ordinal) {
        const StreamItem item = cached_item(a, schedule, ordinal);
        if (item.empty())
          continue;
        // One query buffer: it is free once every score instruction of the previous item is done.
        // The K tiles of this item do not have to wait for that, so the query load is issued
        // from inside the waits for ring slots, as soon as the buffer is released. (It cannot
        // simply come first: the ring would drain. It cannot simply come last: the ring may be
        // full of this item's tiles, which nothing consumes before the queries arrive.)
        const uint32_t query_parity = (local & 1U) ^ 1U;
        ++local;
        bool query_pending = true;
        auto load_queries = [&]() {
          ptx::mbarrier_arrive_expect_tx(query_full_bar, Shape::query_bytes);
#pragma unroll
          for (int sub = 0; sub < subtiles; ++sub)
            ptx::tma_load_2d(query_tiles + sub * padded_rows * 128, &query_map, sub * 64,
                             item.query_row0, query_full_bar, reuse_policy);
          query_pending = false;
        };
        auto wait_for_slot = [&]() -> bool {
          const uint32_t bar = empty_bar + 8U * cursor.stage;
          const uint32_t parity = cursor.phase ^ 1U;
          if (ptx::mbarrier_try_wait(bar, parity))
            return true;
          const long long start = clock64();
          for (;;) {
            if (query_pending && ptx::mbarrier_try_wait(query_free_bar, query_parity))
              load_queries();
            if (ptx::mbarrier_try_wait(bar, parity))
              return true;
            if (*abort_flag != 0)
              return false;
            if (clock64() - start > ptx::wait_cycle_limit) {
              *abort_flag = 1;
              atomicExch(args.device_error, 41);
              return false;
            }
          }
        };
        if (ptx::mbarrier_try_wait(query_free_bar, query_parity))
          load_queries();
        if (item.proposals > 0) {
#pragma unroll 1
          for (int pair = 0; pair < subtiles / 2 && healthy; ++pair) {
            if (!wait_for_slot()) {
              healthy = false;
              break;
            }
            ptx::mbarrier_arrive_expect_tx(full_bar + 8U * cursor.stage,
                                           2 * proposal_columns * 128);
#pragma unroll
            for (int half = 0; half < 2; ++half)
              ptx::tma_load_2d(ring + cursor.stage * stream_stage_bytes +
                                   half * stream_subtile_bytes,
                               &new_key_map, (pair * 2 + half) * 64, item.staged_row0,
                               full_bar + 8U * cursor.stage, reuse_policy);
            cursor.advance();
          }
        }
        const int tiles = (item.rows_here + stream_tile_keys - 1) / stream_tile_keys;
        for (int tile = 0; tile < tiles && healthy; ++tile) {
          const int row = item.cache_row0 + item.first_row + tile * stream_tile_keys;
#pragma unroll
          for (int pair = 0; pair < subtiles / 2; ++pair) {
            if (!wait_for_slot()) {
              healthy = false;
              break;
            }
            ptx::mbarrier_arrive_expect_tx(full_bar + 8U * cursor.stage, stream_stage_bytes);
#pragma unroll
            for (int half = 0; half < 2; ++half)
              ptx::tma_load_2d(ring + cursor.stage * stream_stage_bytes +
                                   half * stream_subtile_bytes,
                               &key_map, (pair * 2 + half) * 64, row,
                               full_bar + 8U * cursor.stage, stream_policy);
            cursor.advance();
          }
        }
        if (healthy && query_pending) {
          if (!ptx::mbarrier_wait_checked(query_free_bar, query_parity, abort_flag, args.device_error, 40)) {
            healthy = false;
            break;
          }
          load_queries();
        }
      }
      if (!healthy) {
        // Let the copies in flight land before the CTA exits: every stage's current phase.
        for (uint32_t stage = 0; stage < static_cast<uint32_t>(stages); ++stage)
          ptx::mbarrier_wait_bounded(full_bar + 8U * stage,
                                     stage < cursor.stage ? cursor.phase : cursor.phase ^ 1U);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint64_t key_desc = ptx::umma_desc_k_major_sw128(ring);
      const uint32_t desc_high = static_cast<uint32_t>(key_desc >> 32);
      const uint32_t key_low = static_cast<uint32_t>(key_desc);
      const uint32_t query_low = static_cast<uint32_t>(ptx::umma_desc_k_major_sw128(query_tiles));
      Cursor<stages> cursor;
      uint32_t accumulator = 0;
      uint32_t accumulator_phase = 0;
      bool healthy = true;
      uint32_t local = 0;
      for (int ordinal = 0; ordinal < schedule.count && healthy; ++ordinal) {
        const StreamItem item = cached_item(a, schedule, ordinal);
        if (item.empty())
          continue;
        if (!ptx::mbarrier_wait_checked(query_full_bar, local & 1U, abort_flag, args.device_error, 42)) {
          healthy = false;
          break;
        }
        ++local;
        const int tiles = (item.proposals > 0 ? 1 : 0) +
                          (item.rows_here + stream_tile_keys - 1) / stream_tile_keys;
        for (int tile = 0; tile < tiles && healthy; ++tile) {
          if (!ptx::mbarrier_wait_checked(acc_empty_bar + 8U * accumulator, accumulator_phase ^ 1U, abort_flag,
                            args.device_error, 43)) {
            healthy = false;
            break;
          }
          ptx::tcgen05_fence_after_thread_sync();
          const uint32_t tmem_scores = tmem_base + accumulator * padded_rows;
#pragma unroll
          for (int pair = 0; pair < subtiles / 2; ++pair) {
            if (!ptx::mbarrier_wait_checked(full_bar + 8U * cursor.stage, cursor.phase, abort_flag,
                              args.device_error, 44)) {
              healthy = false;
              break;
            }
            ptx::tcgen05_fence_after_thread_sync();
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const int sub = pair * 2 + half;
              const uint32_t a_low = key_low + cursor.stage * (stream_stage_bytes >> 4) +
                                     half * (stream_subtile_bytes >> 4);
              const uint32_t b_low = query_low + sub * ((padded_rows * 128) >> 4);
#pragma unroll
              for (int step = 0; step < 4; ++step)
                ptx::tcgen05_mma_f16_split(tmem_scores, a_low + 2 * step, desc_high,
                                           b_low + 2 * step, desc_high, idesc,
                                           (sub > 0 || step > 0) ? 1U : 0U);
            }
            ptx::tcgen05_commit(empty_bar + 8U * cursor.stage);
            cursor.advance();
          }
          if (healthy)
            ptx::tcgen05_commit(acc_full_bar + 8U * accumulator);
          accumulator ^= 1U;
          if (accumulator == 0)
            accumulator_phase ^= 1U;
        }
        if (healthy)
          ptx::tcgen05_commit(query_free_bar);
      }
    }
  } else {
    const int epilogue_warp = warp - 2;
    const int quarter = warp & 3;                 // TMEM lane quarter this warp may read
    const int row_group = epilogue_warp >> 2;     // which share of the query rows this warp owns
    const int thread = quarter * 32 + lane;       // key inside a tile
    const int epilogue_thread = epilogue_warp * 32 + lane;
    const int mode = a.draft ? 0 : a.new_keys == nullptr ? 1 : a.window > 0 ? 2 : 0;
    // The warp owns query rows [first_row, last_row): TMEM columns it reads 16 at a time. The
    // loop bodies below are branch-free per row so that the rows' dependency chains interleave.
    const int rows_per_group = (rows + scores_row_groups - 1) / scores_row_groups;
    const int first_row = row_group * rows_per_group;
    const int last_row = min(rows, first_row + rows_per_group);
    // token_slots[group][t]: bit s set iff slot s of that row group holds query token t
    // (slot s is row first_row + s, whose token is its index modulo depth). A key's visible
    // tokens then turn into a per-slot bit mask with a few ORs, and a slot's visibility is one
    // bit test with a compile-time shift.
    if (lane < proposal_columns && quarter == 0) {
      uint32_t mask = 0;
      for (int slot = 0; slot < slots; ++slot) {
        if ((first_row + slot) % a.depth == lane)
          mask |= 1U << slot;
      }
      token_slots[row_group][lane] = mask;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(scores_epilogue_threads) : "memory");
    auto *scores = static_cast<__nv_bfloat16 *>(a.scores);
    uint32_t tiles_done = 0;
    for (int ordinal = 0; ordinal < schedule.count; ++ordinal) {
      const StreamItem item = cached_item(a, schedule, ordinal);
      if (item.empty())
        continue;
      const int newest_row = item.position > 0 ? (item.position - 1) % a.capacity : 0;
      __nv_bfloat16 *score_rows =
          scores + static_cast<size_t>(item.query_row0 + first_row) * a.score_stride;
      float maxima[slots];
      float sums[slots];
#pragma unroll
      for (int slot = 0; slot < slots; ++slot) {
        maxima[slot] = masked_score;
        sums[slot] = 0.0F;
      }
      const int proposal_tiles = item.proposals > 0 ? 1 : 0;
      const int tiles = proposal_tiles + (item.rows_here + stream_tile_keys - 1) / stream_tile_keys;
      for (int tile = 0; tile < tiles; ++tile, ++tiles_done) {
        const uint32_t buffer = tiles_done & 1U;
        const bool ready =
            __all_sync(0xFFFFFFFFU, ptx::mbarrier_wait_checked(acc_full_bar + 8U * buffer, (tiles_done >> 1) & 1U,
                                                 abort_flag, args.device_error, 45)
                                        ? 1
                                        : 0) != 0;
        if (!ready)
          continue;
        ptx::tcgen05_fence_after_thread_sync();
        TokenRange range{1 << 30, -1};
        int column = -1;
        if (tile < proposal_tiles) {
          if (thread < proposal_columns) {
            column = thread;
            range = proposal_range(thread, item.proposals);
          }
        } else {
          const int cache_row = item.first_row + (tile - proposal_tiles) * stream_tile_keys + thread;
          column = proposal_columns + cache_row;
          range = cache_range(a, mode, cache_row, item.cache_rows, item.position, newest_row);
        }
        // Slots whose token lies in first..last.
        const int low = range.first < 0 ? 0 : range.first;
        const int high = range.last >= a.depth ? a.depth - 1 : range.last;
        uint32_t slot_mask = 0;
        for (int token = low; token <= high; ++token)
          slot_mask |= token_slots[row_group][token];
        const uint32_t lane_address = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                      buffer * padded_rows + first_row;
        __nv_bfloat16 *cell = score_rows + (column >= 0 ? column : 0);
#pragma unroll
        for (int part = 0; part < parts; ++part) {
          if (first_row + part * 16 < last_row) {     // warp-uniform
            uint32_t values[16];
            ptx::tmem_load_32x32b_x16(lane_address + part * 16, values);
            ptx::tmem_load_wait();
#pragma unroll
            for (int entry = 0; entry < 16; ++entry) {
              const int slot = part * 16 + entry;
              const bool visible = ((slot_mask >> slot) & 1U) != 0U;
              const __nv_bfloat16 rounded =
                  __float2bfloat16_rn(visible ? __uint_as_float(values[entry]) : -CUDART_INF_F);
              if (column >= 0 && first_row + slot < last_row)
                cell[static_cast<size_t>(slot) * a.score_stride] = rounded;
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
        ptx::tcgen05_fence_before_thread_sync();
        __syncwarp();
        if (lane == 0)
          ptx::mbarrier_arrive(acc_empty_bar + 8U * buffer);
      }
      // One (maximum, sum) pair per query row for this chunk. Threads whose key was never
      // visible (or lanes beyond the proposal columns) carry the neutral pair.
      {
        float warp_maximum[slots];
#pragma unroll
        for (int slot = 0; slot < slots; ++slot)
          warp_maximum[slot] = warp_max(maxima[slot]);
#pragma unroll
        for (int slot = 0; slot < slots; ++slot)
          sums[slot] = warp_sum(sums[slot] * __expf(maxima[slot] - warp_maximum[slot]));
        if (lane == 0) {
#pragma unroll
          for (int slot = 0; slot < slots; ++slot) {
            warp_maxima[epilogue_warp][slot] = warp_maximum[slot];
            warp_sums[epilogue_warp][slot] = sums[slot];
          }
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(scores_epilogue_threads) : "memory");
      if (epilogue_thread < rows) {
        const int row = epilogue_thread;
        const int owner = row / rows_per_group;
        const int slot = row - owner * rows_per_group;
        const int first_warp = owner * 4;
        float maximum = masked_score;
#pragma unroll
        for (int other = 0; other < 4; ++other)
          maximum = fmaxf(maximum, warp_maxima[first_warp + other][slot]);
        float total = 0.0F;
#pragma unroll
        for (int other = 0; other < 4; ++other)
          total += warp_sums[first_warp + other][slot] *
                   __expf(warp_maxima[first_warp + other][slot] - maximum);
        a.stats[static_cast<size_t>(item.query_row0 + row) * a.stats_stride + item.chunk] =
            make_float2(maximum, total);
      }
      asm volatile("bar.sync 1, %0;" ::"n"(scores_epilogue_threads) : "memory");
    }
  }

  ptx::tcgen05_fence_before_thread_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tcgen05_fence_after_thread_sync();
    ptx::tmem_dealloc(tmem_base, tmem_columns);
  }
}

// ------------------------------------------------------------------------------------ P.V
constexpr int values_output_warps = 4;
constexpr int values_builder_warps = 8;
constexpr int values_builder_threads = values_builder_warps * 32;
// warp 0 TMA, warp 1 MMA + TMEM, warps 2-5 output, warps 6-13 probability builders
constexpr int values_threads = 64 + values_output_warps * 32 + values_builder_threads;

template <int dimension, int padded_rows> struct ValuesShape {
  static constexpr int slices = dimension / 128;                  // UMMA M = 128 components each
  static constexpr int boxes = dimension / 64;                    // V boxes per stage
  static constexpr int value_box_bytes = stream_value_keys * 128; // [32 keys x 64 components]
  static constexpr int stage_bytes = boxes * value_box_bytes;     // 32 KB at 512, 16 KB at 256
  static constexpr int probability_box_bytes = padded_rows * 128; // [rows x 64 keys]
  static constexpr int probability_boxes = 6;
  static constexpr int budget = 227 * 1024 - 1024 - 6144 - probability_boxes * probability_box_bytes;
  static constexpr int fit = budget / stage_bytes;
  static constexpr int stages = fit > 10 ? 10 : fit;
  static constexpr int output_columns = slices * padded_rows;
  static constexpr int output_buffers = 2 * output_columns <= 512 ? 2 : 1;
  static constexpr int shared_bytes =
      probability_boxes * probability_box_bytes + stages * stage_bytes + 1024;
  // 16-byte chunks of one probability box a builder thread looks after
  static constexpr int chunks_per_thread =
      (padded_rows * 8 + values_builder_threads - 1) / values_builder_threads;
};

template <int dimension, int padded_rows>
__global__ void __launch_bounds__(values_threads, 1)
values_stream_kernel(const __grid_constant__ CUtensorMap value_map,
                     const __grid_constant__ CUtensorMap new_value_map,
                     const StreamArguments args) {
  using Shape = ValuesShape<dimension, padded_rows>;
  constexpr int stages = Shape::stages;
  constexpr int probability_boxes = Shape::probability_boxes;
  constexpr int output_buffers = Shape::output_buffers;
  // bf16 x bf16 -> fp32, A (V^T) MN-major: bit 15.
  constexpr uint32_t idesc = ptx::umma_idesc(1, 1, 128, padded_rows) | (1U << 15);
  constexpr uint32_t tmem_columns = tmem_columns_for(output_buffers * Shape::output_columns);
  const AttentionArguments &a = args.a;

  extern __shared__ unsigned char shared_raw[];
  // full[stages] empty[stages] p_full[boxes] p_empty[boxes] o_full[2] o_empty[2]
  __shared__ __align__(8) unsigned long long barriers[2 * stages + 2 * probability_boxes + 4];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_word;
  __shared__ StreamSchedule schedule;
  // Element offset of query row r inside a (request, kv head) block of the output:
  // token(r) * width + head(r) * dimension.
  __shared__ int row_offset[padded_rows];
  __shared__ float row_maximum[2][padded_rows];
  __shared__ float row_inverse_sum[2][padded_rows];
  volatile int *abort_flag = &abort_word;
  const uint32_t base = (ptx::smem_u32(shared_raw) + 1023U) & ~1023U;
  const uint32_t probability_ring = base;
  const uint32_t ring = base + probability_boxes * Shape::probability_box_bytes;
  unsigned char *const probability_generic = shared_raw + (base - ptx::smem_u32(shared_raw));
  const uint32_t full_bar = ptx::smem_u32(&barriers[0]);
  const uint32_t empty_bar = ptx::smem_u32(&barriers[stages]);
  const uint32_t p_full_bar = ptx::smem_u32(&barriers[2 * stages]);
  const uint32_t p_empty_bar = ptx::smem_u32(&barriers[2 * stages + probability_boxes]);
  const uint32_t o_full_bar = ptx::smem_u32(&barriers[2 * stages + 2 * probability_boxes]);
  const uint32_t o_empty_bar = ptx::smem_u32(&barriers[2 * stages + 2 * probability_boxes + 2]);

  const int warp = static_cast<int>(threadIdx.x) / 32;
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int group = a.query_heads / a.kv_heads;
  const int rows = group * a.depth;

  grid_dependency_launch();
  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int stage = 0; stage < stages; ++stage) {
      ptx::mbarrier_init(full_bar + 8U * stage, 1);
      ptx::mbarrier_init(empty_bar + 8U * stage, 1);
    }
    for (int box = 0; box < probability_boxes; ++box) {
      ptx::mbarrier_init(p_full_bar + 8U * box, values_builder_threads);
      ptx::mbarrier_init(p_empty_bar + 8U * box, 1);
    }
    for (int buffer = 0; buffer < 2; ++buffer) {
      ptx::mbarrier_init(o_full_bar + 8U * buffer, 1);
      ptx::mbarrier_init(o_empty_bar + 8U * buffer, values_output_warps);
    }
    ptx::fence_mbarrier_init();
    ptx::prefetch_tensormap(&value_map);
  }
  if (static_cast<int>(threadIdx.x) < padded_rows) {
    const int head = static_cast<int>(threadIdx.x) / a.depth;
    const int token = static_cast<int>(threadIdx.x) - head * a.depth;
    row_offset[threadIdx.x] = token * a.query_heads * dimension + head * dimension;
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&tmem_base_slot), tmem_columns);
    ptx::tmem_relinquish_alloc_permit();
  }
  ptx::tcgen05_fence_before_thread_sync();
  __syncthreads();
  ptx::tcgen05_fence_after_thread_sync();
  const uint32_t tmem_base = tmem_base_slot;
  // The schedule depends on the requests' positions only; when those are the step's inputs it is
  // laid out while the previous grid still runs.
  if (a.inputs_static != 0)
    build_schedule(a, schedule);
  grid_dependency_wait();
  if (a.inputs_static == 0)
    build_schedule(a, schedule);
  __syncthreads();

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t stream_policy = ptx::policy_evict_first();
      const uint64_t reuse_policy = ptx::policy_evict_last();
      Cursor<stages> cursor;
      bool healthy = true;
      for (int ordinal = 0; ordinal < schedule.count && healthy; ++ordinal) {
        const StreamItem item = cached_item(a, schedule, ordinal);
        if (item.empty())
          continue;
        if (item.proposals > 0) {
          if (!ptx::mbarrier_wait_checked(empty_bar + 8U * cursor.stage, cursor.phase ^ 1U, abort_flag,
                            args.device_error, 50)) {
            healthy = false;
            break;
          }
          const uint32_t destination = ring + cursor.stage * Shape::stage_bytes;
          ptx::mbarrier_arrive_expect_tx(full_bar + 8U * cursor.stage,
                                         Shape::boxes * proposal_columns * 128);
#pragma unroll
          for (int box = 0; box < Shape::boxes; ++box)
            ptx::tma_load_2d(destination + box * Shape::value_box_bytes, &new_value_map, box * 64,
                             item.staged_row0, full_bar + 8U * cursor.stage, reuse_policy);
          cursor.advance();
        }
        const int key_groups = (item.rows_here + stream_value_keys - 1) / stream_value_keys;
        int row = item.cache_row0 + item.first_row;
        for (int key_group = 0; key_group < key_groups; ++key_group, row += stream_value_keys) {
          if (!ptx::mbarrier_wait_checked(empty_bar + 8U * cursor.stage, cursor.phase ^ 1U, abort_flag,
                            args.device_error, 50)) {
            healthy = false;
            break;
          }
          const uint32_t destination = ring + cursor.stage * Shape::stage_bytes;
          ptx::mbarrier_arrive_expect_tx(full_bar + 8U * cursor.stage, Shape::stage_bytes);
#pragma unroll
          for (int box = 0; box < Shape::boxes; ++box)
            ptx::tma_load_2d(destination + box * Shape::value_box_bytes, &value_map, box * 64, row,
                             full_bar + 8U * cursor.stage, stream_policy);
          cursor.advance();
        }
      }
      if (!healthy) {
        for (uint32_t stage = 0; stage < static_cast<uint32_t>(stages); ++stage)
          ptx::mbarrier_wait_bounded(full_bar + 8U * stage,
                                     stage < cursor.stage ? cursor.phase : cursor.phase ^ 1U);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint64_t value_desc = ptx::umma_desc_mn_major_sw128(ring, Shape::value_box_bytes);
      const uint32_t desc_high = static_cast<uint32_t>(value_desc >> 32);
      const uint32_t value_low = static_cast<uint32_t>(value_desc);
      const uint32_t probability_low =
          static_cast<uint32_t>(ptx::umma_desc_k_major_sw128(probability_ring));
      Cursor<stages> cursor;
      Cursor<probability_boxes> probability_cursor;
      bool healthy = true;
      uint32_t local = 0;
      for (int ordinal = 0; ordinal < schedule.count && healthy; ++ordinal) {
        const StreamItem item = cached_item(a, schedule, ordinal);
        if (item.empty())
          continue;
        const uint32_t buffer = output_buffers == 2 ? (local & 1U) : 0U;
        const uint32_t use = output_buffers == 2 ? (local >> 1) : local;
        ++local;
        if (!ptx::mbarrier_wait_checked(o_empty_bar + 8U * buffer, (use & 1U) ^ 1U, abort_flag,
                          args.device_error, 51)) {
          healthy = false;
          break;
        }
        ptx::tcgen05_fence_after_thread_sync();
        const uint32_t tmem_output = tmem_base + buffer * Shape::output_columns;
        uint32_t accumulate = 0;
        if (item.proposals > 0) {
          if (!ptx::mbarrier_wait_checked(p_full_bar + 8U * probability_cursor.stage, probability_cursor.phase,
                            abort_flag, args.device_error, 52) ||
              !ptx::mbarrier_wait_checked(full_bar + 8U * cursor.stage, cursor.phase, abort_flag,
                            args.device_error, 53)) {
            healthy = false;
            break;
          }
          ptx::tcgen05_fence_after_thread_sync();
          const uint32_t a_low = value_low + cursor.stage * (Shape::stage_bytes >> 4);
          const uint32_t b_low =
              probability_low + probability_cursor.stage * (Shape::probability_box_bytes >> 4);
#pragma unroll
          for (int slice = 0; slice < Shape::slices; ++slice)
            ptx::tcgen05_mma_f16_split(tmem_output + slice * padded_rows,
                                       a_low + slice * ((2 * Shape::value_box_bytes) >> 4),
                                       desc_high, b_low, desc_high, idesc, 0U);
          accumulate = 1;
          ptx::tcgen05_commit(empty_bar + 8U * cursor.stage);
          ptx::tcgen05_commit(p_empty_bar + 8U * probability_cursor.stage);
          cursor.advance();
          probability_cursor.advance();
        }
        const int key_groups = (item.rows_here + stream_value_keys - 1) / stream_value_keys;
        for (int key_group = 0; key_group < key_groups; ++key_group) {
          const int half = key_group & 1;
          if (half == 0 &&
              !ptx::mbarrier_wait_checked(p_full_bar + 8U * probability_cursor.stage, probability_cursor.phase,
                            abort_flag, args.device_error, 52)) {
            healthy = false;
            break;
          }
          if (!ptx::mbarrier_wait_checked(full_bar + 8U * cursor.stage, cursor.phase, abort_flag,
                            args.device_error, 53)) {
            healthy = false;
            break;
          }
          ptx::tcgen05_fence_after_thread_sync();
          const uint32_t a_low = value_low + cursor.stage * (Shape::stage_bytes >> 4);
          // 32 keys = 64 bytes along the 128-byte rows of the probability box.
          const uint32_t b_low = probability_low +
                                 probability_cursor.stage * (Shape::probability_box_bytes >> 4) +
                                 half * 4;
#pragma unroll
          for (int step = 0; step < 2; ++step) {
#pragma unroll
            for (int slice = 0; slice < Shape::slices; ++slice) {
              // 16 keys per instruction = two 8-row swizzle atoms of a V box (2048 bytes); the
              // two 64-component halves of a 128-component slice are consecutive boxes.
              ptx::tcgen05_mma_f16_split(
                  tmem_output + slice * padded_rows,
                  a_low + slice * ((2 * Shape::value_box_bytes) >> 4) + step * (2048 >> 4),
                  desc_high, b_low + 2 * step, desc_high, idesc, step > 0 ? 1U : accumulate);
            }
          }
          accumulate = 1;
          ptx::tcgen05_commit(empty_bar + 8U * cursor.stage);
          cursor.advance();
          if (half == 1 || key_group + 1 == key_groups) {
            ptx::tcgen05_commit(p_empty_bar + 8U * probability_cursor.stage);
            probability_cursor.advance();
          }
        }
        if (healthy)
          ptx::tcgen05_commit(o_full_bar + 8U * buffer);
      }
    }
  } else if (warp < 2 + values_output_warps) {
    // ---- output: O[component, row] -> fp32 chunk partials, or bf16 when there is one chunk.
    // Chunks that hold none of a request's rows are not written at all: the request's chunk
    // count goes to a.request_chunks and the consumer of the partials stops there.
    const int quarter = warp & 3;
    const int width = a.query_heads * dimension;
    const size_t chunk_elements = static_cast<size_t>(a.requests) * a.depth * width;
    uint32_t local = 0;
    for (int ordinal = 0; ordinal < schedule.count; ++ordinal) {
      const StreamItem item = cached_item(a, schedule, ordinal);
      if (item.empty())
        continue;
      if (a.chunks > 1 && item.chunk == 0 && item.kv_head == 0 && warp == 2 && lane == 0) {
        const int by_rows = (item.cache_rows + a.chunk_keys - 1) / a.chunk_keys;
        a.request_chunks[item.request] = by_rows > 0 ? by_rows : 1;
      }
      const uint32_t buffer = output_buffers == 2 ? (local & 1U) : 0U;
      const uint32_t use = output_buffers == 2 ? (local >> 1) : local;
      ++local;
      const bool ready =
          __all_sync(0xFFFFFFFFU, ptx::mbarrier_wait_checked(o_full_bar + 8U * buffer, use & 1U, abort_flag,
                                               args.device_error, 54)
                                      ? 1
                                      : 0) != 0;
      ptx::tcgen05_fence_after_thread_sync();
      if (ready) {
        const uint32_t lane_address = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                      buffer * Shape::output_columns;
        // First element of this (request, kv head) block, plus this thread's component.
        const size_t block_base = static_cast<size_t>(item.request) * a.depth * width +
                                  static_cast<size_t>(item.kv_head) * group * dimension +
                                  quarter * 32 + lane;
        float *partial_base =
            a.chunks > 1 ? a.chunk_partials + item.chunk * chunk_elements + block_base : nullptr;
        __nv_bfloat16 *output_base =
            a.chunks > 1 ? nullptr : static_cast<__nv_bfloat16 *>(a.output) + block_base;
#pragma unroll
        for (int slice = 0; slice < Shape::slices; ++slice) {
#pragma unroll
          for (int part = 0; part < padded_rows / 16; ++part) {
            if (part * 16 < rows) {           // warp-uniform
              uint32_t values[16];
              ptx::tmem_load_32x32b_x16(lane_address + slice * padded_rows + part * 16, values);
              ptx::tmem_load_wait();
#pragma unroll
              for (int entry = 0; entry < 16; ++entry) {
                const int row = part * 16 + entry;
                if (row < rows) {
                  const int offset = row_offset[row] + slice * 128;
                  if (a.chunks > 1)
                    partial_base[offset] = __uint_as_float(values[entry]);
                  else
                    output_base[offset] = __float2bfloat16_rn(__uint_as_float(values[entry]));
                }
              }
            }
          }
        }
      }
      ptx::tcgen05_fence_before_thread_sync();
      __syncwarp();
      if (lane == 0)
        ptx::mbarrier_arrive(o_empty_bar + 8U * buffer);
    }
  } else {
    // ---- probability builders
    const int builder_thread = (warp - 2 - values_output_warps) * 32 + lane;
    const auto *scores = static_cast<const __nv_bfloat16 *>(a.scores);
    Cursor<probability_boxes> cursor;
    uint32_t local = 0;
    for (int ordinal = 0; ordinal < schedule.count; ++ordinal) {
      const StreamItem item = cached_item(a, schedule, ordinal);
      if (item.empty())
        continue;
      const uint32_t parity = local & 1U;
      ++local;
      // Merge the chunk statistics of this head group's rows (same result in every chunk's CTA).
      if (builder_thread < rows) {
        const int request_chunks_by_rows = (item.cache_rows + a.chunk_keys - 1) / a.chunk_keys;
        const KeyGeometry g = key_geometry(a, item.request);
        const int request_chunks =
            request_chunks_by_rows > 0 ? request_chunks_by_rows : (g.proposals > 0 ? 1 : 0);
        const float2 *stats =
            a.stats + static_cast<size_t>(item.query_row0 + builder_thread) * a.stats_stride;
        float maximum = masked_score;
        for (int chunk = 0; chunk < request_chunks; ++chunk)
          maximum = fmaxf(maximum, stats[chunk].x);
        float total = 0.0F;
        for (int chunk = 0; chunk < request_chunks; ++chunk)
          total += stats[chunk].y * __expf(stats[chunk].x - maximum);
        row_maximum[parity][builder_thread] = maximum;
        row_inverse_sum[parity][builder_thread] = 1.0F / total;
      }
      asm volatile("bar.sync 2, %0;" ::"n"(values_builder_threads) : "memory");
      const __nv_bfloat16 *score_rows =
          scores + static_cast<size_t>(item.query_row0) * a.score_stride;
      const int proposal_boxes = item.proposals > 0 ? 1 : 0;
      const int boxes = proposal_boxes + (item.rows_here + 63) / 64;
      auto load_box = [&](int box, uint4 (&destination)[Shape::chunks_per_thread]) {
        const bool proposal = box < proposal_boxes;
        const int chunk_shift = proposal ? 1 : 3;
        const int box_chunks = rows << chunk_shift;
        const int column0 =
            proposal ? 0 : proposal_columns + item.first_row + (box - proposal_boxes) * 64;
#pragma unroll
        for (int mine = 0; mine < Shape::chunks_per_thread; ++mine) {
          const int chunk_index = builder_thread + mine * values_builder_threads;
          if (chunk_index < box_chunks) {
            const int row = chunk_index >> chunk_shift;
            const int chunk = chunk_index & ((1 << chunk_shift) - 1);
            destination[mine] = *reinterpret_cast<const uint4 *>(
                score_rows + static_cast<size_t>(row) * a.score_stride + column0 + chunk * 8);
          }
        }
      };
      uint4 ahead[Shape::chunks_per_thread];
      load_box(0, ahead);
      for (int box = 0; box < boxes; ++box) {
        const bool proposal = box < proposal_boxes;
        // 16-byte chunks of eight keys: two per row for the proposal box, eight otherwise.
        const int chunk_shift = proposal ? 1 : 3;
        const int box_chunks = rows << chunk_shift;
        // The scores of this box were requested one box ago; request the next box's now so that
        // their L2 latency overlaps this box's arithmetic.
        uint4 raw[Shape::chunks_per_thread];
#pragma unroll
        for (int mine = 0; mine < Shape::chunks_per_thread; ++mine)
          raw[mine] = ahead[mine];
        if (box + 1 < boxes)
          load_box(box + 1, ahead);
        const bool free_slot =
            __all_sync(0xFFFFFFFFU, ptx::mbarrier_wait_checked(p_empty_bar + 8U * cursor.stage,
                                                 cursor.phase ^ 1U, abort_flag, args.device_error,
                                                 55)
                                        ? 1
                                        : 0) != 0;
        unsigned char *slot = probability_generic + cursor.stage * Shape::probability_box_bytes;
        if (free_slot) {
#pragma unroll
          for (int mine = 0; mine < Shape::chunks_per_thread; ++mine) {
            const int chunk_index = builder_thread + mine * values_builder_threads;
            if (chunk_index < box_chunks) {
              const int row = chunk_index >> chunk_shift;
              const int chunk = chunk_index & ((1 << chunk_shift) - 1);
              const float maximum = row_maximum[parity][row];
              const float inverse_sum = row_inverse_sum[parity][row];
              auto *pairs = reinterpret_cast<__nv_bfloat162 *>(&raw[mine]);
#pragma unroll
              for (int pair = 0; pair < 4; ++pair) {
                const float2 both = __bfloat1622float2(pairs[pair]);
                pairs[pair] =
                    __halves2bfloat162(__float2bfloat16_rn(expf(both.x - maximum) * inverse_sum),
                                       __float2bfloat16_rn(expf(both.y - maximum) * inverse_sum));
              }
              *reinterpret_cast<uint4 *>(slot + row * 128 + ((chunk ^ (row & 7)) << 4)) = raw[mine];
            }
          }
        }
        // Make the generic-proxy writes visible to the tensor core before signalling.
        ptx::fence_proxy_async();
        ptx::mbarrier_arrive(p_full_bar + 8U * cursor.stage);
        cursor.advance();
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

// output[i] = bf16(sum over the request's chunks of partials[chunk, i]), in index order.
__global__ void sum_chunks_kernel(const float *partials, const int *request_chunks,
                                  size_t request_elements, size_t elements,
                                  __nv_bfloat16 *output) {
  grid_dependency_launch();
  grid_dependency_wait();
  const size_t index = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (index >= elements)
    return;
  const int chunks = request_chunks[index / request_elements];
  float4 total = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
  for (int chunk = 0; chunk < chunks; ++chunk) {
    const float4 part = *reinterpret_cast<const float4 *>(partials + chunk * elements + index);
    total.x += part.x;
    total.y += part.y;
    total.z += part.z;
    total.w += part.w;
  }
  __nv_bfloat162 low = __halves2bfloat162(__float2bfloat16_rn(total.x), __float2bfloat16_rn(total.y));
  __nv_bfloat162 high = __halves2bfloat162(__float2bfloat16_rn(total.z), __float2bfloat16_rn(total.w));
  uint2 packed;
  packed.x = *reinterpret_cast<const uint32_t *>(&low);
  packed.y = *reinterpret_cast<const uint32_t *>(&high);
  *reinterpret_cast<uint2 *>(output + index) = packed;
}

// UMMA N for `rows` query rows per KV head is attention_padded_rows(rows): 16, 48 or 80.
template <int dimension, int padded_rows>
int launch_stream(const AttentionArguments &a, int *device_error, cudaStream_t stream) {
  using Scores = ScoresShape<dimension, padded_rows>;
  using Values = ValuesShape<dimension, padded_rows>;
  static PerDeviceOnce configured;
  if (configured.run([] {
        const cudaError_t first = cudaFuncSetAttribute(
            scores_stream_kernel<dimension, padded_rows>,
            cudaFuncAttributeMaxDynamicSharedMemorySize, Scores::shared_bytes);
        if (first != cudaSuccess)
          return first;
        return cudaFuncSetAttribute(values_stream_kernel<dimension, padded_rows>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Values::shared_bytes);
      }) != cudaSuccess) {
    return -10;
  }
  const int multiprocessors = device_multiprocessors();
  const AttentionMaps &maps = *a.maps;
  const int items = a.chunks * a.requests * a.kv_heads;
  const StreamArguments arguments{a, device_error, items};
  const bool staged = a.new_keys != nullptr;
  const dim3 grid(static_cast<unsigned>(items < multiprocessors ? items : multiprocessors));
  cudaError_t status = launch_chained(
      scores_stream_kernel<dimension, padded_rows>, grid, dim3(scores_threads),
      Scores::shared_bytes, stream, false, maps.keys, staged ? maps.new_keys : maps.keys,
      maps.queries, arguments);
  if (status != cudaSuccess)
    return -11;
  status = launch_chained(values_stream_kernel<dimension, padded_rows>, grid, dim3(values_threads),
                          Values::shared_bytes, stream, false, maps.values32,
                          staged ? maps.new_values : maps.values32, arguments);
  if (status != cudaSuccess)
    return -11;
  if (a.chunks > 1 && a.sum_chunks != 0) {
    const size_t elements =
        static_cast<size_t>(a.requests) * a.depth * a.query_heads * dimension;
    const unsigned blocks = static_cast<unsigned>((elements / 4 + 255) / 256);
    const size_t request_elements = static_cast<size_t>(a.depth) * a.query_heads * dimension;
    status = launch_chained(sum_chunks_kernel, dim3(blocks), dim3(256), 0, stream, false,
                            static_cast<const float *>(a.chunk_partials),
                            static_cast<const int *>(a.request_chunks), request_elements,
                            elements, static_cast<__nv_bfloat16 *>(a.output));
  }
  return status == cudaSuccess ? 0 : -11;
}

template <int dimension>
int launch_stream_rows(const AttentionArguments &a, int *device_error, cudaStream_t stream) {
  switch (a.maps->padded_rows) {
  case 16:
    return launch_stream<dimension, 16>(a, device_error, stream);
  case 48:
    return launch_stream<dimension, 48>(a, device_error, stream);
  case 80:
    return launch_stream<dimension, 80>(a, device_error, stream);
  default:
    return -2;
  }
}


} // namespace

int launch_attention_stream(const AttentionArguments &a, int *device_error, cudaStream_t stream) {
  if (a.maps == nullptr || a.stats == nullptr || a.stats_stride < a.chunks || a.chunks < 1 ||
      (a.chunks > 1 && (a.chunk_partials == nullptr || a.request_chunks == nullptr)) ||
      a.requests > schedule_requests || a.chunk_keys <= 0 ||
      a.chunk_keys % stream_tile_keys != 0 ||
      a.capacity % stream_tile_keys != 0) {
    return -1;
  }
  switch (a.head_dim) {
  case 256:
    return launch_stream_rows<256>(a, device_error, stream);
  case 512:
    return launch_stream_rows<512>(a, device_error, stream);
  default:
    return -3;
  }
}


} // namespace carat_b200
