// Tensor-core attention phases 1 (scores) and 3 (P.V) for head_dim 256 / 512.
//
// Both are "stream one operand from HBM exactly once" kernels: the K (or V) cache rows of one
// (request, kv head) are the UMMA M-side operand streamed through a TMA ring, the handful of query
// rows (or probability rows) of that head group is the UMMA N side, accumulators live in TMEM.
//   scores: S[key, row] = K[key, :] . Q[row, :]     A = K tile (K-major), B = Q (K-major)
//   P.V   : O[d, row]   = sum_key V[key, d] P[row, key]
//                                                   A = V tile read as V^T (MN-major), B = P
// Every wait is bounded; a wait that runs out records a code in the device error word.
#include "attention.cuh"
#include "attention_geometry.cuh"
#include "attention_tc.cuh"
#include "context.cuh"
#include "launch.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>

namespace carat_b200 {
namespace {

constexpr int tc_threads = 192;        // warp 0 TMA, warp 1 MMA + TMEM, warps 2-5 epilogue
constexpr int tile_rows = 128;         // cache rows per tile (UMMA M)
constexpr int subtile_bytes = tile_rows * 128;   // [128 rows x 64 bf16]
constexpr int score_chunk_rows = 1024; // cache rows one scores CTA covers

__host__ __device__ constexpr uint32_t tmem_columns_for(int columns) {
  return columns <= 32 ? 32U : columns <= 64 ? 64U : columns <= 128 ? 128U : 256U;
}

struct TcArguments {
  AttentionArguments a;
  int *device_error;
};

// ------------------------------------------------------------------------------------ scores
template <int dimension, int padded_rows>
__global__ void __launch_bounds__(tc_threads, 1)
scores_tc_kernel(const __grid_constant__ CUtensorMap key_map,
                 const __grid_constant__ CUtensorMap new_key_map,
                 const __grid_constant__ CUtensorMap query_map, const TcArguments args) {
  constexpr int subtiles = dimension / 64;        // 128-byte column blocks of a row
  constexpr int units = dimension / 256;          // pipeline units (4 subtiles) per key tile
  constexpr int stages = 2;
  constexpr uint32_t stage_bytes = 4 * subtile_bytes;
  constexpr uint32_t query_subtile_bytes = padded_rows * 128;
  constexpr uint32_t idesc = ptx::umma_idesc(1, 1, tile_rows, padded_rows);
  constexpr uint32_t tmem_columns = tmem_columns_for(2 * padded_rows);
  const AttentionArguments &a = args.a;

  extern __shared__ unsigned char shared_raw[];
  __shared__ __align__(8) unsigned long long barriers[2 * stages + 5];
  __shared__ uint32_t tmem_base_slot;
  const uint32_t base = (ptx::smem_u32(shared_raw) + 1023U) & ~1023U;
  const uint32_t query_tiles = base;
  const uint32_t key_stages = base + subtiles * query_subtile_bytes;
  // query_subtile_bytes is a multiple of 2048, so key_stages stays 1024-byte aligned.
  const uint32_t full_bar = ptx::smem_u32(&barriers[0]);
  const uint32_t empty_bar = ptx::smem_u32(&barriers[stages]);
  const uint32_t acc_full_bar = ptx::smem_u32(&barriers[2 * stages]);
  const uint32_t acc_empty_bar = ptx::smem_u32(&barriers[2 * stages + 2]);
  const uint32_t query_bar = ptx::smem_u32(&barriers[2 * stages + 4]);

  const int warp = static_cast<int>(threadIdx.x) / 32;
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int chunk = static_cast<int>(blockIdx.x);
  const int kv_head = static_cast<int>(blockIdx.y);
  const int request = static_cast<int>(blockIdx.z);
  const int group = a.query_heads / a.kv_heads;
  const int rows = group * a.depth;
  const KeyGeometry g = key_geometry(a, request);
  const int total_tiles = (g.cache_rows + tile_rows - 1) / tile_rows;
  const int first_tile = chunk * (score_chunk_rows / tile_rows);
  const int last_tile = min(total_tiles, first_tile + score_chunk_rows / tile_rows);
  const int cache_items = max(0, last_tile - first_tile);
  const int proposal_items = (chunk == 0 && g.proposals > 0) ? 1 : 0;
  const int items = proposal_items + cache_items;
  grid_dependency_launch();
  if (items == 0)
    return;
  const int query_row0 = (request * a.query_heads + kv_head * group) * a.depth;
  const long long cache_row0 =
      (static_cast<long long>(a.slots[request]) * a.kv_heads + kv_head) * a.capacity;
  const int staged_row0 = (request * a.kv_heads + kv_head) * a.depth;

  if (threadIdx.x == 0) {
    for (int stage = 0; stage < stages; ++stage) {
      ptx::mbarrier_init(full_bar + 8U * stage, 1);
      ptx::mbarrier_init(empty_bar + 8U * stage, 1);
    }
    for (int buffer = 0; buffer < 2; ++buffer) {
      ptx::mbarrier_init(acc_full_bar + 8U * buffer, 1);
      ptx::mbarrier_init(acc_empty_bar + 8U * buffer, 4);
    }
    ptx::mbarrier_init(query_bar, 1);
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
  grid_dependency_wait();

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t stream_policy = ptx::policy_evict_first();
      const uint64_t reuse_policy = ptx::policy_evict_last();
      ptx::mbarrier_arrive_expect_tx(query_bar, subtiles * query_subtile_bytes);
      for (int sub = 0; sub < subtiles; ++sub)
        ptx::tma_load_2d(query_tiles + sub * query_subtile_bytes, &query_map, sub * 64, query_row0,
                         query_bar, reuse_policy);
      int issued = 0;
      bool healthy = true;
      for (int item = 0; item < items && healthy; ++item) {
        const bool proposal = item < proposal_items;
        const int tile = first_tile + item - proposal_items;
        for (int unit = 0; unit < units; ++unit, ++issued) {
          const int stage = issued % stages;
          const uint32_t phase = static_cast<uint32_t>(issued / stages) & 1U;
          if (!ptx::mbarrier_wait_bounded(empty_bar + 8U * stage, phase ^ 1U)) {
            healthy = false;
            atomicExch(args.device_error, 11);
            break;
          }
          const uint32_t destination = key_stages + stage * stage_bytes;
          if (proposal) {
            ptx::mbarrier_arrive_expect_tx(full_bar + 8U * stage, 4 * proposal_columns * 128);
            for (int sub = 0; sub < 4; ++sub)
              ptx::tma_load_2d(destination + sub * subtile_bytes, &new_key_map,
                               (unit * 4 + sub) * 64, staged_row0, full_bar + 8U * stage,
                               reuse_policy);
          } else {
            ptx::mbarrier_arrive_expect_tx(full_bar + 8U * stage, stage_bytes);
            for (int sub = 0; sub < 4; ++sub)
              ptx::tma_load_2d(destination + sub * subtile_bytes, &key_map, (unit * 4 + sub) * 64,
                               static_cast<int>(cache_row0 + static_cast<long long>(tile) * tile_rows),
                               full_bar + 8U * stage, stream_policy);
          }
        }
      }
      if (!healthy) {
        const int first = issued > stages ? issued - stages : 0;
        for (int index = first; index < issued; ++index)
          ptx::mbarrier_wait_bounded(full_bar + 8U * (index % stages),
                                     static_cast<uint32_t>(index / stages) & 1U);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool healthy = ptx::mbarrier_wait_bounded(query_bar, 0);
      if (!healthy)
        atomicExch(args.device_error, 12);
      int consumed = 0;
      for (int item = 0; item < items && healthy; ++item) {
        const int buffer = item & 1;
        const uint32_t use = static_cast<uint32_t>(item >> 1);
        if (!ptx::mbarrier_wait_bounded(acc_empty_bar + 8U * buffer, (use & 1U) ^ 1U)) {
          healthy = false;
          atomicExch(args.device_error, 13);
          break;
        }
        ptx::tcgen05_fence_after_thread_sync();
        for (int unit = 0; unit < units; ++unit, ++consumed) {
          const int stage = consumed % stages;
          const uint32_t phase = static_cast<uint32_t>(consumed / stages) & 1U;
          if (!ptx::mbarrier_wait_bounded(full_bar + 8U * stage, phase)) {
            healthy = false;
            atomicExch(args.device_error, 14);
            break;
          }
          ptx::tcgen05_fence_after_thread_sync();
#pragma unroll
          for (int sub = 0; sub < 4; ++sub) {
            const uint64_t key_desc = ptx::umma_desc_k_major_sw128(
                key_stages + stage * stage_bytes + sub * subtile_bytes);
            const uint64_t query_desc = ptx::umma_desc_k_major_sw128(
                query_tiles + (unit * 4 + sub) * query_subtile_bytes);
#pragma unroll
            for (int step = 0; step < 4; ++step)
              ptx::tcgen05_mma_f16(tmem_base + buffer * padded_rows, key_desc + 2ULL * step,
                                   query_desc + 2ULL * step, idesc,
                                   (unit > 0 || sub > 0 || step > 0) ? 1U : 0U);
          }
          ptx::tcgen05_commit(empty_bar + 8U * stage);
        }
        if (healthy)
          ptx::tcgen05_commit(acc_full_bar + 8U * buffer);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int tile_row = quarter * 32 + lane;
    auto *score_rows = static_cast<__nv_bfloat16 *>(a.scores) +
                       static_cast<size_t>(query_row0) * a.score_stride;
    for (int item = 0; item < items; ++item) {
      const int buffer = item & 1;
      const uint32_t use = static_cast<uint32_t>(item >> 1);
      const bool ready =
          __all_sync(0xFFFFFFFFU,
                     ptx::mbarrier_wait_bounded(acc_full_bar + 8U * buffer, use & 1U) ? 1 : 0) != 0;
      if (!ready) {
        if (lane == 0)
          atomicExch(args.device_error, 15);
        break;
      }
      ptx::tcgen05_fence_after_thread_sync();
      const bool proposal = item < proposal_items;
      const int tile = first_tile + item - proposal_items;
      int column = -1;
      if (proposal) {
        if (tile_row < g.proposals)
          column = tile_row;
      } else if (tile * tile_rows + tile_row < g.cache_rows) {
        column = proposal_columns + tile * tile_rows + tile_row;
      }
      const uint32_t lane_address =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buffer * padded_rows;
#pragma unroll
      for (int part = 0; part < padded_rows / 16; ++part) {
        if (part * 16 < rows) {
          uint32_t values[16];
          ptx::tmem_load_32x32b_x16(lane_address + part * 16, values);
          ptx::tmem_load_wait();
          if (column >= 0) {
#pragma unroll
            for (int index = 0; index < 16; ++index) {
              const int row = part * 16 + index;
              if (row < rows)
                score_rows[static_cast<size_t>(row) * a.score_stride + column] =
                    __float2bfloat16_rn(__uint_as_float(values[index]));
            }
          }
        }
      }
      ptx::tcgen05_fence_before_thread_sync();
      __syncwarp();
      if (lane == 0)
        ptx::mbarrier_arrive(acc_empty_bar + 8U * buffer);
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
// One CTA covers every output component of one (request, kv head) over one chunk of cache rows, so
// whole V rows are fetched (a row is head_dim * 2 bytes of contiguous HBM) and the probability
// tile is loaded once. A pipeline stage holds 64 KB of V: 128 keys at head_dim 256, 64 keys at 512.
template <int dimension> struct PvShape {
  static constexpr int slices = dimension / 128;               // UMMA M = 128 components each
  static constexpr int stage_keys = 32768 / dimension;         // 128 or 64
  static constexpr int boxes = dimension / 64;                 // V boxes per stage
  static constexpr int box_bytes = stage_keys * 128;
  static constexpr int value_bytes = boxes * box_bytes;        // 64 KB
  static constexpr int score_boxes = stage_keys / 64;
};

template <int dimension, int padded_rows> __host__ __device__ constexpr int pv_stage_bytes() {
  return PvShape<dimension>::value_bytes + PvShape<dimension>::score_boxes * padded_rows * 128;
}

template <int dimension, int padded_rows> __host__ __device__ constexpr int pv_stages() {
  return (220 * 1024) / pv_stage_bytes<dimension, padded_rows>() >= 3 ? 3 : 2;
}

template <int dimension, int padded_rows>
__global__ void __launch_bounds__(tc_threads, 1)
pv_tc_kernel(const __grid_constant__ CUtensorMap value_map,
             const __grid_constant__ CUtensorMap new_value_map,
             const __grid_constant__ CUtensorMap score_map, const TcArguments args) {
  using Shape = PvShape<dimension>;
  constexpr int stages = pv_stages<dimension, padded_rows>();
  constexpr uint32_t score_box_bytes = padded_rows * 128;      // [padded_rows x 64 keys]
  constexpr uint32_t stage_bytes = pv_stage_bytes<dimension, padded_rows>();
  // bf16 x bf16 -> fp32, A (V^T) MN-major: bit 15.
  constexpr uint32_t idesc = ptx::umma_idesc(1, 1, 128, padded_rows) | (1U << 15);
  constexpr uint32_t tmem_columns =
      Shape::slices * padded_rows <= 256 ? tmem_columns_for(Shape::slices * padded_rows) : 512U;
  const AttentionArguments &a = args.a;

  extern __shared__ unsigned char shared_raw[];
  __shared__ __align__(8) unsigned long long barriers[2 * stages + 1];
  __shared__ uint32_t tmem_base_slot;
  const uint32_t base = (ptx::smem_u32(shared_raw) + 1023U) & ~1023U;
  const uint32_t full_bar = ptx::smem_u32(&barriers[0]);
  const uint32_t empty_bar = ptx::smem_u32(&barriers[stages]);
  const uint32_t acc_bar = ptx::smem_u32(&barriers[2 * stages]);

  const int warp = static_cast<int>(threadIdx.x) / 32;
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int chunk = static_cast<int>(blockIdx.x);
  const int kv_head = static_cast<int>(blockIdx.y);
  const int request = static_cast<int>(blockIdx.z);
  const int group = a.query_heads / a.kv_heads;
  const int rows = group * a.depth;
  const KeyGeometry g = key_geometry(a, request);
  const int total_tiles = (g.cache_rows + Shape::stage_keys - 1) / Shape::stage_keys;
  const int tiles_per_chunk = a.chunk_keys / Shape::stage_keys;
  const int first_tile = chunk * tiles_per_chunk;
  const int last_tile = min(total_tiles, first_tile + tiles_per_chunk);
  const int cache_items = max(0, last_tile - first_tile);
  const int proposal_items = (chunk == 0 && g.proposals > 0) ? 1 : 0;
  const int items = proposal_items + cache_items;
  const int query_row0 = (request * a.query_heads + kv_head * group) * a.depth;
  const long long cache_row0 =
      (static_cast<long long>(a.slots[request]) * a.kv_heads + kv_head) * a.capacity;
  const int staged_row0 = (request * a.kv_heads + kv_head) * a.depth;

  grid_dependency_launch();
  if (threadIdx.x == 0) {
    for (int stage = 0; stage < stages; ++stage) {
      ptx::mbarrier_init(full_bar + 8U * stage, 1);
      ptx::mbarrier_init(empty_bar + 8U * stage, 1);
    }
    ptx::mbarrier_init(acc_bar, 1);
    ptx::fence_mbarrier_init();
    ptx::prefetch_tensormap(&value_map);
    ptx::prefetch_tensormap(&score_map);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&tmem_base_slot), tmem_columns);
    ptx::tmem_relinquish_alloc_permit();
  }
  ptx::tcgen05_fence_before_thread_sync();
  __syncthreads();
  ptx::tcgen05_fence_after_thread_sync();
  const uint32_t tmem_base = tmem_base_slot;
  grid_dependency_wait();

  if (warp == 0) {
    if (lane == 0 && items > 0) {
      const uint64_t stream_policy = ptx::policy_evict_first();
      const uint64_t reuse_policy = ptx::policy_evict_last();
      int issued = 0;
      bool healthy = true;
      for (int item = 0; item < items; ++item, ++issued) {
        const int stage = issued % stages;
        const uint32_t phase = static_cast<uint32_t>(issued / stages) & 1U;
        if (!ptx::mbarrier_wait_bounded(empty_bar + 8U * stage, phase ^ 1U)) {
          healthy = false;
          atomicExch(args.device_error, 21);
          break;
        }
        const uint32_t values = base + stage * stage_bytes;
        const uint32_t scores = values + Shape::value_bytes;
        if (item < proposal_items) {
          ptx::mbarrier_arrive_expect_tx(full_bar + 8U * stage,
                                         Shape::boxes * proposal_columns * 128 + score_box_bytes);
          for (int box = 0; box < Shape::boxes; ++box)
            ptx::tma_load_2d(values + box * Shape::box_bytes, &new_value_map, box * 64, staged_row0,
                             full_bar + 8U * stage, reuse_policy);
          ptx::tma_load_2d(scores, &score_map, 0, query_row0, full_bar + 8U * stage, reuse_policy);
        } else {
          const int tile = first_tile + item - proposal_items;
          ptx::mbarrier_arrive_expect_tx(full_bar + 8U * stage, stage_bytes);
          for (int box = 0; box < Shape::boxes; ++box)
            ptx::tma_load_2d(
                values + box * Shape::box_bytes, &value_map, box * 64,
                static_cast<int>(cache_row0 + static_cast<long long>(tile) * Shape::stage_keys),
                full_bar + 8U * stage, stream_policy);
          for (int box = 0; box < Shape::score_boxes; ++box)
            ptx::tma_load_2d(scores + box * score_box_bytes, &score_map,
                             proposal_columns + tile * Shape::stage_keys + box * 64, query_row0,
                             full_bar + 8U * stage, reuse_policy);
        }
      }
      if (!healthy) {
        const int first = issued > stages ? issued - stages : 0;
        for (int index = first; index < issued; ++index)
          ptx::mbarrier_wait_bounded(full_bar + 8U * (index % stages),
                                     static_cast<uint32_t>(index / stages) & 1U);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && items > 0) {
      for (int item = 0; item < items; ++item) {
        const int stage = item % stages;
        const uint32_t phase = static_cast<uint32_t>(item / stages) & 1U;
        if (!ptx::mbarrier_wait_bounded(full_bar + 8U * stage, phase)) {
          atomicExch(args.device_error, 22);
          break;
        }
        ptx::tcgen05_fence_after_thread_sync();
        const uint32_t values = base + stage * stage_bytes;
        const uint32_t scores = values + Shape::value_bytes;
        const int steps = item < proposal_items ? 1 : Shape::stage_keys / 16;
        for (int step = 0; step < steps; ++step) {
          // 16 keys per instruction: two 8-row swizzle atoms of a V box (2048 bytes), and 32
          // bytes along the key axis of the probability box that holds them.
          const uint64_t score_desc =
              ptx::umma_desc_k_major_sw128(scores + (step / 4) * score_box_bytes) +
              2ULL * (step % 4);
#pragma unroll
          for (int slice = 0; slice < Shape::slices; ++slice) {
            const uint64_t value_desc = ptx::umma_desc_mn_major_sw128(
                values + 2 * slice * Shape::box_bytes + step * 2048, Shape::box_bytes);
            ptx::tcgen05_mma_f16(tmem_base + slice * padded_rows, value_desc, score_desc, idesc,
                                 (item > 0 || step > 0) ? 1U : 0U);
          }
        }
        ptx::tcgen05_commit(empty_bar + 8U * stage);
      }
      ptx::tcgen05_commit(acc_bar);
    }
  } else {
    const int quarter = warp & 3;
    bool ready = true;
    if (items > 0) {
      ready = __all_sync(0xFFFFFFFFU, ptx::mbarrier_wait_bounded(acc_bar, 0) ? 1 : 0) != 0;
      if (!ready && lane == 0)
        atomicExch(args.device_error, 23);
      ptx::tcgen05_fence_after_thread_sync();
    }
    const int width = a.query_heads * dimension;
    const uint32_t lane_address = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll
    for (int slice = 0; slice < Shape::slices; ++slice) {
      const int component = slice * 128 + quarter * 32 + lane;
#pragma unroll
      for (int part = 0; part < padded_rows / 16; ++part) {
        if (part * 16 < rows && ready) {
          uint32_t values[16];
          if (items > 0) {
            ptx::tmem_load_32x32b_x16(lane_address + slice * padded_rows + part * 16, values);
            ptx::tmem_load_wait();
          } else {
#pragma unroll
            for (int index = 0; index < 16; ++index)
              values[index] = 0U;
          }
#pragma unroll
          for (int index = 0; index < 16; ++index) {
            const int row = part * 16 + index;
            if (row < rows) {
              const int local_head = row / a.depth;
              const int token = row % a.depth;
              const size_t out_row = static_cast<size_t>(request) * a.depth + token;
              const size_t column =
                  static_cast<size_t>(kv_head * group + local_head) * dimension + component;
              const float value = __uint_as_float(values[index]);
              if (a.chunks > 1) {
                a.chunk_partials[(static_cast<size_t>(chunk) * a.requests * a.depth + out_row) *
                                     width +
                                 column] = value;
              } else {
                static_cast<__nv_bfloat16 *>(a.output)[out_row * width + column] =
                    __float2bfloat16_rn(value);
              }
            }
          }
        }
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

using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                 const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                 const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_entry() {
  static EncodeTiled entry = [] {
    void *function = nullptr;
    cudaDriverEntryPointQueryResult status{};
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &function, cudaEnableDefault, &status) !=
            cudaSuccess ||
        status != cudaDriverEntryPointSuccess) {
      return static_cast<EncodeTiled>(nullptr);
    }
    return reinterpret_cast<EncodeTiled>(function);
  }();
  return entry;
}

// bf16 matrix [rows, columns] row-major, box [box_rows, 64 columns], 128-byte swizzle.
bool encode_bf16_rows(CUtensorMap *map, const void *base, long long rows, long long columns,
                      int box_rows) {
  const EncodeTiled encode = encode_entry();
  if (encode == nullptr || base == nullptr || rows <= 0 || columns <= 0)
    return false;
  const cuuint64_t dimensions[2] = {static_cast<cuuint64_t>(columns), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(columns) * 2};
  const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t element_strides[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dimensions,
                strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int dimension, int padded_rows>
int launch_tc(const AttentionArguments &a, int *device_error, cudaStream_t stream) {
  constexpr int score_shared =
      (dimension / 64) * padded_rows * 128 + 2 * 4 * subtile_bytes + 1024;
  constexpr int pv_shared =
      pv_stages<dimension, padded_rows>() * pv_stage_bytes<dimension, padded_rows>() + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(scores_tc_kernel<dimension, padded_rows>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             score_shared) != cudaSuccess ||
        cudaFuncSetAttribute(pv_tc_kernel<dimension, padded_rows>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, pv_shared) != cudaSuccess) {
      return -10;
    }
    configured = true;
  }
  const AttentionMaps &maps = *a.maps;
  const TcArguments arguments{a, device_error};
  const bool staged = a.new_keys != nullptr;
  const dim3 score_grid(static_cast<unsigned>(attention_chunks(a.max_cache_rows, score_chunk_rows)),
                        static_cast<unsigned>(a.kv_heads), static_cast<unsigned>(a.requests));
  launch_chained(scores_tc_kernel<dimension, padded_rows>, score_grid, dim3(tc_threads),
                 score_shared, stream, false, maps.keys, staged ? maps.new_keys : maps.keys,
                 maps.queries, arguments);
  const int status = launch_attention_softmax(a, stream);
  if (status != 0)
    return status;
  const dim3 pv_grid(static_cast<unsigned>(a.chunks),
                     static_cast<unsigned>(a.kv_heads), static_cast<unsigned>(a.requests));
  launch_chained(pv_tc_kernel<dimension, padded_rows>, pv_grid, dim3(tc_threads), pv_shared, stream,
                 false, maps.values, staged ? maps.new_values : maps.values, maps.scores,
                 arguments);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -11;
}

template <int dimension>
int launch_tc_rows(const AttentionArguments &a, int *device_error, cudaStream_t stream) {
  switch (a.maps->padded_rows) {
  case 16:
    return launch_tc<dimension, 16>(a, device_error, stream);
  case 48:
    return launch_tc<dimension, 48>(a, device_error, stream);
  case 80:
    return launch_tc<dimension, 80>(a, device_error, stream);
  default:
    return -2;
  }
}

// CARAT_B200_FUSED_ATTENTION=0 keeps the three-kernel path everywhere (for comparisons).
bool fused_enabled() {
  static const bool enabled = [] {
    const char *configured = std::getenv("CARAT_B200_FUSED_ATTENTION");
    return configured == nullptr || configured[0] != '0';
  }();
  return enabled;
}

} // namespace

int make_attention_maps(AttentionMaps *maps, const void *key_cache, const void *value_cache,
                        long long cache_rows, const void *staged_keys, const void *staged_values,
                        long long staged_rows, const void *queries, long long query_rows,
                        const void *scores, long long score_rows, int score_stride, int head_dim,
                        int padded_rows) {
  if (maps == nullptr || (head_dim != 256 && head_dim != 512) || score_stride % 8 != 0 ||
      (padded_rows != 16 && padded_rows != 48 && padded_rows != 80)) {
    return -1;
  }
  AttentionMaps result{};
  result.padded_rows = padded_rows;
  if (!encode_bf16_rows(&result.keys, key_cache, cache_rows, head_dim, tile_rows) ||
      !encode_bf16_rows(&result.values, value_cache, cache_rows, head_dim, 32768 / head_dim) ||
      !encode_bf16_rows(&result.queries, queries, query_rows, head_dim, padded_rows) ||
      !encode_bf16_rows(&result.scores, scores, score_rows, score_stride, padded_rows)) {
    return -5;
  }
  if (head_dim == 256) {
    if (!encode_bf16_rows(&result.values32, value_cache, cache_rows, head_dim, 32))
      return -5;
    result.has_fused = 1;
  }
  if (staged_keys != nullptr) {
    if (!encode_bf16_rows(&result.new_keys, staged_keys, staged_rows, head_dim, proposal_columns) ||
        !encode_bf16_rows(&result.new_values, staged_values, staged_rows, head_dim,
                          proposal_columns)) {
      return -5;
    }
  }
  *maps = result;
  return 0;
}

int launch_attention_tc(const AttentionArguments &a, cudaStream_t stream) {
  const int status = validate_attention(a);
  if (status != 0)
    return status;
  if (a.maps == nullptr || a.capacity % tile_rows != 0 ||
      a.query_heads / a.kv_heads * a.depth > a.maps->padded_rows) {
    return -1;
  }
  int *device_error = device_error_word();
  if (device_error == nullptr)
    return -101;
  if (attention_fused_applies(a) && fused_enabled())
    return launch_attention_fused(a, device_error, stream);
  switch (a.head_dim) {
  case 256:
    return launch_tc_rows<256>(a, device_error, stream);
  case 512:
    return launch_tc_rows<512>(a, device_error, stream);
  default:
    return -3;
  }
}

} // namespace carat_b200
