// Tensor maps and dispatch of the tensor-core attention kernels (head_dim 256 / 512).
//
// All kernels are "stream one operand from HBM exactly once" kernels: the K (or V) cache rows of
// one (request, kv head) are the UMMA M-side operand streamed through a TMA ring, the handful of
// query rows (or probability rows) of that head group is the UMMA N side, accumulators live in TMEM.
//   scores: S[key, row] = K[key, :] . Q[row, :]     A = K tile (K-major), B = Q (K-major)
//   P.V   : O[d, row]   = sum_key V[key, d] P[row, key]
//                                                   A = V tile read as V^T (MN-major), B = P
// attention_fused.cu holds the one-kernel form for sliding layers, attention_stream.cu the
// two-kernel form for everything else.
#include "attention.cuh"
#include "attention_geometry.cuh"
#include "attention_tc.cuh"
#include "context.cuh"
#include "launch.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>

namespace carat_b200 {
namespace {

constexpr int tile_rows = 128;         // cache rows per K tile
constexpr int stream_value_rows = 32;  // cache rows per V stage

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

// CARAT_B200_FUSED_ATTENTION=0 sends every layer through the two-kernel path (for comparisons).
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
      !encode_bf16_rows(&result.queries, queries, query_rows, head_dim, padded_rows) ||
      scores == nullptr || score_rows <= 0) {
    return -5;
  }
  if (!encode_bf16_rows(&result.values32, value_cache, cache_rows, head_dim, stream_value_rows))
    return -5;
  result.has_fused = head_dim == 256 ? 1 : 0;
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

int attention_tc_launches(const AttentionArguments &a) {
  if (attention_fused_applies(a) && fused_enabled())
    return 1;
  return 2 + ((a.chunks > 1 && a.sum_chunks != 0) ? 1 : 0);
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
  return launch_attention_stream(a, device_error, stream);
}

} // namespace carat_b200
