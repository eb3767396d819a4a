// Tensor maps of the tensor-core attention kernels. All tiles are bf16 with 128-byte rows
// (64 elements) and the 128-byte swizzle, so one tile row is one swizzle-atom row.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

namespace carat_b200 {

struct AttentionMaps {
  CUtensorMap keys;        // cache K as [slots * kv_heads * capacity, head_dim], box 128 rows
  CUtensorMap new_keys;    // staged proposals as [requests * kv_heads * depth, head_dim], box 16 rows
  CUtensorMap new_values;
  CUtensorMap queries;     // [query rows, head_dim], box padded_rows rows
  int padded_rows;         // UMMA N: 16, 48 or 80 (>= query_heads / kv_heads * depth)
  CUtensorMap values32;    // cache V with 32-row boxes
  int has_fused;           // head_dim 256: the one-kernel path may be used
};

// UMMA N for `rows` query rows per KV head, or 0 when there are too many.
inline int attention_padded_rows(int rows) {
  return rows <= 16 ? 16 : rows <= 48 ? 48 : rows <= 80 ? 80 : 0;
}

// Encodes the maps. `staged_*` may be null (global layers, drafter). row counts are the extents
// of the underlying buffers (an upper bound is fine: rows beyond what a launch uses are never
// stored). Returns 0 or a negative code.
int make_attention_maps(AttentionMaps *maps, const void *key_cache, const void *value_cache,
                        long long cache_rows, const void *staged_keys, const void *staged_values,
                        long long staged_rows, const void *queries, long long query_rows,
                        const void *scores, long long score_rows, int score_stride, int head_dim,
                        int padded_rows);

struct AttentionArguments;

// The one-kernel path (scores, softmax and P.V inside one CTA per (request, kv head)): head_dim
// 256, at most 16 query rows per KV head, at most 1024 cache rows, a single chunk, and either
// staged proposals or drafter semantics.
bool attention_fused_applies(const AttentionArguments &arguments);
int launch_attention_fused(const AttentionArguments &arguments, int *device_error,
                           cudaStream_t stream);

// The two-kernel path for everything else the tensor cores cover (head_dim 256 or 512, any number
// of chunks): persistent scores kernel with per-chunk softmax statistics, persistent P.V kernel
// that builds the probabilities on the fly. Needs arguments.stats.
int launch_attention_stream(const AttentionArguments &arguments, int *device_error,
                            cudaStream_t stream);

} // namespace carat_b200
