// Q/K/V post-processing of the packed QKV projection: per-head RMSNorm, rotate-half RoPE with bf16
// cos/sin tables, and the K/V store (reference: cuda/qkv.cu:44-64,387-422,477-530).
#pragma once

#include <cuda_runtime.h>

namespace carat_b200 {

// bf16 tables [positions, head_dim]; sliding layers rotate every pair with theta^(-2i/D); global
// layers ("proportional") rotate only the first D/8 pairs, the rest have angle 0
// (cuda/qkv.cu:44-64). Both halves of a row hold the same values.
int launch_rope_tables(void *cosine, void *sine, int positions, int head_dim, float theta,
                       bool proportional, cudaStream_t stream);

struct QkvPostArguments {
  const void *packed;          // [rows, query_width + kv_width * (key_equals_value ? 1 : 2)] bf16
  const void *query_norm;      // [head_dim] bf16
  const void *key_norm;        // [head_dim] bf16
  const void *cosine;          // [positions, head_dim] bf16
  const void *sine;
  void *queries;               // out [requests, query_heads, depth, head_dim] bf16
  // K/V rows of request r, head h, proposal t are written to
  //   base + slot_stride * slots[r] + head_stride * h + row * head_dim, where
  //   row = (positions[r] + t) % capacity  when `direct` (global layers: straight into the cache)
  //   row = t                              otherwise (sliding layers: a staging area indexed by
  //                                        request instead of slot; slot_stride is per request)
  void *key_base;
  void *value_base;
  long long slot_stride;       // elements
  long long head_stride;       // elements
  const int *positions;        // [requests] first proposal's logical position
  const int *slots;            // [requests]; ignored (request index used) when !direct
  int direct;
  int capacity;
  int requests;
  int depth;
  int query_heads;
  int kv_heads;
  int head_dim;                // 64, 256 or 512
  int key_equals_value;
  int max_positions;           // rows in the cos/sin tables
  float epsilon;
  int inputs_static;           // 1: positions (and slots) were written before the chain of
                               // dependent launches began; the kernel then fetches them and the
                               // cos/sin rows while the previous grid still runs
};

int launch_qkv_post(const QkvPostArguments &arguments, cudaStream_t stream);

// Query-only variant for the drafter (cuda/qkv.cu run_query_ragged): one row per request,
// rotated at positions[r] + position_offset. Output [requests, query_heads, 1, head_dim].
// inputs_static: as in QkvPostArguments.
int launch_query_post(const void *projected, const void *query_norm, const void *cosine,
                      const void *sine, void *queries, const int *positions, int position_offset,
                      int requests, int query_heads, int head_dim, int max_positions,
                      float epsilon, cudaStream_t stream, bool inputs_static = false);

} // namespace carat_b200
