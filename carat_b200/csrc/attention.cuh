// Attention of the verify step (depth proposal rows per request over that request's KV cache plus
// the proposals themselves) and of the drafter (one row per request over the target's cache).
//
// Reference semantics (cuda/prefill_gemm_attention.cu:165-349,552-730, cuda/gemm_attention.cu:88-132):
// scale 1.0; scores rounded to bf16; fp32 max / exp / sum over the visible keys; probabilities
// rounded to bf16 (masked keys are exactly 0); P.V accumulated in fp32 and rounded to bf16 once.
// Every implementation keeps these rounding points and streams each K and V row from HBM exactly
// once: the CUDA-core path in three kernels over a bf16 score buffer (like the reference's QK GEMM
// -> softmax -> PV GEMM), the tensor-core paths in one kernel (sliding layers: scores stay in
// shared memory) or two (scores + statistics, then P.V with the probabilities built on the fly).
//
// The score buffer's column layout (proposals in columns 0..15, cache rows from column 16 on) is
// described in attention_geometry.cuh. A sliding ring is read in place: physical row r holds the
// newest logical position p <= position-1 with p % capacity == r, and query t (at logical
// position position + t) sees it iff p >= position + t - (window - 1). Proposal u is visible to
// query t iff u <= t.
#pragma once

#include <cuda_runtime.h>

namespace carat_b200 {

struct AttentionArguments {
  const void *queries;       // [requests, query_heads, depth, head_dim] bf16
  const void *key_cache;     // layer base; row r of (slot, head) at
  const void *value_cache;   //   base + slot*slot_stride + head*head_stride + r*head_dim
  long long slot_stride;     // elements
  long long head_stride;     // elements
  // Proposal rows. When null the proposals are already in the cache at rows position + t
  // (global layers); otherwise row t of (request, head) is at
  //   new_keys + request*new_request_stride + head*new_head_stride + t*head_dim.
  const void *new_keys;
  const void *new_values;
  long long new_request_stride;
  long long new_head_stride;
  const int *positions;      // [requests] logical position of proposal 0
  const int *slots;          // [requests]
  void *scores;              // scratch [requests, query_heads, depth, score_stride] bf16
  int score_stride;          // >= score_columns(max_cache_rows), multiple of 8
  void *output;              // [requests * depth, query_heads * head_dim] bf16 (single chunk)
  float *chunk_partials;     // [chunks, requests * depth, query_heads * head_dim] fp32 (chunks > 1)
  int chunks;                // cache-row chunks the P.V phase is split into (1 = write bf16
                             // output); the proposal columns belong to chunk 0
  int chunk_keys;            // cache rows per chunk (multiple of 128)
  int requests;
  int depth;
  int query_heads;
  int kv_heads;
  int head_dim;              // 64, 256 or 512
  int capacity;              // rows per (slot, head) in the cache
  int window;                // sliding window, 0 = causal over the whole cache
  int max_cache_rows;        // upper bound over the requests of the cache rows that take part
                             // (see attention_geometry.cuh); sizes the grids
  // Tensor maps for the tensor-core kernels (null: the CUDA-core kernels run).
  const struct AttentionMaps *maps;
  // Scratch of the two-kernel tensor-core path: one (maximum, sum of exp) pair per score row and
  // chunk, [score rows, stats_stride] with stats_stride >= chunks.
  float2 *stats;
  int stats_stride;
  // chunks > 1 only: [requests] receives the number of chunks that hold any of the request's
  // rows. Chunk partials beyond that count are NOT written; whoever sums them must stop there.
  int *request_chunks;
  int sum_chunks;            // chunks > 1 only: also sum the chunk partials into `output` (bf16);
                             // otherwise the consumer of `chunk_partials` does the sum
  int draft;                 // 1: drafter semantics (depth == 1, no proposal rows, the first
                             //    min(position + 1, capacity) cache rows are visible)
  // 1: `positions` and `slots` were last written before the chain of dependent launches this
  // call is part of began (the runner's step inputs, copied in ahead of the first kernel): the
  // kernels then read them, and lay out their work, before they wait for the previous grid.
  int inputs_static;
  // 1 (needs inputs_static): the cache rows this call reads and `positions` / `slots` were last written before the
  // chain of dependent launches this call is part of began (a verify or draft step: the rings
  // change only in the commit at its end). The one-kernel path then requests its first key tiles
  // before it waits for the previous grid. 0 (any other caller): nothing is read early.
  int cache_static;
  // Optional, one-kernel path only (attention_fused_applies): a word, zero on entry, that receives
  // the float bits of the largest |output| as written (bf16-rounded), so that the quantiser for
  // the o projection needs no pass of its own over the rows to find it.
  unsigned int *amax_bits;
};

// Plain CUDA-core implementation of the three phases. It is the bring-up path and the on-device
// cross-check for the tensor-core kernels.
int launch_attention_simt(const AttentionArguments &arguments, cudaStream_t stream);

// Tensor-core implementation (tcgen05 + TMA): head_dim 256 or 512, capacity a multiple of 128,
// arguments.maps and arguments.stats set (and request_chunks when chunks > 1). Same rounding
// points. Chooses the one-kernel path when it applies, else the two-kernel path.
int launch_attention_tc(const AttentionArguments &arguments, cudaStream_t stream);

// Kernels launch_attention_tc launches for these arguments (the CUDA-core path launches three).
int attention_tc_launches(const AttentionArguments &arguments);

// Argument checks shared by both implementations (0 = fine).
int validate_attention(const AttentionArguments &arguments);

// Shared phase 2 (in-place softmax over the score buffer).
int launch_attention_softmax(const AttentionArguments &arguments, cudaStream_t stream);

// Number of cache-row chunks needed for `max_cache_rows` at `chunk_keys` rows per chunk.
inline int attention_chunks(int max_cache_rows, int chunk_keys) {
  const int chunks = (max_cache_rows + chunk_keys - 1) / chunk_keys;
  return chunks < 1 ? 1 : chunks;
}

} // namespace carat_b200
