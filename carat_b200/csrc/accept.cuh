// Greedy prefix-accept, hidden-state hand-off and KV commit / rollback kernels: the bookkeeping
// the reference does on the host after a device-to-host copy of the target predictions
// (cuda/batch_model_runner.cu:1730-1808) stays on the device here.
#pragma once

#include <cuda_runtime.h>

namespace carat_b200 {

struct AcceptArguments {
  const unsigned long long *best;  // [requests * depth] packed argmax keys of the LM head
  const int *proposals;            // [requests * depth]
  const int *target_first;         // [requests]
  const int *caps;                 // [requests] or null (= depth)
  int assume_match;                // 1: every proposal counts as matching (cap alone decides)
  int *accepted;                   // out [requests]
  int *next_tokens;                // out [requests]
  int *predictions;                // out [requests * depth] target argmax per row
  const void *final_hidden;        // [requests * depth, hidden] bf16, final-normed rows
  void *hidden_by_slot;            // [slots, hidden] bf16; row (accepted - 1) lands in slots[r]
  const int *slots;                // [requests]
  int requests;
  int depth;
  int hidden;
};

// accepted = longest prefix with proposal[i] == (i == 0 ? target_first : prediction[i-1]), capped;
// next = accepted == 0 ? target_first : prediction[accepted-1]
// (cuda/batch_model_runner.cu:1735-1759); then the hand-off of :1761-1783. The position update
// of :1805-1807 stays on the host, which owns the slot positions.
int launch_accept(const AcceptArguments &arguments, cudaStream_t stream);

// One sliding layer's share of the commit: proposal rows t < accepted[r] move from the staging
// area [requests, kv_heads, depth, head_dim] into ring row (position + t) % capacity of slot
// slots[r]; rows t >= accepted[r] never touch the ring, which is the visible state the
// reference reaches by backup + restore (cuda/ops.cu:827-871).
struct CommitLayer {
  void *key_cache;
  void *value_cache;
  const void *staged_keys;
  const void *staged_values;
  long long slot_stride;   // elements
  long long head_stride;   // elements
  int kv_heads;
  int head_dim;
  int capacity;
  int pad;
};

int launch_commit(const CommitLayer *device_layers, int layers, const int *positions,
                  const int *accepted, const int *slots, int requests, int depth,
                  int max_row_elements, cudaStream_t stream);

// Stand-alone forms of the reference's rollback primitives
// (include/carat/cuda_ops.h backup_kv_ring_spans_bf16 / restore_kv_ring_suffixes_bf16).
int launch_backup_kv_ring_spans(const void *const *key_sources, const void *const *value_sources,
                                void *backup_keys, void *backup_values, const int *positions,
                                int requests, int heads, int tokens, int head_dim, int capacity,
                                cudaStream_t stream);
int launch_restore_kv_ring_suffixes(const void *backup_keys, const void *backup_values,
                                    void *const *key_destinations,
                                    void *const *value_destinations, const int *positions,
                                    const int *accepted, int requests, int heads, int tokens,
                                    int head_dim, int capacity, cudaStream_t stream);

// Plain argmax over bf16 rows with ties to the lowest index (cuda/ops.cu:890-981).
int launch_argmax_bf16_rows(const void *values, int rows, int elements, int *output,
                            cudaStream_t stream);

// output[r, :] = input[indices[r], :] and output[indices[r], :] = input[r, :]
// (cuda/ops.cu gather_rows / scatter_rows).
int launch_gather_rows(const void *input, const int *indices, void *output, int rows, int width,
                       cudaStream_t stream);
int launch_scatter_rows(const void *input, const int *indices, void *output, int rows, int width,
                        cudaStream_t stream);

} // namespace carat_b200
