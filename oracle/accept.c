/* Plain-C restatement of the integer bookkeeping on the speculative-decoding path.
 * TEST INFRASTRUCTURE: only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may
 * load this; the product library never links or calls it.
 *
 * Each function cites the reference code it follows (paths inside the Gradiated/carat tree).
 * Pinned against the reference's known-answer tests (tests/speculation_tests.cpp:15-60,
 * tests/cuda_ops_tests.cu:1137-1164) and against the reference's own speculation.cpp compiled into
 * oracle/_ref (see oracle/Makefile). */
#include <stdint.h>
#include <string.h>

static int contains(const int *set, int count, int value) {
  for (int index = 0; index < count; ++index)
    if (set[index] == value)
      return 1;
  return 0;
}

/* src/runtime/speculation.cpp:7-18 */
int oracle_acceptance_cap(int depth, int remaining, const int *proposals, int proposal_count,
                          const int *stop_ids, int stop_count) {
  const int cap = depth < remaining ? depth : remaining;
  const int inspected = cap < proposal_count ? cap : proposal_count;
  for (int index = 1; index < inspected; ++index)
    if (contains(stop_ids, stop_count, proposals[index]))
      return index + 1;
  return cap;
}

/* src/runtime/speculation.cpp:20-36. resident/emitted must hold accepted_count + 1 entries.
 * Returns 1 when an accepted draft was a stop token. */
int oracle_commit_speculation(int forced_token, const int *accepted_drafts, int accepted_count,
                              int next_token, const int *stop_ids, int stop_count, int *resident,
                              int *resident_count, int *emitted, int *emitted_count) {
  int residents = 0, emits = 0;
  resident[residents++] = forced_token;
  for (int index = 0; index < accepted_count; ++index) {
    resident[residents++] = accepted_drafts[index];
    emitted[emits++] = accepted_drafts[index];
    if (contains(stop_ids, stop_count, accepted_drafts[index])) {
      *resident_count = residents;
      *emitted_count = emits;
      return 1;
    }
  }
  emitted[emits++] = next_token;
  *resident_count = residents;
  *emitted_count = emits;
  return 0;
}

/* cuda/batch_model_runner.cu:1735-1759. proposals and predictions are [requests][depth];
 * caps may be NULL (= depth). assume_match is not in the reference: it makes the cap alone decide
 * the accepted length (used to inject accept lengths in throughput runs). */
void oracle_greedy_prefix_accept(const int *proposals, const int *target_first,
                                 const int *predictions, const int *caps, int requests, int depth,
                                 int assume_match, int *accepted_tokens, int *next_tokens) {
  for (int request = 0; request < requests; ++request) {
    int cap = depth;
    if (caps != 0) {
      cap = caps[request] < 0 ? 0 : caps[request];
      cap = cap > depth ? depth : cap;
    }
    const int start = request * depth;
    int accepted = 0;
    while (accepted < cap) {
      const int expected =
          accepted == 0 ? target_first[request] : predictions[start + accepted - 1];
      if (!assume_match && proposals[start + accepted] != expected)
        break;
      ++accepted;
    }
    accepted_tokens[request] = accepted;
    next_tokens[request] =
        accepted == 0 ? target_first[request] : predictions[start + accepted - 1];
  }
}

static float bf16_to_float(uint16_t bits) {
  const uint32_t wide = (uint32_t)bits << 16;
  float value;
  memcpy(&value, &wide, sizeof(value));
  return value;
}

/* cuda/ops.cu:890-981: row argmax over bf16 values, ties to the lowest index, NaN never chosen. */
void oracle_argmax_bf16_rows(const uint16_t *values, int rows, int elements, int *output) {
  for (int row = 0; row < rows; ++row) {
    float best = -__builtin_inff();
    int best_index = 0;
    const uint16_t *line = values + (size_t)row * elements;
    for (int index = 0; index < elements; ++index) {
      const float value = bf16_to_float(line[index]);
      if (value > best) {
        best = value;
        best_index = index;
      }
    }
    output[row] = best_index;
  }
}

/* cuda/ops.cu:827-847: backup[req][head][t][:] = cache[req][head][(pos + t) % capacity][:]. */
void oracle_backup_kv_ring_spans(const uint16_t *const *keys, const uint16_t *const *values,
                                 uint16_t *backup_keys, uint16_t *backup_values,
                                 const int *positions, int requests, int heads, int tokens,
                                 int dimension, int capacity) {
  for (int request = 0; request < requests; ++request)
    for (int head = 0; head < heads; ++head)
      for (int token = 0; token < tokens; ++token) {
        const size_t source =
            ((size_t)head * capacity + (size_t)((positions[request] + token) % capacity)) *
            dimension;
        const size_t destination =
            (((size_t)request * heads + head) * tokens + token) * dimension;
        memcpy(backup_keys + destination, keys[request] + source, 2 * (size_t)dimension);
        memcpy(backup_values + destination, values[request] + source, 2 * (size_t)dimension);
      }
}

/* cuda/ops.cu:849-871: rows token >= accepted[req] are written back from the backup. */
void oracle_restore_kv_ring_suffixes(const uint16_t *backup_keys, const uint16_t *backup_values,
                                     uint16_t *const *keys, uint16_t *const *values,
                                     const int *positions, const int *accepted, int requests,
                                     int heads, int tokens, int dimension, int capacity) {
  for (int request = 0; request < requests; ++request)
    for (int head = 0; head < heads; ++head)
      for (int token = accepted[request] < 0 ? 0 : accepted[request]; token < tokens; ++token) {
        const size_t destination =
            ((size_t)head * capacity + (size_t)((positions[request] + token) % capacity)) *
            dimension;
        const size_t source = (((size_t)request * heads + head) * tokens + token) * dimension;
        memcpy(keys[request] + destination, backup_keys + source, 2 * (size_t)dimension);
        memcpy(values[request] + destination, backup_values + source, 2 * (size_t)dimension);
      }
}
