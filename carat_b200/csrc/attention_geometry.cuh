// Column layout of the bf16 score buffer, shared by every attention kernel.
//
// One score row per (request, query head, proposal t). Its columns are
//   [0, 16)                proposal rows u = column (only u < proposals is meaningful), and
//   [16, 16 + cache_rows)  cache rows r = column - 16 in physical order.
// Keeping the proposals in front makes every 128-row cache tile start at a column that is a
// multiple of 8 elements, which a TMA tile load needs (16-byte aligned innermost coordinate).
//
//   sliding ring : cache_rows = min(position, capacity), proposals = depth (staged on the side)
//   global cache : cache_rows = position + depth, proposals = 0 (proposals were written in place)
//   drafter      : cache_rows = min(position + 1, capacity), proposals = 0, everything visible
#pragma once

#include "attention.cuh"

namespace carat_b200 {

constexpr int proposal_columns = 16;

struct KeyGeometry {
  int cache_rows;
  int proposals;
  __host__ __device__ int columns() const { return proposal_columns + cache_rows; }
};

__host__ __device__ inline KeyGeometry key_geometry(int position, int depth, int capacity,
                                                    int window, bool staged, bool draft) {
  KeyGeometry g;
  if (draft) {
    g.cache_rows = position + 1 < capacity ? position + 1 : capacity;
    g.proposals = 0;
  } else if (staged) {
    g.cache_rows = position < capacity ? position : capacity;
    g.proposals = depth;
  } else {
    g.cache_rows = position + depth;
    g.proposals = 0;
  }
  (void)window;
  return g;
}

#ifdef __CUDACC__
__device__ __forceinline__ KeyGeometry key_geometry(const AttentionArguments &a, int request) {
  return key_geometry(a.positions[request], a.depth, a.capacity, a.window, a.new_keys != nullptr,
                      a.draft != 0);
}

#endif

// Columns a launch has to cover for contexts up to `max_cache_rows`, rounded to whole 128-row
// cache tiles so that padding columns exist (and are zeroed by the softmax).
__host__ __device__ inline int score_columns(int max_cache_rows) {
  return proposal_columns + (max_cache_rows + 127) / 128 * 128;
}

} // namespace carat_b200
