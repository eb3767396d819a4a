// Work-item bookkeeping shared by the weight-streaming linears (e4m3 and int4 weights): kernel
// arguments, the (feature tile, K piece) item list a persistent CTA walks, and the host-side
// schedule that picks split-K factors and the K-cut tail round.
#pragma once

#include "context.cuh"
#include "fp8_linear.cuh"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace carat_b200 {

constexpr int tile_features = 128;    // UMMA M: output features per tile
constexpr int tile_k_elements = 128;  // K bytes per block of the item list (one swizzle atom)

struct KernelArguments {
  const float *input_scale;
  const float *weight_scale;
  __nv_bfloat16 *output;
  float *partial;             // mode 1: [splits, rows, output_width]
  unsigned long long *best;   // mode 2
  int *device_error;
  int rows;
  int output_width;
  int tiles;
  int k_blocks;
  int splits;                 // K pieces per tile (1 unless mode 1)
  int k_blocks_per_split;
  // Mode 0 only: the last `tail_tiles` feature tiles are cut into `tail_splits` K pieces whose
  // fp32 partial sums go to tail_partial [piece, rows, tail_tiles * 128] instead of `output`.
  float *tail_partial;
  int tail_tiles;
  int tail_splits;
  int tail_k_blocks_per_split;
  // Mode 3 (gated): a tile is 64 gate features and the 64 up features that go with them; the
  // epilogue writes bf16(gelu(gate) * up) [rows, gated_width] to `output` and folds the largest
  // magnitude into `amax_bits`. K-cut tail tiles leave their pieces in tail_partial; after a
  // grid-wide barrier (grid_counter, zero between launches) all CTAs share the work of summing
  // and finishing them. With fp8_output set, a second barrier makes the maximum final and the
  // CTAs quantise the rows: scale = max / 448 to scale_out, e4m3 rows to fp8_output.
  unsigned int *amax_bits;
  unsigned int *grid_counter;
  unsigned char *fp8_output;
  float *scale_out;
  int gated_width;
};

struct WorkItem {
  int tile;
  int piece;
  int k_begin;
  int k_count;
  bool tail;
};

// Items are numbered piece-major so that the pieces of one tile land on different CTAs; the whole
// tiles come first and the pieces of the tail tiles last, so they fill the last partial round.
__device__ __forceinline__ WorkItem decode_item(const KernelArguments &args, int index) {
  WorkItem item;
  const int whole_items = (args.tiles - args.tail_tiles) * args.splits;
  if (index < whole_items) {
    const int whole_tiles = args.tiles - args.tail_tiles;
    item.tile = index % whole_tiles;
    item.piece = index / whole_tiles;
    item.k_begin = item.piece * args.k_blocks_per_split;
    item.k_count = min(args.k_blocks, item.k_begin + args.k_blocks_per_split) - item.k_begin;
    item.tail = false;
  } else {
    const int tail_index = index - whole_items;
    item.tile = args.tiles - args.tail_tiles + tail_index % args.tail_tiles;
    item.piece = tail_index / args.tail_tiles;
    item.k_begin = item.piece * args.tail_k_blocks_per_split;
    item.k_count = min(args.k_blocks, item.k_begin + args.tail_k_blocks_per_split) - item.k_begin;
    item.tail = true;
  }
  return item;
}

__device__ __forceinline__ int item_count(const KernelArguments &args) {
  return (args.tiles - args.tail_tiles) * args.splits + args.tail_tiles * args.tail_splits;
}

using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                 const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                 const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiled encode_tiled_entry() {
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

inline void schedule_linear(LinearPlan *plan, int rows, int input_width, int output_width,
                     int requested_splits, int element_bytes = 1) {
  LinearPlan &result = *plan;
  result.rows = rows;
  result.input_width = input_width;
  result.output_width = output_width;
  result.element_bytes = element_bytes;
  result.padded_rows = rows <= 32 ? 32 : rows <= 64 ? 64 : rows <= 128 ? 128 : rows <= 192 ? 192 : 256;
  result.tiles = (output_width + tile_features - 1) / tile_features;
  result.k_blocks = (input_width * element_bytes + tile_k_elements - 1) / tile_k_elements;
  result.ctas = device_multiprocessors();
  int splits = requested_splits;
  if (splits <= 0) {
    // Fewer tiles than SMs: cut K so that most SMs stream; keep at least four K blocks a piece.
    splits = result.tiles >= result.ctas ? 1 : result.ctas / result.tiles;
    const int most = result.k_blocks / 4 < 1 ? 1 : result.k_blocks / 4;
    splits = splits > most ? most : splits;
  }
  if (splits > result.k_blocks)
    splits = result.k_blocks;
  result.k_blocks_per_split = (result.k_blocks + splits - 1) / splits;
  result.splits = (result.k_blocks + result.k_blocks_per_split - 1) / result.k_blocks_per_split;
  // More tiles than SMs with a short last round: cutting the last round's tiles along K lets every
  // SM take part in it (336 tiles on 148 SMs: 2 + 1/3 rounds instead of 3).
  result.tail_tiles = 0;
  result.tail_splits = 1;
  result.tail_k_blocks_per_split = result.k_blocks;
  const int remainder = result.tiles % result.ctas;
  if (result.splits == 1 && result.tiles > result.ctas && remainder > 0 &&
      remainder * 2 <= result.ctas && output_width % tile_features == 0) {
    int pieces = result.ctas / remainder;
    const int most = result.k_blocks / 4 < 1 ? 1 : result.k_blocks / 4;
    pieces = pieces > most ? most : pieces;
    if (pieces > 1) {
      result.tail_tiles = remainder;
      result.tail_k_blocks_per_split = (result.k_blocks + pieces - 1) / pieces;
      result.tail_splits = (result.k_blocks + result.tail_k_blocks_per_split - 1) /
                           result.tail_k_blocks_per_split;
    }
  }
}

} // namespace carat_b200
