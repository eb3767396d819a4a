// C entry points for the row operators, attention-side operators and bookkeeping kernels
// (declared in include/carat_b200.h).
#include "../../include/carat_b200.h"
#include "accept.cuh"
#include "attention.cuh"
#include "attention_tc.cuh"
#include "context.cuh"
#include "qkv_post.cuh"
#include "row_ops.cuh"

#include <string>

using namespace carat_b200;

namespace {

int finish(int status, const char *what) {
  if (status == 0)
    return 0;
  const cudaError_t last = cudaGetLastError();
  if (status == -1) {
    set_last_error(std::string("invalid ") + what + " arguments");
  } else if (status == -2) {
    set_last_error(std::string(what) + " shape exceeds what one launch supports");
  } else if (status == -3) {
    set_last_error(std::string(what) + ": unsupported head dimension");
  } else {
    set_last_error(std::string(what) + " launch failed: " + cudaGetErrorString(last));
  }
  return status;
}

// Clears the caller's scratch word on the stream, then hands out the quantisation target.
int prepare_target(QuantTarget *target, void *fp8_output, float *scale, void *scratch,
                   cudaStream_t stream) {
  if (fp8_output == nullptr || scale == nullptr || scratch == nullptr) {
    set_last_error("invalid FP8 quantization shape");
    return -1;
  }
  const int status =
      check_cuda(cudaMemsetAsync(scratch, 0, sizeof(unsigned int), stream), "clear FP8 amax");
  if (status != 0)
    return status;
  *target = QuantTarget{fp8_output, scale, static_cast<unsigned int *>(scratch)};
  return 0;
}

} // namespace

extern "C" int carat_b200_quantize_bf16_to_fp8(const void *bf16_input, void *fp8_output,
                                               float *device_scale, void *device_scratch,
                                               int rows, int width, void *stream) {
  const auto cuda_stream = static_cast<cudaStream_t>(stream);
  QuantTarget target{};
  const int status = prepare_target(&target, fp8_output, device_scale, device_scratch, cuda_stream);
  if (status != 0)
    return status;
  return finish(launch_quant(bf16_input, nullptr, 0, nullptr, 1, target, rows, width, cuda_stream),
                "FP8 quantization");
}

extern "C" int carat_b200_quantize_bf16_to_fp8_from_amax(const void *bf16_input,
                                                         const unsigned int *device_amax_bits,
                                                         void *fp8_output, float *device_scale,
                                                         size_t elements, void *stream) {
  if (bf16_input == nullptr || device_amax_bits == nullptr || fp8_output == nullptr ||
      device_scale == nullptr || elements == 0 || elements % 8 != 0) {
    set_last_error("invalid FP8 quantization shape");
    return -1;
  }
  QuantTarget target{};
  target.fp8_output = fp8_output;
  target.scale = device_scale;
  target.amax_bits = const_cast<unsigned int *>(device_amax_bits);
  return finish(launch_quantize_rows(bf16_input, target, elements,
                                     static_cast<cudaStream_t>(stream)),
                "FP8 quantization");
}

extern "C" int carat_b200_quantize_bf16_tensor_to_fp8(const void *bf16_input, void *fp8_output,
                                                      float *device_scale, void *device_scratch,
                                                      size_t elements, void *stream) {
  const auto cuda_stream = static_cast<cudaStream_t>(stream);
  QuantTarget target{};
  const int status = prepare_target(&target, fp8_output, device_scale, device_scratch, cuda_stream);
  if (status != 0)
    return status;
  return finish(launch_quant_tensor(bf16_input, fp8_output, device_scale, target.amax_bits,
                                    elements, cuda_stream),
                "FP8 quantization");
}

extern "C" int carat_b200_rms_norm_quantize(const void *bf16_input, const void *bf16_weight,
                                            void *bf16_normalized, void *fp8_output,
                                            float *device_scale, void *device_scratch, int rows,
                                            int width, float epsilon, void *stream) {
  const auto cuda_stream = static_cast<cudaStream_t>(stream);
  QuantTarget target{};
  const int status = prepare_target(&target, fp8_output, device_scale, device_scratch, cuda_stream);
  if (status != 0)
    return status;
  return finish(launch_norm_quant(bf16_input, bf16_weight, bf16_normalized, target, rows, width,
                                  epsilon, cuda_stream),
                "RMSNorm quantization");
}

extern "C" int carat_b200_rms_norm_add_and_norm_quantize(
    const void *bf16_input, const void *bf16_weight, const void *bf16_residual,
    const void *bf16_next_weight, void *bf16_first, void *fp8_output, float *device_scale,
    void *device_scratch, int rows, int width, float epsilon, void *stream) {
  const auto cuda_stream = static_cast<cudaStream_t>(stream);
  QuantTarget target{};
  const int status = prepare_target(&target, fp8_output, device_scale, device_scratch, cuda_stream);
  if (status != 0)
    return status;
  return finish(launch_post_attention_norms_quant(bf16_input, PartialSource{}, bf16_weight,
                                                  bf16_residual, bf16_next_weight, bf16_first,
                                                  target, rows, width, epsilon, cuda_stream),
                "RMSNorm add-and-norm quantization");
}

extern "C" int carat_b200_gelu_gate_quantize(const void *bf16_packed_gate_up, void *fp8_output,
                                             float *device_scale, void *device_scratch, int rows,
                                             int width, void *stream) {
  const auto cuda_stream = static_cast<cudaStream_t>(stream);
  QuantTarget target{};
  const int status = prepare_target(&target, fp8_output, device_scale, device_scratch, cuda_stream);
  if (status != 0)
    return status;
  return finish(launch_geglu_quant(bf16_packed_gate_up, TailSource{}, target, rows, width, cuda_stream),
                "GeGLU quantization");
}

extern "C" int carat_b200_rms_norm_add_scale_then_norm_quantize(
    const void *bf16_input, const void *bf16_weight, const void *bf16_residual,
    const void *bf16_scalar, void *bf16_output, const void *bf16_next_weight, void *bf16_next,
    void *fp8_output, float *device_scale, void *device_scratch, int rows, int width,
    float epsilon, void *stream) {
  const auto cuda_stream = static_cast<cudaStream_t>(stream);
  QuantTarget target{};
  const int status = prepare_target(&target, fp8_output, device_scale, device_scratch, cuda_stream);
  if (status != 0)
    return status;
  return finish(launch_layer_output_norm_quant(bf16_input, PartialSource{}, bf16_weight,
                                               bf16_residual, bf16_scalar, bf16_output,
                                               bf16_next_weight, bf16_next, target, rows, width,
                                               epsilon, cuda_stream),
                "layer output quantization");
}

extern "C" int carat_b200_rope_tables(void *bf16_cosine, void *bf16_sine, int positions,
                                      int head_dim, float theta, int proportional, void *stream) {
  return finish(launch_rope_tables(bf16_cosine, bf16_sine, positions, head_dim, theta,
                                   proportional != 0, static_cast<cudaStream_t>(stream)),
                "RoPE table");
}

extern "C" int carat_b200_qkv_postprocess(const void *bf16_packed, const void *bf16_query_norm,
                                          const void *bf16_key_norm, const void *bf16_cosine,
                                          const void *bf16_sine, void *bf16_queries,
                                          void *bf16_keys, void *bf16_values,
                                          const int *device_positions, int requests, int depth,
                                          int query_heads, int kv_heads, int head_dim,
                                          int key_equals_value, int table_positions, float epsilon,
                                          void *stream) {
  QkvPostArguments a{};
  a.packed = bf16_packed;
  a.query_norm = bf16_query_norm;
  a.key_norm = bf16_key_norm;
  a.cosine = bf16_cosine;
  a.sine = bf16_sine;
  a.queries = bf16_queries;
  a.key_base = bf16_keys;
  a.value_base = bf16_values;
  a.head_stride = static_cast<long long>(depth) * head_dim;
  a.slot_stride = a.head_stride * kv_heads;
  a.positions = device_positions;
  a.direct = 0;
  a.capacity = depth > 0 ? depth : 1;
  a.requests = requests;
  a.depth = depth;
  a.query_heads = query_heads;
  a.kv_heads = kv_heads;
  a.head_dim = head_dim;
  a.key_equals_value = key_equals_value;
  a.max_positions = table_positions;
  a.epsilon = epsilon;
  return finish(launch_qkv_post(a, static_cast<cudaStream_t>(stream)), "QKV post-processing");
}

namespace {
__global__ void identity_slots_kernel(int *slots, int count) {
  const int index = static_cast<int>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (index < count)
    slots[index] = index;
}
} // namespace

namespace {

// Scratch the op-level attention entry points keep for the library's life, one set per device.
struct AttentionScratch {
  int *identity_slots = nullptr;     // [1024]: request r owns cache r
  float2 *stats = nullptr;           // one (maximum, sum) pair per score row and chunk
  long long stats_rows = 0;
  float *partials = nullptr;         // chunk partial outputs of long linear caches
  size_t partial_bytes = 0;
  int *request_chunks = nullptr;     // [1024]: chunk counts of the last chunked call
};
PerDevice<AttentionScratch> attention_scratch;

int run_verify_attention(bool tensor_cores, const void *bf16_queries, const void *bf16_key_caches,
                         const void *bf16_value_caches, const void *bf16_new_keys,
                         const void *bf16_new_values, const int *device_positions,
                         void *bf16_output, void *bf16_scores, int score_stride, int requests,
                         int depth, int query_heads, int kv_heads, int head_dim, int capacity,
                         int window, int max_position, void *stream) {
  if (requests <= 0 || requests > 1024 || kv_heads <= 0 || query_heads <= 0 || depth <= 0 ||
      (window > 0 && (bf16_new_keys == nullptr || bf16_new_values == nullptr))) {
    set_last_error("invalid verify attention arguments");
    return -1;
  }
  const auto cuda_stream = static_cast<cudaStream_t>(stream);
  AttentionScratch *scratch_slot = attention_scratch.slot();
  if (scratch_slot == nullptr) {
    set_last_error("verify attention: no current device");
    return -100;
  }
  std::lock_guard<std::mutex> scratch_lock(attention_scratch.lock());
  int *&identity_slots = scratch_slot->identity_slots;
  if (identity_slots == nullptr) {
    if (check_cuda(cudaMalloc(&identity_slots, sizeof(int) * 1024), "allocate slot table") != 0)
      return -100;
    identity_slots_kernel<<<4, 256, 0, cuda_stream>>>(identity_slots, 1024);
  }
  AttentionArguments a{};
  a.queries = bf16_queries;
  a.key_cache = bf16_key_caches;
  a.value_cache = bf16_value_caches;
  a.head_stride = static_cast<long long>(capacity) * head_dim;
  a.slot_stride = a.head_stride * kv_heads;
  a.new_keys = bf16_new_keys;
  a.new_values = bf16_new_values;
  a.new_head_stride = static_cast<long long>(depth) * head_dim;
  a.new_request_stride = a.new_head_stride * kv_heads;
  a.positions = device_positions;
  a.slots = identity_slots;
  a.scores = bf16_scores;
  a.score_stride = score_stride;
  a.output = bf16_output;
  a.chunks = 1;
  a.requests = requests;
  a.depth = depth;
  a.query_heads = query_heads;
  a.kv_heads = kv_heads;
  a.head_dim = head_dim;
  a.capacity = capacity;
  a.window = window;
  const bool staged = bf16_new_keys != nullptr;
  a.max_cache_rows = staged ? (max_position < capacity ? max_position : capacity)
                            : max_position + depth;
  a.chunk_keys = (a.max_cache_rows + 127) / 128 * 128;
  if (a.chunk_keys == 0)
    a.chunk_keys = 128;
  AttentionMaps maps;
  if (tensor_cores && (head_dim == 256 || head_dim == 512) && capacity % 128 == 0) {
    const int padded = attention_padded_rows(query_heads / kv_heads * depth);
    const long long score_rows = static_cast<long long>(requests) * query_heads * depth;
    const int status = make_attention_maps(
        &maps, bf16_key_caches, bf16_value_caches,
        static_cast<long long>(requests) * kv_heads * capacity, bf16_new_keys, bf16_new_values,
        static_cast<long long>(requests) * kv_heads * depth, bf16_queries, score_rows, bf16_scores,
        score_rows, score_stride, head_dim, padded);
    if (status != 0) {
      set_last_error("verify attention: tensor map encoding failed");
      return status;
    }
    // One (maximum, sum) pair per score row: scratch of the two-kernel path, kept for the
    // library's life and grown when a call needs more (cudaFree waits for the device first).
    float2 *&stats = scratch_slot->stats;
    long long &stats_rows = scratch_slot->stats_rows;
    float *&partials = scratch_slot->partials;
    size_t &partial_bytes = scratch_slot->partial_bytes;
    int *&request_chunks = scratch_slot->request_chunks;
    if (request_chunks == nullptr &&
        check_cuda(cudaMalloc(&request_chunks, sizeof(int) * 1024), "allocate chunk counts") != 0)
      return -100;
    a.request_chunks = request_chunks;
    constexpr int long_chunk_keys = 1024;
    if (!staged && a.max_cache_rows > long_chunk_keys) {
      // Long linear caches are cut into chunks like the runner does; the chunk partials live in
      // library scratch and are summed into the caller's output.
      a.chunk_keys = long_chunk_keys;
      a.chunks = attention_chunks(a.max_cache_rows, long_chunk_keys);
      a.sum_chunks = 1;
      const size_t need = sizeof(float) * static_cast<size_t>(a.chunks) * requests * depth *
                          query_heads * head_dim;
      if (need > partial_bytes) {
        if (partials != nullptr)
          cudaFree(partials);
        partials = nullptr;
        partial_bytes = 0;
        if (check_cuda(cudaMalloc(&partials, need), "allocate attention chunk partials") != 0)
          return -100;
        partial_bytes = need;
      }
      a.chunk_partials = partials;
    }
    const long long stats_need = score_rows * a.chunks;
    if (stats_need > stats_rows) {
      if (stats != nullptr)
        cudaFree(stats);
      stats = nullptr;
      stats_rows = 0;
      if (check_cuda(cudaMalloc(&stats, sizeof(float2) * static_cast<size_t>(stats_need)),
                     "allocate attention statistics") != 0)
        return -100;
      stats_rows = stats_need;
    }
    a.stats = stats;
    a.stats_stride = a.chunks;
    a.maps = &maps;
    return finish(launch_attention_tc(a, cuda_stream), "verify attention");
  }
  return finish(launch_attention_simt(a, cuda_stream), "verify attention");
}

} // namespace

extern "C" int carat_b200_verify_attention(const void *bf16_queries, const void *bf16_key_caches,
                                           const void *bf16_value_caches,
                                           const void *bf16_new_keys, const void *bf16_new_values,
                                           const int *device_positions, void *bf16_output,
                                           void *bf16_scores, int score_stride, int requests,
                                           int depth, int query_heads, int kv_heads, int head_dim,
                                           int capacity, int window, int max_position,
                                           void *stream) {
  return run_verify_attention(true, bf16_queries, bf16_key_caches, bf16_value_caches,
                              bf16_new_keys, bf16_new_values, device_positions, bf16_output,
                              bf16_scores, score_stride, requests, depth, query_heads, kv_heads,
                              head_dim, capacity, window, max_position, stream);
}

extern "C" int carat_b200_verify_attention_check(
    const void *bf16_queries, const void *bf16_key_caches, const void *bf16_value_caches,
    const void *bf16_new_keys, const void *bf16_new_values, const int *device_positions,
    void *bf16_output, void *bf16_scores, int score_stride, int requests, int depth,
    int query_heads, int kv_heads, int head_dim, int capacity, int window, int max_position,
    void *stream) {
  return run_verify_attention(false, bf16_queries, bf16_key_caches, bf16_value_caches,
                              bf16_new_keys, bf16_new_values, device_positions, bf16_output,
                              bf16_scores, score_stride, requests, depth, query_heads, kv_heads,
                              head_dim, capacity, window, max_position, stream);
}

extern "C" int carat_b200_backup_kv_ring_spans(const void *const *device_key_sources,
                                               const void *const *device_value_sources,
                                               void *backup_keys, void *backup_values,
                                               const int *device_position_starts, int requests,
                                               int heads, int tokens, int head_dim,
                                               int source_capacity, void *stream) {
  return finish(launch_backup_kv_ring_spans(device_key_sources, device_value_sources, backup_keys,
                                            backup_values, device_position_starts, requests, heads,
                                            tokens, head_dim, source_capacity,
                                            static_cast<cudaStream_t>(stream)),
                "KV ring backup");
}

extern "C" int carat_b200_restore_kv_ring_suffixes(
    const void *backup_keys, const void *backup_values, void *const *device_key_destinations,
    void *const *device_value_destinations, const int *device_position_starts,
    const int *device_accepted_tokens, int requests, int heads, int tokens, int head_dim,
    int destination_capacity, void *stream) {
  return finish(launch_restore_kv_ring_suffixes(
                    backup_keys, backup_values, device_key_destinations, device_value_destinations,
                    device_position_starts, device_accepted_tokens, requests, heads, tokens,
                    head_dim, destination_capacity, static_cast<cudaStream_t>(stream)),
                "KV ring restore");
}

extern "C" int carat_b200_argmax_bf16_rows(const void *bf16_values, int rows, int elements,
                                           int *device_output, void *stream) {
  return finish(launch_argmax_bf16_rows(bf16_values, rows, elements, device_output,
                                        static_cast<cudaStream_t>(stream)),
                "argmax");
}

namespace {
__global__ void accept_only_kernel(const int *proposals, const int *target_first,
                                   const int *predictions, const int *caps, int requests,
                                   int depth, int *accepted_tokens, int *next_tokens) {
  const int request = static_cast<int>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (request >= requests)
    return;
  int cap = depth;
  if (caps != nullptr)
    cap = min(max(caps[request], 0), depth);
  const int start = request * depth;
  int accepted = 0;
  while (accepted < cap) {
    const int expected = accepted == 0 ? target_first[request] : predictions[start + accepted - 1];
    if (proposals[start + accepted] != expected)
      break;
    ++accepted;
  }
  accepted_tokens[request] = accepted;
  next_tokens[request] = accepted == 0 ? target_first[request] : predictions[start + accepted - 1];
}
} // namespace

extern "C" int carat_b200_greedy_prefix_accept(const int *device_proposals,
                                               const int *device_target_first,
                                               const int *device_predictions,
                                               const int *device_caps, int requests, int depth,
                                               int *device_accepted, int *device_next_tokens,
                                               void *stream) {
  if (device_proposals == nullptr || device_target_first == nullptr ||
      device_predictions == nullptr || device_accepted == nullptr ||
      device_next_tokens == nullptr || requests <= 0 || depth <= 0) {
    set_last_error("invalid greedy verification batch");
    return -1;
  }
  accept_only_kernel<<<(requests + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      device_proposals, device_target_first, device_predictions, device_caps, requests, depth,
      device_accepted, device_next_tokens);
  return finish(cudaPeekAtLastError() == cudaSuccess ? 0 : -11, "greedy prefix accept");
}
