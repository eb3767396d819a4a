// The batch runner: request slots, KV arenas and the verify / draft steps, i.e. the part of
// carat::Gemma4BatchModelRunner and carat::Gemma4AssistantRunner that the speculative-decoding
// loop calls (cuda/batch_model_runner.cu:1617-1836, cuda/assistant_runner.cu:218-338), exported as
// C entry points. Every per-step decision that the reference takes on the host after a
// device-to-host copy (accept lengths, hidden hand-off, rollback) runs on the device here; one
// host-to-device copy starts a step and one device-to-host copy ends it.
#include "../../include/carat_b200.h"
#include "accept.cuh"
#include "attention.cuh"
#include "attention_geometry.cuh"
#include "attention_tc.cuh"
#include "context.cuh"
#include "fp8_linear.cuh"
#include "int4_linear.cuh"
#include "qkv_post.cuh"
#include "row_ops.cuh"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

using namespace carat_b200;

namespace {

constexpr int maximum_depth = 9;       // k = 8 drafts + the forced token
constexpr int prefill_pieces = 64;     // (slot, eight-token piece) entries one prefill step takes
constexpr int maximum_rows = 256;      // rows one FP8 linear launch accepts (24 slots x depth 9 = 216)
constexpr int global_chunk_keys = 1024;

struct Failure {
  std::string message;
};

void require_cuda(cudaError_t result, const char *operation) {
  if (result != cudaSuccess)
    throw Failure{std::string(operation) + ": " + cudaGetErrorString(result)};
}

void require_launch(int status, const char *operation) {
  if (status != 0) {
    const cudaError_t last = cudaGetLastError();
    throw Failure{std::string(operation) + " failed (" + std::to_string(status) + "): " +
                  cudaGetErrorString(last)};
  }
}

class DeviceBuffer {
public:
  DeviceBuffer() = default;
  explicit DeviceBuffer(size_t bytes, bool zero = false) { allocate(bytes, zero); }
  DeviceBuffer(const DeviceBuffer &) = delete;
  DeviceBuffer &operator=(const DeviceBuffer &) = delete;
  DeviceBuffer(DeviceBuffer &&other) noexcept : pointer_(other.pointer_), bytes_(other.bytes_) {
    other.pointer_ = nullptr;
    other.bytes_ = 0;
  }
  ~DeviceBuffer() { cudaFree(pointer_); }
  void allocate(size_t bytes, bool zero = false) {
    bytes_ = bytes < 256 ? 256 : bytes;
    require_cuda(cudaMalloc(&pointer_, bytes_), "allocate runner memory");
    if (zero)
      require_cuda(cudaMemset(pointer_, 0, bytes_), "clear runner memory");
  }
  template <typename T = void> T *get() const { return static_cast<T *>(pointer_); }
  size_t bytes() const { return bytes_; }

private:
  void *pointer_{nullptr};
  size_t bytes_{0};
};

class PinnedBuffer {
public:
  PinnedBuffer() = default;
  PinnedBuffer(const PinnedBuffer &) = delete;
  PinnedBuffer &operator=(const PinnedBuffer &) = delete;
  ~PinnedBuffer() { cudaFreeHost(pointer_); }
  void allocate(size_t bytes) {
    require_cuda(cudaMallocHost(&pointer_, bytes), "allocate pinned mailbox");
  }
  template <typename T> T *get() const { return static_cast<T *>(pointer_); }

private:
  void *pointer_{nullptr};
};

struct LayerState {
  carat_b200_layer_shape shape{};
  carat_b200_layer_weights weights{};
  int capacity{0};
  int rope{0};  // index into Runner::rope_tables
  DeviceBuffer kv;        // K region then V region
  size_t value_offset{0}; // bytes
  long long slot_stride{0};
  long long head_stride{0};
  DeviceBuffer staged;    // sliding layers: proposal K then V, [requests, kv_heads, depth, D]
  size_t staged_value_offset{0};
  int query_width() const { return shape.query_heads * shape.head_dim; }
  int kv_width() const { return shape.kv_heads * shape.head_dim; }
  int packed_width() const { return query_width() + kv_width() * (shape.key_equals_value ? 1 : 2); }
  void *keys() const { return kv.get<unsigned char>(); }
  void *values() const { return kv.get<unsigned char>() + value_offset; }
  void *staged_keys() const { return staged.get<unsigned char>(); }
  void *staged_values() const { return staged.get<unsigned char>() + staged_value_offset; }
};

struct RopeTable {
  int head_dim;
  float theta;
  bool proportional;
  DeviceBuffer cosine;
  DeviceBuffer sine;
};

struct LayerPlans {
  LinearPlan qkv, o, gate_up, down;
  LinearPlan gate_up_gated;   // gate_up with GeGLU in its epilogue (Runner::fused_geglu)
  Int4LinearPlan gate_up_int4, down_int4;   // used instead when the INT4 MLP variant is on
};

struct StepPlans {
  std::vector<LayerPlans> layers;
  LinearPlan head;        // LM head (argmax epilogue)
  LinearPlan pre, post;   // drafter projections
};

} // namespace

struct carat_b200_runner {
  // ---- model
  carat_b200_model_config config{};
  std::vector<carat_b200_layer_shape> shapes;
  carat_b200_model_weights weights{};
  std::vector<LayerState> layers;
  std::vector<std::unique_ptr<RopeTable>> rope_tables;
  int batch{0};
  int maximum_context{0};
  int shared_sliding{-1};
  int shared_global{-1};
  // ---- assistant
  bool has_assistant{false};
  carat_b200_assistant_config assistant{};
  std::vector<int32_t> assistant_kinds;
  carat_b200_assistant_weights assistant_weights{};
  std::vector<carat_b200_layer_weights> assistant_layers;
  // ---- state
  std::vector<int> slot_positions;
  DeviceBuffer hidden_by_slot;
  cudaStream_t stream{nullptr};
  cudaEvent_t start_event{nullptr};
  cudaEvent_t stop_event{nullptr};
  float last_verify_ms{0.0F};
  float last_draft_ms{0.0F};
  int last_verify_launches{0};
  int last_draft_launches{0};
  int launches{0};
  int last_rows{0};
  std::vector<int> last_predictions;
  // ---- workspaces (target)
  DeviceBuffer hidden_a, hidden_b, residual, final_hidden;
  DeviceBuffer quantized;    // e4m3 activation feeding the next linear
  DeviceBuffer packed;       // QKV projection output
  DeviceBuffer queries;
  DeviceBuffer attention_out;
  DeviceBuffer attention_partials;
  DeviceBuffer scores;
  DeviceBuffer attention_stats;   // float2 [score rows, global chunks]
  DeviceBuffer request_chunks;    // int [batch]: chunks the last chunked attention wrote per request
  DeviceBuffer two_launch_rows;   // bf16 [maximum_rows, widest row]: row kernels with more rows than CTAs
  int stats_stride{0};
  DeviceBuffer projected;    // bf16 output of a linear that did not split K
  DeviceBuffer gate_up;
  DeviceBuffer split_partials;  // fp32 [splits, rows, width] left for a fused consumer
  DeviceBuffer scratch_words;  // [amax words | argmax keys]
  DeviceBuffer scales;
  DeviceBuffer step_inputs;    // tokens, positions, slots, target_first, caps
  DeviceBuffer step_results;   // accepted, next, predictions, error word
  DeviceBuffer commit_layers;
  int commit_layer_count{0};
  PinnedBuffer host_inputs;
  PinnedBuffer host_results;
  int amax_words{0};
  int score_stride_sliding{0};
  int score_stride_global{0};
  int *device_error{nullptr};
  std::map<int, StepPlans> verify_plans;
  // ---- INT4 weight-only MLP variant (off unless carat_b200_runner_use_int4_mlp was called)
  std::vector<carat_b200_int4_mlp_layer> int4_layers;
  int int4_group{0};
  DeviceBuffer pre_mlp;      // bf16 [rows, hidden]: input of the INT4 gate_up linear
  DeviceBuffer activated;    // bf16 [rows, intermediate]: input of the INT4 down linear
  DeviceBuffer gated_rows;   // bf16 [rows, intermediate]: GeGLU rows out of the gated gate_up linear
  DeviceBuffer grid_counter;   // barrier word of the gated linear; zero between launches
  bool fused_geglu{false};
  bool cooperative_rows{false};   // CARAT_B200_COOPERATIVE_ROWS=1: row kernels as cooperative launches
  bool early_keys{true};          // the one-kernel attention requests its first cache tiles before
                                  // the previous grid has finished (CARAT_B200_EARLY_KEYS=0: after)
  bool attention_amax{true};      // the one-kernel attention also finds the largest |output|, so
                                  // the quantiser after it is one pass without a grid barrier
                                  // (CARAT_B200_ATTENTION_AMAX=0: the row kernel finds it)
  DeviceBuffer unit_scale;   // one fp32 1.0: INT4 partial sums carry no tensor scales
  std::map<std::pair<int, int>, AttentionMaps> verify_maps;  // (layer, depth)
  std::map<int, AttentionMaps> draft_maps;                   // assistant layer
  // ---- workspaces (assistant)
  DeviceBuffer a_hidden_a, a_hidden_b, a_residual, a_final_hidden, a_quantized, a_projected,
      a_queries, a_attention_out, a_attention_partials, a_scores, a_linear_out, a_gate_up,
      a_previous_hidden, a_scratch_words, a_scales, a_tokens, a_proposals;
  int a_amax_words{0};
  std::map<int, StepPlans> draft_plans;
  // ---- BF16 prefill: the target's bf16 matrices, bf16 inputs of its linears, plans per row count
  std::vector<carat_b200_layer_bf16_weights> bf16_layers;
  DeviceBuffer p_normed, p_pre_mlp, p_activated;
  // Prefill steps may list a slot several times (consecutive eight-token pieces of one prompt),
  // so their per-request inputs are sized for prefill_pieces entries, not for the batch.
  DeviceBuffer p_step_inputs, p_request_chunks;
  PinnedBuffer p_host_inputs;
  std::map<std::pair<int, int>, AttentionMaps> direct_maps;   // sliding layers read as linear caches
  std::map<int, StepPlans> prefill_plans;
  // ---- drafter precision (CARAT_B200_ASSISTANT_FP8_*): bf16 matrices and their plans
  int assistant_mode{CARAT_B200_ASSISTANT_FP8_ALL};
  bool assistant_has_fp8{false};
  carat_b200_assistant_bf16_weights assistant_bf16{};
  std::vector<carat_b200_assistant_bf16_layer> assistant_bf16_layers;
  DeviceBuffer a_concat, a_normed, a_pre_mlp, a_activated;   // bf16 inputs of the bf16 linears
  std::map<int, StepPlans> draft_plans_bf16;

  ~carat_b200_runner() {
    if (start_event != nullptr)
      cudaEventDestroy(start_event);
    if (stop_event != nullptr)
      cudaEventDestroy(stop_event);
    if (stream != nullptr)
      cudaStreamDestroy(stream);
  }
};

namespace {

using Runner = carat_b200_runner;

LinearPlan plan_linear(const void *input, const void *weight, int rows, int in, int out,
                       int splits) {
  LinearPlan plan;
  const char *message = "invalid FP8 linear shape";
  if (make_linear_plan(&plan, input, weight, rows, in, out, splits, &message) != 0)
    throw Failure{message};
  return plan;
}

int find_rope(Runner &runner, int head_dim, float theta, bool proportional) {
  for (size_t index = 0; index < runner.rope_tables.size(); ++index) {
    const RopeTable &table = *runner.rope_tables[index];
    if (table.head_dim == head_dim && table.theta == theta && table.proportional == proportional)
      return static_cast<int>(index);
  }
  auto table = std::make_unique<RopeTable>();
  table->head_dim = head_dim;
  table->theta = theta;
  table->proportional = proportional;
  const size_t bytes = static_cast<size_t>(runner.maximum_context) * head_dim * 2;
  table->cosine.allocate(bytes);
  table->sine.allocate(bytes);
  require_launch(launch_rope_tables(table->cosine.get(), table->sine.get(), runner.maximum_context,
                                    head_dim, theta, proportional, runner.stream),
                 "build RoPE tables");
  runner.rope_tables.push_back(std::move(table));
  return static_cast<int>(runner.rope_tables.size()) - 1;
}

size_t align_up(size_t value, size_t alignment = 256) {
  return (value + alignment - 1) / alignment * alignment;
}

void build_runner(Runner &runner, const carat_b200_model_config &config,
                  const carat_b200_model_weights &weights, int batch, int maximum_context,
                  const carat_b200_assistant_config *assistant,
                  const carat_b200_assistant_weights *assistant_weights) {
  if (batch <= 0 || maximum_context <= 0 || config.layer_count <= 0 || config.layers == nullptr ||
      weights.layers == nullptr || config.hidden_size <= 0 || config.hidden_size % 16 != 0 ||
      config.intermediate_size <= 0 || config.intermediate_size % 16 != 0 ||
      config.vocabulary_size <= 0 || config.sliding_window <= 0 ||
      weights.token_embedding == nullptr || weights.token_embedding_fp8 == nullptr ||
      weights.token_embedding_scale == nullptr || weights.final_norm == nullptr) {
    throw Failure{"invalid batch model runner shape"};
  }
  runner.config = config;
  runner.shapes.assign(config.layers, config.layers + config.layer_count);
  runner.config.layers = runner.shapes.data();
  runner.weights = weights;
  runner.batch = batch;
  runner.maximum_context = maximum_context;
  require_cuda(cudaStreamCreateWithFlags(&runner.stream, cudaStreamNonBlocking),
               "create runner stream");
  require_cuda(cudaEventCreate(&runner.start_event), "create timing event");
  require_cuda(cudaEventCreate(&runner.stop_event), "create timing event");
  runner.device_error = device_error_word();
  if (runner.device_error == nullptr)
    throw Failure{"device error word is unavailable"};

  const int hidden = config.hidden_size;
  const int rows = maximum_rows;
  int widest_query = 0;
  int widest_packed = 0;
  std::vector<CommitLayer> commit;
  runner.layers.resize(static_cast<size_t>(config.layer_count));
  for (int index = 0; index < config.layer_count; ++index) {
    LayerState &layer = runner.layers[static_cast<size_t>(index)];
    layer.shape = config.layers[index];
    layer.weights = weights.layers[index];
    const auto &shape = layer.shape;
    if (shape.query_heads <= 0 || shape.kv_heads <= 0 || shape.query_heads % shape.kv_heads != 0 ||
        (shape.head_dim != 64 && shape.head_dim != 256 && shape.head_dim != 512)) {
      throw Failure{"unsupported Gemma 4 attention shape"};
    }
    if (shape.global_attention) {
      runner.shared_global = index;
    } else {
      runner.shared_sliding = index;
    }
    layer.capacity = shape.global_attention ? maximum_context
                                            : std::min(maximum_context, config.sliding_window);
    layer.head_stride = static_cast<long long>(layer.capacity) * shape.head_dim;
    layer.slot_stride = layer.head_stride * shape.kv_heads;
    const size_t payload = align_up(static_cast<size_t>(batch) * layer.slot_stride * 2);
    layer.value_offset = payload;
    layer.kv.allocate(2 * payload, true);
    layer.rope = find_rope(runner, shape.head_dim, shape.rope_theta, shape.global_attention != 0);
    if (!shape.global_attention) {
      const size_t staged = align_up(static_cast<size_t>(batch) * shape.kv_heads * maximum_depth *
                                     shape.head_dim * 2);
      layer.staged_value_offset = staged;
      layer.staged.allocate(2 * staged, true);
      CommitLayer entry{};
      entry.key_cache = layer.keys();
      entry.value_cache = layer.values();
      entry.staged_keys = layer.staged_keys();
      entry.staged_values = layer.staged_values();
      entry.slot_stride = layer.slot_stride;
      entry.head_stride = layer.head_stride;
      entry.kv_heads = shape.kv_heads;
      entry.head_dim = shape.head_dim;
      entry.capacity = layer.capacity;
      commit.push_back(entry);
    }
    widest_query = std::max(widest_query, layer.query_width());
    widest_packed = std::max(widest_packed, layer.packed_width());
  }
  runner.commit_layer_count = static_cast<int>(commit.size());
  if (!commit.empty()) {
    runner.commit_layers.allocate(commit.size() * sizeof(CommitLayer));
    require_cuda(cudaMemcpy(runner.commit_layers.get(), commit.data(),
                            commit.size() * sizeof(CommitLayer), cudaMemcpyHostToDevice),
                 "copy commit table");
  }

  runner.slot_positions.assign(static_cast<size_t>(batch), 0);
  runner.hidden_by_slot.allocate(static_cast<size_t>(batch) * hidden * 2, true);
  const size_t row_hidden = static_cast<size_t>(rows) * hidden * 2;
  runner.hidden_a.allocate(row_hidden);
  runner.hidden_b.allocate(row_hidden);
  runner.residual.allocate(row_hidden);
  runner.final_hidden.allocate(row_hidden, true);
  const int widest_input = std::max({hidden, config.intermediate_size, widest_query});
  runner.quantized.allocate(static_cast<size_t>(rows) * widest_input);
  runner.packed.allocate(static_cast<size_t>(rows) * widest_packed * 2);
  runner.queries.allocate(static_cast<size_t>(rows) * widest_query * 2);
  runner.attention_out.allocate(static_cast<size_t>(rows) * widest_query * 2);
  const int global_chunks = attention_chunks(maximum_context, global_chunk_keys);
  runner.attention_partials.allocate(static_cast<size_t>(global_chunks) * rows * widest_query * 4);
  const int sliding_capacity = std::min(maximum_context, config.sliding_window);
  runner.score_stride_sliding = score_columns(sliding_capacity);
  runner.score_stride_global = score_columns(maximum_context);
  int most_heads = 0;
  for (const LayerState &layer : runner.layers)
    most_heads = std::max(most_heads, layer.shape.query_heads);
  runner.scores.allocate(static_cast<size_t>(rows) * most_heads *
                         std::max(runner.score_stride_sliding, runner.score_stride_global) * 2);
  runner.request_chunks.allocate(static_cast<size_t>(batch) * sizeof(int), true);
  runner.two_launch_rows.allocate(static_cast<size_t>(rows) * widest_input * 2);
  runner.stats_stride = global_chunks;
  runner.attention_stats.allocate(static_cast<size_t>(rows) * most_heads * global_chunks *
                                  sizeof(float2));
  runner.projected.allocate(row_hidden);
  runner.gate_up.allocate(static_cast<size_t>(rows) * 2 * config.intermediate_size * 2);
  // CARAT_B200_FUSED_GEGLU=1 runs gate_up, GeGLU and the activation quantisation as one launch
  // (launch_linear_gated) instead of linear -> GeGLU kernel. Off by default: measured on the 31B
  // shapes it is no faster, because the separate GeGLU kernel finishes the linear's K-cut tail
  // tiles across the whole device for free, while the one-launch form pays two grid-wide
  // barriers for the same work.
  const char *fused = std::getenv("CARAT_B200_FUSED_GEGLU");
  runner.fused_geglu = config.intermediate_size % 64 == 0 && fused != nullptr && fused[0] == '1';
  const char *cooperative = std::getenv("CARAT_B200_COOPERATIVE_ROWS");
  runner.cooperative_rows = cooperative != nullptr && cooperative[0] == '1';
  const char *early_keys = std::getenv("CARAT_B200_EARLY_KEYS");
  runner.early_keys = early_keys == nullptr || early_keys[0] != '0';
  const char *attention_amax = std::getenv("CARAT_B200_ATTENTION_AMAX");
  runner.attention_amax = attention_amax == nullptr || attention_amax[0] != '0';
  runner.gated_rows.allocate(static_cast<size_t>(rows) * config.intermediate_size * 2);
  runner.grid_counter.allocate(256, true);
  // Split-K partials [splits, rows, features] fp32; plans that would need more are rejected.
  runner.split_partials.allocate(static_cast<size_t>(16) * rows * std::max(hidden, 4096) * 4);
  // One (maximum, barrier count) pair of words per quantisation of a step.
  runner.amax_words = (config.layer_count + 1) * 4 * 2;
  runner.scratch_words.allocate(static_cast<size_t>(runner.amax_words + 2 * rows) * 4, true);
  runner.scales.allocate(static_cast<size_t>(runner.amax_words) * 4, true);
  runner.step_inputs.allocate(sizeof(int) * (rows + 4 * batch), true);
  runner.step_results.allocate(sizeof(int) * (2 * batch + rows + 1), true);
  runner.host_inputs.allocate(sizeof(int) * (rows + 4 * batch));
  runner.host_results.allocate(sizeof(int) * (2 * batch + rows + 1 + batch * maximum_depth));

  if (assistant != nullptr && assistant_weights != nullptr) {
    if (assistant->hidden_size <= 0 || assistant->hidden_size % 16 != 0 ||
        assistant->intermediate_size <= 0 || assistant->intermediate_size % 16 != 0 ||
        assistant->query_heads <= 0 || assistant->layer_count <= 0 ||
        assistant->layer_global == nullptr || assistant_weights->layers == nullptr ||
        assistant_weights->final_norm == nullptr) {
      throw Failure{"invalid assistant shape"};
    }
    // e4m3 matrices are optional: without them only the bf16 precision can be selected.
    runner.assistant_has_fp8 = assistant_weights->token_embedding != nullptr &&
                               assistant_weights->pre_projection != nullptr &&
                               assistant_weights->post_projection != nullptr;
    runner.assistant_mode = runner.assistant_has_fp8 ? CARAT_B200_ASSISTANT_FP8_ALL : -1;
    runner.has_assistant = true;
    runner.assistant = *assistant;
    runner.assistant_kinds.assign(assistant->layer_global,
                                  assistant->layer_global + assistant->layer_count);
    runner.assistant.layer_global = runner.assistant_kinds.data();
    runner.assistant_weights = *assistant_weights;
    runner.assistant_layers.assign(assistant_weights->layers,
                                   assistant_weights->layers + assistant->layer_count);
    runner.assistant_weights.layers = runner.assistant_layers.data();
    int widest = 0;
    for (int index = 0; index < assistant->layer_count; ++index) {
      const int shared = assistant->layer_global[index] ? runner.shared_global : runner.shared_sliding;
      if (shared < 0)
        throw Failure{"assistant layer has no target KV layer to share"};
      const auto &shape = runner.layers[static_cast<size_t>(shared)].shape;
      if (assistant->query_heads % shape.kv_heads != 0)
        throw Failure{"assistant query heads do not divide into the shared KV heads"};
      widest = std::max(widest, assistant->query_heads * shape.head_dim);
    }
    const int a_hidden = assistant->hidden_size;
    const size_t a_row_hidden = static_cast<size_t>(batch) * a_hidden * 2;
    runner.a_hidden_a.allocate(a_row_hidden);
    runner.a_hidden_b.allocate(a_row_hidden);
    runner.a_residual.allocate(a_row_hidden);
    runner.a_final_hidden.allocate(a_row_hidden);
    runner.a_linear_out.allocate(std::max(a_row_hidden, static_cast<size_t>(batch) * hidden * 2));
    const int a_widest_input =
        std::max({2 * hidden, assistant->intermediate_size, widest, a_hidden});
    runner.a_quantized.allocate(static_cast<size_t>(batch) * a_widest_input);
    runner.a_projected.allocate(static_cast<size_t>(batch) * widest * 2);
    runner.a_queries.allocate(static_cast<size_t>(batch) * widest * 2);
    runner.a_attention_out.allocate(static_cast<size_t>(batch) * widest * 2);
    runner.a_attention_partials.allocate(static_cast<size_t>(global_chunks) * batch * widest * 4);
    runner.a_scores.allocate(static_cast<size_t>(batch) * assistant->query_heads *
                             runner.score_stride_global * 2);
    runner.a_gate_up.allocate(static_cast<size_t>(batch) * 2 * assistant->intermediate_size * 2);
    runner.a_previous_hidden.allocate(static_cast<size_t>(batch) * hidden * 2);
    runner.a_amax_words = (2 + 4 * assistant->layer_count) * 2;
    // One set of scratch words per draft iteration, so that one clear serves the whole call.
    runner.a_scratch_words.allocate(
        static_cast<size_t>(runner.a_amax_words + 2 * batch) * 4 * maximum_depth, true);
    runner.a_scales.allocate(static_cast<size_t>(runner.a_amax_words) * 4, true);
    runner.a_concat.allocate(static_cast<size_t>(batch) * 2 * hidden * 2);
    runner.a_normed.allocate(a_row_hidden);
    runner.a_pre_mlp.allocate(a_row_hidden);
    runner.a_activated.allocate(static_cast<size_t>(batch) * assistant->intermediate_size * 2);
    runner.a_tokens.allocate(sizeof(int) * 4 * batch, true);
    runner.a_proposals.allocate(sizeof(int) * batch * maximum_depth, true);
  }
  require_cuda(cudaStreamSynchronize(runner.stream), "finish runner construction");
}

StepPlans &verify_plans_for(Runner &runner, int rows) {
  const auto found = runner.verify_plans.find(rows);
  if (found != runner.verify_plans.end())
    return found->second;
  StepPlans plans;
  const int hidden = runner.config.hidden_size;
  const int intermediate = runner.config.intermediate_size;
  for (const LayerState &layer : runner.layers) {
    LayerPlans entry;
    entry.qkv = plan_linear(runner.quantized.get(), layer.weights.qkv, rows, hidden,
                            layer.packed_width(), 0);
    entry.o = plan_linear(runner.quantized.get(), layer.weights.o, rows, layer.query_width(),
                          hidden, 0);
    entry.gate_up = plan_linear(runner.quantized.get(), layer.weights.gate_up, rows, hidden,
                                2 * intermediate, 0);
    entry.down = plan_linear(runner.quantized.get(), layer.weights.down, rows, intermediate,
                             hidden, 0);
    for (const LinearPlan *plan : {&entry.qkv, &entry.o, &entry.gate_up, &entry.down}) {
      if (linear_partial_bytes(*plan) > runner.split_partials.bytes())
        throw Failure{"split-K workspace is too small for this model shape"};
    }
    if (runner.fused_geglu) {
      const char *message = "invalid FP8 linear shape";
      if (make_gated_linear_plan(&entry.gate_up_gated, runner.quantized.get(),
                                 layer.weights.gate_up, rows, hidden, intermediate,
                                 &message) != 0) {
        throw Failure{message};
      }
      if (linear_tail_bytes(entry.gate_up_gated) > runner.split_partials.bytes())
        throw Failure{"split-K workspace is too small for this model shape"};
    }
    if (!runner.int4_layers.empty()) {
      const auto &int4 = runner.int4_layers[plans.layers.size()];
      const char *message = "invalid BF16 INT4 linear weight shape";
      if (make_int4_linear_plan(&entry.gate_up_int4, runner.pre_mlp.get(), int4.gate_up_codes,
                                int4.gate_up_scales, rows, hidden, 2 * intermediate,
                                runner.int4_group, 0, &message) != 0 ||
          make_int4_linear_plan(&entry.down_int4, runner.activated.get(), int4.down_codes,
                                int4.down_scales, rows, intermediate, hidden, runner.int4_group, 0,
                                &message) != 0) {
        throw Failure{message};
      }
      if (int4_linear_partial_bytes(entry.gate_up_int4) > runner.split_partials.bytes() ||
          int4_linear_partial_bytes(entry.down_int4) > runner.split_partials.bytes()) {
        throw Failure{"split-K workspace is too small for this model shape"};
      }
    }
    plans.layers.push_back(entry);
  }
  plans.head = plan_linear(runner.quantized.get(), runner.weights.token_embedding_fp8, rows, hidden,
                           runner.config.vocabulary_size, 1);
  return runner.verify_plans.emplace(rows, std::move(plans)).first->second;
}

const LayerState &shared_layer(const Runner &runner, int assistant_layer) {
  const int index = runner.assistant_kinds[static_cast<size_t>(assistant_layer)]
                        ? runner.shared_global
                        : runner.shared_sliding;
  return runner.layers[static_cast<size_t>(index)];
}

StepPlans &draft_plans_for(Runner &runner, int rows) {
  const auto found = runner.draft_plans.find(rows);
  if (found != runner.draft_plans.end())
    return found->second;
  StepPlans plans;
  const int hidden = runner.config.hidden_size;
  const int a_hidden = runner.assistant.hidden_size;
  const int intermediate = runner.assistant.intermediate_size;
  size_t most_partial = 0;
  for (int index = 0; index < runner.assistant.layer_count; ++index) {
    const auto &weights = runner.assistant_layers[static_cast<size_t>(index)];
    const int query_width = runner.assistant.query_heads * shared_layer(runner, index).shape.head_dim;
    LayerPlans entry;
    // Short K (a few K blocks) and a bf16 result: one piece per tile beats a split plus a
    // finishing kernel even when the tiles do not fill the device.
    entry.qkv = plan_linear(runner.a_quantized.get(), weights.qkv, rows, a_hidden, query_width, 1);
    entry.o = plan_linear(runner.a_quantized.get(), weights.o, rows, query_width, a_hidden, 0);
    entry.gate_up =
        plan_linear(runner.a_quantized.get(), weights.gate_up, rows, a_hidden, 2 * intermediate, 0);
    entry.down = plan_linear(runner.a_quantized.get(), weights.down, rows, intermediate, a_hidden, 0);
    for (const LinearPlan *plan : {&entry.qkv, &entry.o, &entry.gate_up, &entry.down})
      most_partial = std::max(most_partial, linear_partial_bytes(*plan));
    plans.layers.push_back(entry);
  }
  plans.head = plan_linear(runner.a_quantized.get(), runner.assistant_weights.token_embedding, rows,
                           a_hidden, runner.config.vocabulary_size, 1);
  plans.pre = plan_linear(runner.a_quantized.get(), runner.assistant_weights.pre_projection, rows,
                          2 * hidden, a_hidden, 0);
  plans.post = plan_linear(runner.a_quantized.get(), runner.assistant_weights.post_projection, rows,
                           a_hidden, hidden, 1);
  most_partial = std::max({most_partial, linear_partial_bytes(plans.pre),
                           linear_partial_bytes(plans.post)});
  if (most_partial > runner.split_partials.bytes())
    throw Failure{"split-K workspace is too small for this assistant shape"};
  return runner.draft_plans.emplace(rows, std::move(plans)).first->second;
}

LinearPlan plan_bf16_linear(const void *input, const void *weight, int rows, int in, int out,
                            int splits) {
  LinearPlan plan;
  const char *message = "invalid BF16 linear shape";
  if (make_linear_plan(&plan, input, weight, rows, in, out, splits, &message, 2) != 0)
    throw Failure{"invalid BF16 linear shape"};
  return plan;
}

// The drafter's linears over bf16 weights and activations; the LM head stays the e4m3 plan of
// draft_plans_for() in the lm_head mode.
StepPlans &draft_plans_bf16_for(Runner &runner, int rows) {
  const auto found = runner.draft_plans_bf16.find(rows);
  if (found != runner.draft_plans_bf16.end())
    return found->second;
  StepPlans plans;
  const int hidden = runner.config.hidden_size;
  const int a_hidden = runner.assistant.hidden_size;
  const int intermediate = runner.assistant.intermediate_size;
  const auto &bf16 = runner.assistant_bf16;
  size_t most_partial = 0;
  for (int index = 0; index < runner.assistant.layer_count; ++index) {
    const auto &weights = runner.assistant_bf16_layers[static_cast<size_t>(index)];
    const int query_width = runner.assistant.query_heads * shared_layer(runner, index).shape.head_dim;
    LayerPlans entry;
    entry.qkv = plan_bf16_linear(runner.a_normed.get(), weights.q, rows, a_hidden, query_width, 1);
    entry.o = plan_bf16_linear(runner.a_attention_out.get(), weights.o, rows, query_width,
                               a_hidden, 0);
    entry.gate_up = plan_bf16_linear(runner.a_pre_mlp.get(), weights.gate_up, rows, a_hidden,
                                     2 * intermediate, 0);
    entry.down = plan_bf16_linear(runner.a_activated.get(), weights.down, rows, intermediate,
                                  a_hidden, 0);
    for (const LinearPlan *plan : {&entry.qkv, &entry.o, &entry.gate_up, &entry.down})
      most_partial = std::max(most_partial, linear_partial_bytes(*plan));
    plans.layers.push_back(entry);
  }
  plans.head = plan_bf16_linear(runner.a_final_hidden.get(), bf16.token_embedding, rows, a_hidden,
                                runner.config.vocabulary_size, 1);
  plans.pre = plan_bf16_linear(runner.a_concat.get(), bf16.pre_projection, rows, 2 * hidden,
                               a_hidden, 0);
  plans.post = plan_bf16_linear(runner.a_final_hidden.get(), bf16.post_projection, rows, a_hidden,
                                hidden, 1);
  most_partial = std::max({most_partial, linear_partial_bytes(plans.pre),
                           linear_partial_bytes(plans.post)});
  if (most_partial > runner.split_partials.bytes())
    throw Failure{"split-K workspace is too small for this assistant shape"};
  return runner.draft_plans_bf16.emplace(rows, std::move(plans)).first->second;
}

StepPlans &prefill_plans_for(Runner &runner, int rows) {
  const auto found = runner.prefill_plans.find(rows);
  if (found != runner.prefill_plans.end())
    return found->second;
  StepPlans plans;
  const int hidden = runner.config.hidden_size;
  const int intermediate = runner.config.intermediate_size;
  for (size_t index = 0; index < runner.layers.size(); ++index) {
    const LayerState &layer = runner.layers[index];
    const carat_b200_layer_bf16_weights &weights = runner.bf16_layers[index];
    LayerPlans entry;
    entry.qkv = plan_bf16_linear(runner.p_normed.get(), weights.qkv, rows, hidden,
                                 layer.packed_width(), 0);
    entry.o = plan_bf16_linear(runner.attention_out.get(), weights.o, rows, layer.query_width(),
                               hidden, 0);
    entry.gate_up = plan_bf16_linear(runner.p_pre_mlp.get(), weights.gate_up, rows, hidden,
                                     2 * intermediate, 0);
    entry.down = plan_bf16_linear(runner.p_activated.get(), weights.down, rows, intermediate,
                                  hidden, 0);
    for (const LinearPlan *plan : {&entry.qkv, &entry.o, &entry.gate_up, &entry.down}) {
      if (linear_partial_bytes(*plan) > runner.split_partials.bytes())
        throw Failure{"split-K workspace is too small for this model shape"};
    }
    plans.layers.push_back(entry);
  }
  plans.head = plan_bf16_linear(runner.final_hidden.get(), runner.weights.token_embedding, rows,
                                hidden, runner.config.vocabulary_size, 1);
  return runner.prefill_plans.emplace(rows, std::move(plans)).first->second;
}

// Runs a linear into bf16 `output`, or leaves split-K partials for a fused consumer. Returns the
// PartialSource the consumer should read (splits == 0 means "read `output`").
PartialSource run_linear(Runner &runner, const LinearPlan &plan, const float *input_scale,
                         const float *weight_scale, void *output, bool consumer_sums) {
  auto *partials = runner.split_partials.get<float>();
  if (plan.splits > 1 && consumer_sums) {
    require_launch(launch_linear_partial(plan, partials, runner.device_error, runner.stream),
                   "FP8 linear");
    runner.launches += 1;
    return PartialSource{partials, plan.splits, input_scale, weight_scale};
  }
  require_launch(launch_linear_bf16(plan, input_scale, weight_scale, output, partials,
                                    runner.device_error, runner.stream),
                 "FP8 linear");
  runner.launches += (plan.splits > 1 || plan.tail_tiles > 0) ? 2 : 1;
  return PartialSource{nullptr, 0, nullptr, nullptr};
}

// Tensor maps of the tensor-core attention for one target layer at one depth (null when the layer
// shape needs the CUDA-core kernels: head_dim 64 or a capacity that is not a multiple of 128).
const AttentionMaps *verify_attention_maps(Runner &runner, int layer_index, int depth) {
  const LayerState &layer = runner.layers[static_cast<size_t>(layer_index)];
  const auto &shape = layer.shape;
  const int padded = attention_padded_rows(shape.query_heads / shape.kv_heads * depth);
  if ((shape.head_dim != 256 && shape.head_dim != 512) || layer.capacity % 128 != 0 || padded == 0)
    return nullptr;
  const auto key = std::make_pair(layer_index, depth);
  const auto found = runner.verify_maps.find(key);
  if (found != runner.verify_maps.end())
    return &found->second;
  const bool staged = !shape.global_attention;
  const int stride = staged ? runner.score_stride_sliding : runner.score_stride_global;
  AttentionMaps maps;
  const int status = make_attention_maps(
      &maps, layer.keys(), layer.values(),
      static_cast<long long>(runner.batch) * shape.kv_heads * layer.capacity,
      staged ? layer.staged_keys() : nullptr, staged ? layer.staged_values() : nullptr,
      static_cast<long long>(runner.batch) * shape.kv_heads * depth, runner.queries.get(),
      static_cast<long long>(runner.queries.bytes() / (2 * shape.head_dim)), runner.scores.get(),
      static_cast<long long>(runner.scores.bytes() / (2 * stride)), stride, shape.head_dim, padded);
  if (status != 0)
    throw Failure{"attention tensor map encoding failed"};
  return &runner.verify_maps.emplace(key, maps).first->second;
}

// The same for a sliding layer whose rings are read as linear caches (prefill before the first
// wrap): no staged proposals, the ring's own rows only.
const AttentionMaps *direct_attention_maps(Runner &runner, int layer_index, int depth) {
  const LayerState &layer = runner.layers[static_cast<size_t>(layer_index)];
  const auto &shape = layer.shape;
  const int padded = attention_padded_rows(shape.query_heads / shape.kv_heads * depth);
  if ((shape.head_dim != 256 && shape.head_dim != 512) || layer.capacity % 128 != 0 || padded == 0)
    return nullptr;
  const auto key = std::make_pair(layer_index, depth);
  const auto found = runner.direct_maps.find(key);
  if (found != runner.direct_maps.end())
    return &found->second;
  const int stride = runner.score_stride_sliding;
  AttentionMaps maps;
  const int status = make_attention_maps(
      &maps, layer.keys(), layer.values(),
      static_cast<long long>(runner.batch) * shape.kv_heads * layer.capacity, nullptr, nullptr, 0,
      runner.queries.get(), static_cast<long long>(runner.queries.bytes() / (2 * shape.head_dim)),
      runner.scores.get(), static_cast<long long>(runner.scores.bytes() / (2 * stride)), stride,
      shape.head_dim, padded);
  if (status != 0)
    throw Failure{"attention tensor map encoding failed"};
  return &runner.direct_maps.emplace(key, maps).first->second;
}

const AttentionMaps *draft_attention_maps(Runner &runner, int assistant_layer) {
  const LayerState &shared = shared_layer(runner, assistant_layer);
  const auto &shape = shared.shape;
  const int padded = attention_padded_rows(runner.assistant.query_heads / shape.kv_heads);
  if ((shape.head_dim != 256 && shape.head_dim != 512) || shared.capacity % 128 != 0 || padded == 0)
    return nullptr;
  const auto found = runner.draft_maps.find(assistant_layer);
  if (found != runner.draft_maps.end())
    return &found->second;
  const int stride = runner.score_stride_global;
  AttentionMaps maps;
  const int status = make_attention_maps(
      &maps, shared.keys(), shared.values(),
      static_cast<long long>(runner.batch) * shape.kv_heads * shared.capacity, nullptr, nullptr, 0,
      runner.a_queries.get(),
      static_cast<long long>(runner.a_queries.bytes() / (2 * shape.head_dim)),
      runner.a_scores.get(), static_cast<long long>(runner.a_scores.bytes() / (2 * stride)), stride,
      shape.head_dim, padded);
  if (status != 0)
    throw Failure{"attention tensor map encoding failed"};
  return &runner.draft_maps.emplace(assistant_layer, maps).first->second;
}

struct StepLayout {
  int *tokens;
  int *positions;
  int *slots;
  int *target_first;
  int *caps;
};

StepLayout layout_inputs(int *base, int rows, int batch) {
  return {base, base + rows, base + rows + batch, base + rows + 2 * batch, base + rows + 3 * batch};
}

void verify_step(Runner &runner, const int *proposals, int requests, int depth,
                 const int *target_first, const int *slots, const int *caps, int flags,
                 bool allow_empty_slot, int *accepted_out, int *next_out) {
  const auto &config = runner.config;
  if (proposals == nullptr || requests <= 0 || requests > runner.batch || depth <= 0 ||
      depth > maximum_depth || requests * depth > maximum_rows || target_first == nullptr ||
      slots == nullptr || accepted_out == nullptr || next_out == nullptr) {
    throw Failure{"invalid greedy verification batch"};
  }
  if (!runner.int4_layers.empty() && requests * depth > 128)
    throw Failure{"invalid BF16 INT4 linear activation shape"};
  std::vector<bool> seen(static_cast<size_t>(runner.batch), false);
  const int rows = requests * depth;
  const StepLayout host = layout_inputs(runner.host_inputs.get<int>(), maximum_rows, runner.batch);
  int longest = 0;
  for (int request = 0; request < requests; ++request) {
    const int slot = slots[request];
    if (slot < 0 || slot >= runner.batch || seen[static_cast<size_t>(slot)])
      throw Failure{"invalid or repeated speculative slot"};
    seen[static_cast<size_t>(slot)] = true;
    const int position = runner.slot_positions[static_cast<size_t>(slot)];
    if ((position <= 0 && !allow_empty_slot) || position + depth > runner.maximum_context)
      throw Failure{"speculative slot is empty or lacks context capacity"};
    for (int token = 0; token < depth; ++token) {
      const int id = proposals[request * depth + token];
      if (id < 0 || id >= config.vocabulary_size)
        throw Failure{"speculative proposal contains an invalid token"};
      host.tokens[request * depth + token] = id;
    }
    host.positions[request] = position;
    host.slots[request] = slot;
    host.target_first[request] = target_first[request];
    host.caps[request] = caps != nullptr ? caps[request] : depth;
    longest = std::max(longest, position);
  }
  StepPlans &plans = verify_plans_for(runner, rows);
  const StepLayout device =
      layout_inputs(runner.step_inputs.get<int>(), maximum_rows, runner.batch);
  cudaStream_t stream = runner.stream;
  require_cuda(cudaMemcpyAsync(runner.step_inputs.get(), runner.host_inputs.get<int>(),
                               sizeof(int) * (maximum_rows + 4 * runner.batch),
                               cudaMemcpyHostToDevice, stream),
               "copy speculative step inputs");
  require_cuda(cudaEventRecord(runner.start_event, stream), "record step start");
  runner.launches = 0;

  const int hidden = config.hidden_size;
  const float epsilon = config.rms_norm_epsilon;
  auto *amax = runner.scratch_words.get<unsigned int>();
  auto *best = reinterpret_cast<unsigned long long *>(amax + runner.amax_words);
  auto *scales = runner.scales.get<float>();
  const auto target = [&](int word) {
    QuantTarget made{runner.quantized.get(), scales + word, amax + 2 * word,
                     runner.two_launch_rows.get()};
    if (!runner.cooperative_rows) {
      made.barrier_word = amax + 2 * word + 1;
      made.barrier_error = runner.device_error;
    }
    return made;
  };
  const auto bf16_target = [](void *rows_out) {
    return QuantTarget{nullptr, nullptr, nullptr, nullptr, rows_out};
  };
  // The running maxima and the packed argmax keys must be zero before the step's first atomic.
  require_cuda(cudaMemsetAsync(amax, 0, sizeof(int) * (runner.amax_words + 2 * maximum_rows),
                               stream),
               "clear step scratch");

  void *current = runner.hidden_a.get();
  void *other = runner.hidden_b.get();
  require_launch(launch_embed_norm_quant(runner.weights.token_embedding, device.tokens,
                                         config.vocabulary_size, runner.layers[0].weights.input_norm,
                                         current, target(0), rows, hidden, epsilon, nullptr, 0,
                                         stream),
                 "embedding and input norm");
  runner.launches += 1;

  for (int index = 0; index < config.layer_count; ++index) {
    const LayerState &layer = runner.layers[static_cast<size_t>(index)];
    const LayerPlans &plan = plans.layers[static_cast<size_t>(index)];
    const auto &shape = layer.shape;
    const auto &w = layer.weights;
    const int word = index * 4;
    const RopeTable &rope = *runner.rope_tables[static_cast<size_t>(layer.rope)];

    run_linear(runner, plan.qkv, scales + word, w.qkv_scale, runner.packed.get(), false);

    QkvPostArguments post{};
    post.inputs_static = runner.early_keys ? 1 : 0;   // positions: step inputs
    post.packed = runner.packed.get();
    post.query_norm = w.q_norm;
    post.key_norm = w.k_norm;
    post.cosine = rope.cosine.get();
    post.sine = rope.sine.get();
    post.queries = runner.queries.get();
    post.positions = device.positions;
    post.slots = device.slots;
    post.requests = requests;
    post.depth = depth;
    post.query_heads = shape.query_heads;
    post.kv_heads = shape.kv_heads;
    post.head_dim = shape.head_dim;
    post.key_equals_value = shape.key_equals_value;
    post.max_positions = runner.maximum_context;
    post.epsilon = epsilon;
    post.capacity = layer.capacity;
    if (shape.global_attention) {
      post.direct = 1;
      post.key_base = layer.keys();
      post.value_base = layer.values();
      post.slot_stride = layer.slot_stride;
      post.head_stride = layer.head_stride;
    } else {
      post.direct = 0;
      post.key_base = layer.staged_keys();
      post.value_base = layer.staged_values();
      post.head_stride = static_cast<long long>(depth) * shape.head_dim;
      post.slot_stride = post.head_stride * shape.kv_heads;
    }
    require_launch(launch_qkv_post(post, stream), "QKV post-processing");
    runner.launches += 1;

    AttentionArguments attention{};
    attention.inputs_static = runner.early_keys ? 1 : 0;   // positions and slots: step inputs
    attention.queries = runner.queries.get();
    attention.key_cache = layer.keys();
    attention.value_cache = layer.values();
    attention.slot_stride = layer.slot_stride;
    attention.head_stride = layer.head_stride;
    attention.positions = device.positions;
    attention.slots = device.slots;
    attention.scores = runner.scores.get();
    attention.output = runner.attention_out.get();
    attention.chunk_partials = runner.attention_partials.get<float>();
    attention.requests = requests;
    attention.depth = depth;
    attention.query_heads = shape.query_heads;
    attention.kv_heads = shape.kv_heads;
    attention.head_dim = shape.head_dim;
    attention.capacity = layer.capacity;
    if (shape.global_attention) {
      attention.window = 0;
      attention.max_cache_rows = longest + depth;
      attention.score_stride = runner.score_stride_global;
      attention.chunk_keys = global_chunk_keys;
      attention.chunks = attention_chunks(longest + depth, global_chunk_keys);
    } else {
      attention.window = config.sliding_window;
      // The rings change only in the commit at the end of the step.
      attention.cache_static = runner.early_keys ? 1 : 0;
      attention.new_keys = layer.staged_keys();
      attention.new_values = layer.staged_values();
      attention.new_request_stride = post.slot_stride;
      attention.new_head_stride = post.head_stride;
      attention.max_cache_rows = std::min(longest, layer.capacity);
      attention.score_stride = runner.score_stride_sliding;
      attention.chunk_keys = (layer.capacity + 127) / 128 * 128;
      attention.chunks = 1;
    }
    attention.stats = runner.attention_stats.get<float2>();
    attention.stats_stride = runner.stats_stride;
    attention.request_chunks = runner.request_chunks.get<int>();
    attention.maps = verify_attention_maps(runner, index, depth);
    // The one-kernel attention leaves the largest |output| in the quantiser's (still zero) word.
    const bool amax_known = runner.attention_amax && attention.maps != nullptr &&
                            attention_tc_launches(attention) == 1;
    if (amax_known)
      attention.amax_bits = target(word + 1).amax_bits;
    require_launch(attention.maps != nullptr ? launch_attention_tc(attention, stream)
                                             : launch_attention_simt(attention, stream),
                   "verify attention");
    runner.launches += attention.maps != nullptr ? attention_tc_launches(attention) : 3;

    // The tensor-core path writes only the chunks a request has rows in and says how many.
    const bool counted = attention.chunks > 1 && attention.maps != nullptr;
    if (amax_known) {
      require_launch(launch_quantize_rows(runner.attention_out.get(), target(word + 1),
                                          static_cast<size_t>(rows) * layer.query_width(), stream),
                     "attention output quantisation");
    } else {
      require_launch(launch_quant(attention.chunks > 1 ? nullptr : runner.attention_out.get(),
                                  attention.chunks > 1 ? runner.attention_partials.get<float>()
                                                       : nullptr,
                                  attention.chunks,
                                  counted ? runner.request_chunks.get<int>() : nullptr, depth,
                                  target(word + 1), rows, layer.query_width(), stream),
                     "attention output quantisation");
    }
    runner.launches += 1;

    const PartialSource o_source = run_linear(runner, plan.o, scales + word + 1, w.o_scale,
                                              runner.projected.get(), true);
    const bool int4_mlp = !runner.int4_layers.empty();
    require_launch(launch_post_attention_norms_quant(
                       runner.projected.get(), o_source, w.post_attention_norm, current,
                       w.pre_mlp_norm, runner.residual.get(),
                       int4_mlp ? bf16_target(runner.pre_mlp.get()) : target(word + 2), rows,
                       hidden, epsilon, stream),
                   "post-attention norms");
    runner.launches += 1;

    if (int4_mlp) {
      // Weight-only INT4 gate_up and down: bf16 activations in, no e4m3 quantisation between.
      const float *unit = runner.unit_scale.get<float>();
      auto *partials = runner.split_partials.get<float>();
      const LinearPlan &up = plan.gate_up_int4.schedule;
      TailSource tail{};
      if (up.splits == 1 && up.tail_tiles > 0 && up.tail_tiles * 128 <= config.intermediate_size) {
        require_launch(launch_int4_linear_bf16_tail(plan.gate_up_int4, runner.gate_up.get(),
                                                    partials, runner.device_error, stream),
                       "INT4 linear");
        runner.launches += 1;
        tail = TailSource{partials, up.tail_splits,
                          2 * config.intermediate_size - up.tail_tiles * 128, up.tail_tiles * 128,
                          unit, unit};
      } else {
        require_launch(launch_int4_linear_bf16(plan.gate_up_int4, runner.gate_up.get(), partials,
                                               runner.device_error, stream),
                       "INT4 linear");
        runner.launches += (up.splits > 1 || up.tail_tiles > 0) ? 2 : 1;
      }
      require_launch(launch_geglu_quant(runner.gate_up.get(), tail,
                                        bf16_target(runner.activated.get()), rows,
                                        config.intermediate_size, stream),
                     "GeGLU");
      runner.launches += 1;
      const LinearPlan &down = plan.down_int4.schedule;
      PartialSource down_source{nullptr, 0, nullptr, nullptr};
      if (down.splits > 1) {
        require_launch(launch_int4_linear_partial(plan.down_int4, partials, runner.device_error,
                                                  stream),
                       "INT4 linear");
        runner.launches += 1;
        down_source = PartialSource{partials, down.splits, unit, unit};
      } else {
        require_launch(launch_int4_linear_bf16(plan.down_int4, runner.projected.get(), partials,
                                               runner.device_error, stream),
                       "INT4 linear");
        runner.launches += down.tail_tiles > 0 ? 2 : 1;
      }
      const bool last = index + 1 == config.layer_count;
      const void *next_norm =
          last ? runner.weights.final_norm
               : runner.layers[static_cast<size_t>(index) + 1].weights.input_norm;
      require_launch(launch_layer_output_norm_quant(
                         runner.projected.get(), down_source, w.post_mlp_norm,
                         runner.residual.get(), w.scalar, other, next_norm,
                         last ? runner.final_hidden.get() : nullptr, target(word + 4), rows, hidden,
                         epsilon, stream),
                     "layer output");
      runner.launches += 1;
      std::swap(current, other);
      continue;
    }

    if (runner.fused_geglu) {
      // GeGLU, the activation maximum and the e4m3 rows of the down projection all come out of
      // the gate_up launch.
      const QuantTarget quantised = target(word + 3);
      require_launch(launch_linear_gated(plan.gate_up_gated, scales + word + 2, w.gate_up_scale,
                                         runner.gated_rows.get(), quantised.amax_bits,
                                         quantised.fp8_output, quantised.scale,
                                         runner.split_partials.get<float>(),
                                         runner.grid_counter.get<unsigned int>(),
                                         runner.device_error, stream),
                     "FP8 gated linear");
      runner.launches += 1;
    } else {
    // 336 feature tiles on 148 SMs leave a short last round; its tiles are cut along K and the
    // GeGLU kernel, which reads the up half anyway, sums the pieces.
    TailSource tail{};
    if (plan.gate_up.tail_tiles > 0 &&
        linear_tail_bytes(plan.gate_up) <= runner.split_partials.bytes() &&
        plan.gate_up.tail_tiles * 128 <= config.intermediate_size) {
      require_launch(launch_linear_bf16_tail(plan.gate_up, scales + word + 2, w.gate_up_scale,
                                             runner.gate_up.get(),
                                             runner.split_partials.get<float>(),
                                             runner.device_error, stream),
                     "FP8 linear");
      runner.launches += 1;
      tail = TailSource{runner.split_partials.get<float>(), plan.gate_up.tail_splits,
                        2 * config.intermediate_size - plan.gate_up.tail_tiles * 128,
                        plan.gate_up.tail_tiles * 128, scales + word + 2, w.gate_up_scale};
    } else {
      run_linear(runner, plan.gate_up, scales + word + 2, w.gate_up_scale, runner.gate_up.get(),
                 false);
    }
    require_launch(launch_geglu_quant(runner.gate_up.get(), tail, target(word + 3), rows,
                                      config.intermediate_size, stream),
                   "GeGLU");
    runner.launches += 1;
    }

    const PartialSource down_source = run_linear(runner, plan.down, scales + word + 3,
                                                 w.down_scale, runner.projected.get(), true);
    const bool last = index + 1 == config.layer_count;
    const void *next_norm = last ? runner.weights.final_norm
                                 : runner.layers[static_cast<size_t>(index) + 1].weights.input_norm;
    require_launch(launch_layer_output_norm_quant(
                       runner.projected.get(), down_source, w.post_mlp_norm, runner.residual.get(),
                       w.scalar, other, next_norm, last ? runner.final_hidden.get() : nullptr,
                       target(word + 4), rows, hidden, epsilon, stream),
                   "layer output");
    runner.launches += 1;
    std::swap(current, other);
  }

  const int head_word = config.layer_count * 4;
  require_launch(launch_linear_argmax(plans.head, scales + head_word,
                                      runner.weights.token_embedding_scale, best,
                                      runner.device_error, stream),
                 "LM head");
  runner.launches += 1;

  int *results = runner.step_results.get<int>();
  AcceptArguments accept{};
  accept.best = best;
  accept.proposals = device.tokens;
  accept.target_first = device.target_first;
  accept.caps = device.caps;
  accept.assume_match = (flags & CARAT_B200_VERIFY_ASSUME_MATCH) != 0 ? 1 : 0;
  accept.accepted = results;
  accept.next_tokens = results + runner.batch;
  accept.predictions = results + 2 * runner.batch;
  accept.final_hidden = runner.final_hidden.get();
  accept.hidden_by_slot = runner.hidden_by_slot.get();
  accept.slots = device.slots;
  accept.requests = requests;
  accept.depth = depth;
  accept.hidden = hidden;
  require_launch(launch_accept(accept, stream), "greedy prefix accept");
  runner.launches += 1;
  if (runner.commit_layer_count > 0) {
    require_launch(launch_commit(runner.commit_layers.get<CommitLayer>(), runner.commit_layer_count,
                                 device.positions, accept.accepted, device.slots, requests, depth, 0,
                                 stream),
                   "KV commit");
    runner.launches += 1;
  }
  require_cuda(cudaEventRecord(runner.stop_event, stream), "record step end");
  int *host_results = runner.host_results.get<int>();
  const int result_words = 2 * runner.batch + maximum_rows;
  require_cuda(cudaMemcpyAsync(host_results, results, sizeof(int) * result_words,
                               cudaMemcpyDeviceToHost, stream),
               "copy speculative results");
  require_cuda(cudaMemcpyAsync(host_results + result_words, runner.device_error, sizeof(int),
                               cudaMemcpyDeviceToHost, stream),
               "copy device error word");
  require_cuda(cudaStreamSynchronize(stream), "synchronize speculative verification");
  require_cuda(cudaEventElapsedTime(&runner.last_verify_ms, runner.start_event, runner.stop_event),
               "read step time");
  runner.last_verify_launches = runner.launches;
  runner.last_rows = rows;
  if (host_results[result_words] != 0) {
    const int code = host_results[result_words];
    cudaMemsetAsync(runner.device_error, 0, sizeof(int), stream);
    throw Failure{"a kernel wait ran out during speculative verification (code " +
                  std::to_string(code) + ")"};
  }
  runner.last_predictions.assign(host_results + 2 * runner.batch,
                                 host_results + 2 * runner.batch + rows);
  for (int request = 0; request < requests; ++request) {
    accepted_out[request] = host_results[request];
    next_out[request] = host_results[runner.batch + request];
    runner.slot_positions[static_cast<size_t>(slots[request])] += host_results[request];
  }
}

// One BF16 forward over `depth` prompt tokens of each listed entry, all of them made resident:
// the verify step's layer loop with bf16 linears and no quantisation, every row committed.
// An entry is a slot; a slot may be listed several times in a row, each entry then being the next
// `depth` tokens of that slot's prompt. That form needs `linear_rings`: every listed slot's
// sliding rings are still unwrapped and stay so through this step, so the ring is a linear cache,
// K and V rows are written in place before the attention runs (as on global layers, and as the
// reference does before the first wrap, cuda/layer_runner.cu:851-878) and each entry attends
// causally to everything before it, the earlier entries of its own step included.
// When `predict` is set the bf16 LM head runs over the step's final-normed rows and
// predictions_out receives the argmax of every row (requests * depth).
void prefill_step(Runner &runner, const int *tokens, int requests, int depth, const int *slots,
                  bool linear_rings, const std::vector<int> &waves, bool predict,
                  int *predictions_out) {
  const auto &config = runner.config;
  const int rows = requests * depth;
  if (requests > prefill_pieces || rows > maximum_rows)
    throw Failure{"invalid batched chunk prefill shape"};
  const StepLayout host =
      layout_inputs(runner.p_host_inputs.get<int>(), maximum_rows, prefill_pieces);
  int longest = 0;
  std::vector<int> advanced(static_cast<size_t>(runner.batch), 0);
  for (int request = 0; request < requests; ++request) {
    const size_t slot = static_cast<size_t>(slots[request]);
    const int position = runner.slot_positions[slot] + advanced[slot];
    if (advanced[slot] > 0 && !linear_rings && waves.size() < 2)
      throw Failure{"invalid batched chunk prefill request"};
    advanced[slot] += depth;
    for (int token = 0; token < depth; ++token)
      host.tokens[request * depth + token] = tokens[request * depth + token];
    host.positions[request] = position;
    host.slots[request] = slots[request];
    host.target_first[request] = tokens[request * depth];
    host.caps[request] = depth;    // doubles as the accept length of the commit: every row stays
    longest = std::max(longest, position);
  }
  StepPlans &plans = prefill_plans_for(runner, rows);
  const StepLayout device =
      layout_inputs(runner.p_step_inputs.get<int>(), maximum_rows, prefill_pieces);
  cudaStream_t stream = runner.stream;
  require_cuda(cudaMemcpyAsync(runner.p_step_inputs.get(), runner.p_host_inputs.get<int>(),
                               sizeof(int) * (maximum_rows + 4 * prefill_pieces),
                               cudaMemcpyHostToDevice, stream),
               "copy prefill step inputs");
  require_cuda(cudaEventRecord(runner.start_event, stream), "record prefill start");
  runner.launches = 0;
  const int hidden = config.hidden_size;
  const float epsilon = config.rms_norm_epsilon;
  const auto rows_only = [](void *rows_out) {
    return QuantTarget{nullptr, nullptr, nullptr, nullptr, rows_out};
  };
  auto *best = reinterpret_cast<unsigned long long *>(runner.scratch_words.get<unsigned int>() +
                                                      runner.amax_words);
  if (predict)
    require_cuda(cudaMemsetAsync(best, 0, sizeof(unsigned long long) * maximum_rows, stream),
                 "clear argmax keys");

  void *current = runner.hidden_a.get();
  void *other = runner.hidden_b.get();
  require_launch(launch_embed_norm_quant(runner.weights.token_embedding, device.tokens,
                                         config.vocabulary_size, runner.layers[0].weights.input_norm,
                                         current, rows_only(runner.p_normed.get()), rows, hidden,
                                         epsilon, nullptr, 0, stream),
                 "embedding and input norm");
  runner.launches += 1;
  int sliding_ordinal = 0;   // index of the layer in the commit table (sliding layers, in order)
  for (int index = 0; index < config.layer_count; ++index) {
    const LayerState &layer = runner.layers[static_cast<size_t>(index)];
    const LayerPlans &plan = plans.layers[static_cast<size_t>(index)];
    const auto &shape = layer.shape;
    const auto &w = layer.weights;
    const RopeTable &rope = *runner.rope_tables[static_cast<size_t>(layer.rope)];
    run_linear(runner, plan.qkv, nullptr, nullptr, runner.packed.get(), false);

    QkvPostArguments post{};
    post.packed = runner.packed.get();
    post.query_norm = w.q_norm;
    post.key_norm = w.k_norm;
    post.cosine = rope.cosine.get();
    post.sine = rope.sine.get();
    post.queries = runner.queries.get();
    post.positions = device.positions;
    post.slots = device.slots;
    post.requests = requests;
    post.depth = depth;
    post.query_heads = shape.query_heads;
    post.kv_heads = shape.kv_heads;
    post.head_dim = shape.head_dim;
    post.key_equals_value = shape.key_equals_value;
    post.max_positions = runner.maximum_context;
    post.epsilon = epsilon;
    post.capacity = layer.capacity;
    const bool in_place = shape.global_attention || linear_rings;
    if (in_place) {
      post.direct = 1;
      post.key_base = layer.keys();
      post.value_base = layer.values();
      post.slot_stride = layer.slot_stride;
      post.head_stride = layer.head_stride;
    } else {
      post.direct = 0;
      post.key_base = layer.staged_keys();
      post.value_base = layer.staged_values();
      post.head_stride = static_cast<long long>(depth) * shape.head_dim;
      post.slot_stride = post.head_stride * shape.kv_heads;
    }
    // Wrapped rings with several pieces of one slot in the step: the pieces of a slot have to see
    // each other's rows through the ring, so the sliding layers go wave by wave (wave w = the w-th
    // piece of every slot that has one): post-process, attend, commit this layer's rows, next wave.
    const bool by_waves = !in_place && waves.size() > 1;
    if (!by_waves) {
      require_launch(launch_qkv_post(post, stream), "QKV post-processing");
      runner.launches += 1;
    }

    AttentionArguments attention{};
    attention.queries = runner.queries.get();
    attention.key_cache = layer.keys();
    attention.value_cache = layer.values();
    attention.slot_stride = layer.slot_stride;
    attention.head_stride = layer.head_stride;
    attention.positions = device.positions;
    attention.slots = device.slots;
    attention.scores = runner.scores.get();
    attention.output = runner.attention_out.get();
    attention.chunk_partials = runner.attention_partials.get<float>();
    attention.requests = requests;
    attention.depth = depth;
    attention.query_heads = shape.query_heads;
    attention.kv_heads = shape.kv_heads;
    attention.head_dim = shape.head_dim;
    attention.capacity = layer.capacity;
    if (shape.global_attention) {
      attention.window = 0;
      attention.max_cache_rows = longest + depth;
      attention.score_stride = runner.score_stride_global;
      attention.chunk_keys = global_chunk_keys;
      attention.chunks = attention_chunks(longest + depth, global_chunk_keys);
    } else if (linear_rings) {
      // Unwrapped ring: rows 0 .. position + depth - 1 in order, all inside the window.
      attention.window = 0;
      attention.max_cache_rows = longest + depth;
      attention.score_stride = runner.score_stride_sliding;
      attention.chunk_keys = (layer.capacity + 127) / 128 * 128;
      attention.chunks = 1;
    } else {
      attention.window = config.sliding_window;
      attention.new_keys = layer.staged_keys();
      attention.new_values = layer.staged_values();
      attention.new_request_stride = post.slot_stride;
      attention.new_head_stride = post.head_stride;
      attention.max_cache_rows = std::min(longest, layer.capacity);
      attention.score_stride = runner.score_stride_sliding;
      attention.chunk_keys = (layer.capacity + 127) / 128 * 128;
      attention.chunks = 1;
    }
    attention.stats = runner.attention_stats.get<float2>();
    attention.stats_stride = runner.stats_stride;
    attention.request_chunks = runner.p_request_chunks.get<int>();
    attention.maps = (linear_rings && !shape.global_attention)
                         ? direct_attention_maps(runner, index, depth)
                         : verify_attention_maps(runner, index, depth);
    if (by_waves) {
      const auto *packed_rows = runner.packed.get<unsigned char>();
      auto *output_rows = runner.attention_out.get<unsigned char>();
      const size_t packed_row_bytes = static_cast<size_t>(layer.packed_width()) * 2;
      const size_t output_row_bytes = static_cast<size_t>(layer.query_width()) * 2;
      const CommitLayer *commit_entry =
          runner.commit_layers.get<CommitLayer>() + sliding_ordinal;
      int base = 0;
      for (const int count : waves) {
        const size_t first_row = static_cast<size_t>(base) * depth;
        post.packed = packed_rows + first_row * packed_row_bytes;
        post.positions = device.positions + base;
        post.slots = device.slots + base;
        post.requests = count;
        require_launch(launch_qkv_post(post, stream), "QKV post-processing");
        attention.positions = device.positions + base;
        attention.slots = device.slots + base;
        attention.requests = count;
        attention.output = output_rows + first_row * output_row_bytes;
        require_launch(attention.maps != nullptr ? launch_attention_tc(attention, stream)
                                                 : launch_attention_simt(attention, stream),
                       "prefill attention");
        require_launch(launch_commit(commit_entry, 1, device.positions + base, device.caps + base,
                                     device.slots + base, count, depth, 0, stream),
                       "KV commit");
        runner.launches += 2 + (attention.maps != nullptr ? attention_tc_launches(attention) : 3);
        base += count;
      }
    } else {
      require_launch(attention.maps != nullptr ? launch_attention_tc(attention, stream)
                                               : launch_attention_simt(attention, stream),
                     "prefill attention");
      runner.launches += attention.maps != nullptr ? attention_tc_launches(attention) : 3;
    }
    if (!shape.global_attention)
      ++sliding_ordinal;
    if (attention.chunks > 1) {
      const bool counted = attention.maps != nullptr;
      require_launch(launch_quant(nullptr, runner.attention_partials.get<float>(),
                                  attention.chunks,
                                  counted ? runner.p_request_chunks.get<int>() : nullptr, depth,
                                  rows_only(runner.attention_out.get()), rows,
                                  layer.query_width(), stream),
                     "prefill attention rows");
      runner.launches += 1;
    }
    const PartialSource o_source =
        run_linear(runner, plan.o, nullptr, nullptr, runner.projected.get(), true);
    require_launch(launch_post_attention_norms_quant(
                       runner.projected.get(), o_source, w.post_attention_norm, current,
                       w.pre_mlp_norm, runner.residual.get(), rows_only(runner.p_pre_mlp.get()),
                       rows, hidden, epsilon, stream),
                   "post-attention norms");
    runner.launches += 1;
    run_linear(runner, plan.gate_up, nullptr, nullptr, runner.gate_up.get(), false);
    require_launch(launch_geglu_quant(runner.gate_up.get(), TailSource{},
                                      rows_only(runner.p_activated.get()), rows,
                                      config.intermediate_size, stream),
                   "GeGLU");
    runner.launches += 1;
    const PartialSource down_source =
        run_linear(runner, plan.down, nullptr, nullptr, runner.projected.get(), true);
    const bool last = index + 1 == config.layer_count;
    const void *next_norm = last ? runner.weights.final_norm
                                 : runner.layers[static_cast<size_t>(index) + 1].weights.input_norm;
    require_launch(launch_layer_output_norm_quant(
                       runner.projected.get(), down_source, w.post_mlp_norm, runner.residual.get(),
                       w.scalar, other, next_norm,
                       last ? runner.final_hidden.get() : runner.p_normed.get(), QuantTarget{},
                       rows, hidden, epsilon, stream),
                   "layer output");
    runner.launches += 1;
    std::swap(current, other);
  }
  if (runner.commit_layer_count > 0 && !linear_rings && waves.size() < 2) {
    require_launch(launch_commit(runner.commit_layers.get<CommitLayer>(), runner.commit_layer_count,
                                 device.positions, device.caps, device.slots, requests, depth, 0,
                                 stream),
                   "KV commit");
    runner.launches += 1;
  }
  int *host_results = runner.host_results.get<int>();
  if (predict) {
    require_launch(launch_linear_argmax(plans.head, nullptr, nullptr, best, runner.device_error,
                                        stream),
                   "BF16 LM head");
    int *predictions = runner.step_results.get<int>() + 2 * runner.batch;
    require_launch(launch_unpack_best(best, predictions, rows, stream), "prefill argmax");
    runner.launches += 2;
    require_cuda(cudaMemcpyAsync(host_results, predictions, sizeof(int) * rows,
                                 cudaMemcpyDeviceToHost, stream),
                 "copy prefill predictions");
  }
  require_cuda(cudaMemcpyAsync(host_results + maximum_rows, runner.device_error, sizeof(int),
                               cudaMemcpyDeviceToHost, stream),
               "copy device error word");
  require_cuda(cudaEventRecord(runner.stop_event, stream), "record prefill end");
  require_cuda(cudaStreamSynchronize(stream), "synchronize prefill step");
  require_cuda(cudaEventElapsedTime(&runner.last_verify_ms, runner.start_event, runner.stop_event),
               "read prefill step time");
  runner.last_verify_launches = runner.launches;
  if (host_results[maximum_rows] != 0) {
    const int code = host_results[maximum_rows];
    cudaMemsetAsync(runner.device_error, 0, sizeof(int), stream);
    throw Failure{"a kernel wait ran out during prefill (code " + std::to_string(code) + ")"};
  }
  if (predict)
    std::copy(host_results, host_results + rows, predictions_out);
  for (int request = 0; request < requests; ++request)
    runner.slot_positions[static_cast<size_t>(slots[request])] += depth;
  runner.last_rows = rows;
}

void draft_step(Runner &runner, const int *last_tokens, const int *slots, const int *forced,
                int requests, int depth, int *proposals_out) {
  if (!runner.has_assistant || last_tokens == nullptr || slots == nullptr || requests <= 0 ||
      proposals_out == nullptr) {
    throw Failure{"assistant is not configured or draft batch is invalid"};
  }
  if (requests > runner.batch || depth <= 0 || depth > maximum_depth)
    throw Failure{"invalid assistant draft batch"};
  const auto &config = runner.config;
  const auto &assistant = runner.assistant;
  int *host = runner.host_inputs.get<int>();
  int *host_tokens = host;
  int *host_context = host + runner.batch;
  int *host_slots = host + 2 * runner.batch;
  int *host_forced = host + 3 * runner.batch;
  int longest = 0;
  for (int row = 0; row < requests; ++row) {
    const int slot = slots[row];
    if (slot < 0 || slot >= runner.batch || runner.slot_positions[static_cast<size_t>(slot)] <= 0)
      throw Failure{"assistant slot is empty or invalid"};
    if (last_tokens[row] < 0 || last_tokens[row] >= config.vocabulary_size)
      throw Failure{"invalid assistant row metadata"};
    host_tokens[row] = last_tokens[row];
    host_context[row] = runner.slot_positions[static_cast<size_t>(slot)] - 1;
    host_slots[row] = slot;
    host_forced[row] = forced != nullptr ? forced[row] : 0;
    longest = std::max(longest, host_context[row] + 1);
  }
  if (runner.assistant_mode < 0)
    throw Failure{"assistant FP8 mode requires quantized assistant weights"};
  // The e4m3 plans also serve the lm_head mode (its LM head); without e4m3 matrices only the
  // bf16 plans exist.
  StepPlans no_fp8_plans;
  StepPlans &plans = runner.assistant_has_fp8 ? draft_plans_for(runner, requests) : no_fp8_plans;
  cudaStream_t stream = runner.stream;
  int *device = runner.a_tokens.get<int>();
  int *device_tokens = device;
  int *device_context = device + runner.batch;
  int *device_slots = device + 2 * runner.batch;
  int *device_forced = device + 3 * runner.batch;
  require_cuda(cudaMemcpyAsync(device, host, sizeof(int) * 4 * runner.batch,
                               cudaMemcpyHostToDevice, stream),
               "copy assistant inputs");
  require_cuda(cudaEventRecord(runner.start_event, stream), "record draft start");
  runner.launches = 0;

  const int hidden = config.hidden_size;
  const int a_hidden = assistant.hidden_size;
  const float epsilon = assistant.rms_norm_epsilon;
  // Every iteration has scratch words of its own (maxima, barrier counts, packed argmax keys), all
  // cleared here: a clear between two iterations would cut the chain of dependent launches.
  auto *scratch = runner.a_scratch_words.get<unsigned int>();
  const size_t scratch_stride = static_cast<size_t>(runner.a_amax_words) + 2 * runner.batch;
  require_cuda(cudaMemsetAsync(scratch, 0, sizeof(int) * scratch_stride * depth, stream),
               "clear assistant scratch");
  unsigned int *amax = scratch;
  auto *best = reinterpret_cast<unsigned long long *>(amax + runner.a_amax_words);
  auto *scales = runner.a_scales.get<float>();
  const auto target = [&](int word) {
    QuantTarget made{runner.a_quantized.get(), scales + word, amax + 2 * word};
    if (!runner.cooperative_rows) {
      made.barrier_word = amax + 2 * word + 1;
      made.barrier_error = runner.device_error;
    }
    return made;
  };
  int *draft_tokens = runner.a_proposals.get<int>();  // [depth][requests]

  if (runner.assistant_mode == CARAT_B200_ASSISTANT_FP8_ALL) {
  for (int draft_index = 0; draft_index < depth; ++draft_index) {
    amax = scratch + draft_index * scratch_stride;
    best = reinterpret_cast<unsigned long long *>(amax + runner.a_amax_words);
    const int *input_tokens =
        draft_index == 0 ? device_tokens : draft_tokens + (draft_index - 1) * requests;
    require_launch(launch_embed_concat_quant(
                       runner.weights.token_embedding, input_tokens, config.vocabulary_size,
                       draft_index == 0 ? runner.hidden_by_slot.get()
                                        : runner.a_previous_hidden.get(),
                       draft_index == 0 ? device_slots : nullptr, target(0), requests, hidden,
                       stream),
                   "assistant input");
    runner.launches += 1;
    void *current = runner.a_hidden_a.get();
    void *other = runner.a_hidden_b.get();
    run_linear(runner, plans.pre, scales + 0, runner.assistant_weights.pre_projection_scale,
               current, false);
    require_launch(launch_norm_quant(current, runner.assistant_layers[0].input_norm, nullptr,
                                     target(1), requests, a_hidden, epsilon, stream),
                   "assistant input norm");
    runner.launches += 1;
    int input_word = 1;
    for (int index = 0; index < assistant.layer_count; ++index) {
      const auto &w = runner.assistant_layers[static_cast<size_t>(index)];
      const LayerPlans &plan = plans.layers[static_cast<size_t>(index)];
      const LayerState &shared = shared_layer(runner, index);
      const auto &shape = shared.shape;
      const int query_width = assistant.query_heads * shape.head_dim;
      const int word = 2 + 4 * index;
      const RopeTable &rope = *runner.rope_tables[static_cast<size_t>(shared.rope)];
      run_linear(runner, plan.qkv, scales + input_word, w.qkv_scale, runner.a_projected.get(),
                 false);
      require_launch(launch_query_post(runner.a_projected.get(), w.q_norm, rope.cosine.get(),
                                       rope.sine.get(), runner.a_queries.get(), device_context,
                                       draft_index, requests, assistant.query_heads,
                                       shape.head_dim, runner.maximum_context, epsilon, stream,
                                       runner.early_keys),
                     "assistant query post-processing");
      runner.launches += 1;
      AttentionArguments attention{};
      attention.inputs_static = runner.early_keys ? 1 : 0;   // positions and slots: step inputs
      attention.queries = runner.a_queries.get();
      attention.key_cache = shared.keys();
      attention.value_cache = shared.values();
      attention.slot_stride = shared.slot_stride;
      attention.head_stride = shared.head_stride;
      attention.positions = device_context;
      attention.slots = device_slots;
      attention.scores = runner.a_scores.get();
      attention.output = runner.a_attention_out.get();
      attention.chunk_partials = runner.a_attention_partials.get<float>();
      attention.requests = requests;
      attention.depth = 1;
      attention.query_heads = assistant.query_heads;
      attention.kv_heads = shape.kv_heads;
      attention.head_dim = shape.head_dim;
      attention.capacity = shared.capacity;
      attention.window = shape.global_attention ? 0 : config.sliding_window;
      attention.draft = 1;
      // Drafting reads the target's caches and writes none.
      attention.cache_static = runner.early_keys ? 1 : 0;
      attention.max_cache_rows = std::min(longest, shared.capacity);
      attention.score_stride = runner.score_stride_global;
      attention.chunk_keys = global_chunk_keys;
      attention.chunks = attention_chunks(attention.max_cache_rows, global_chunk_keys);
      attention.stats = runner.attention_stats.get<float2>();
      attention.stats_stride = runner.stats_stride;
      attention.request_chunks = runner.request_chunks.get<int>();
      attention.maps = draft_attention_maps(runner, index);
      const bool amax_known = runner.attention_amax && attention.maps != nullptr &&
                              attention_tc_launches(attention) == 1;
      if (amax_known)
        attention.amax_bits = target(word).amax_bits;
      require_launch(attention.maps != nullptr ? launch_attention_tc(attention, stream)
                                               : launch_attention_simt(attention, stream),
                     "assistant attention");
      runner.launches += attention.maps != nullptr ? attention_tc_launches(attention) : 3;
      const bool counted = attention.chunks > 1 && attention.maps != nullptr;
      if (amax_known) {
        require_launch(launch_quantize_rows(runner.a_attention_out.get(), target(word),
                                            static_cast<size_t>(requests) * query_width, stream),
                       "assistant attention quantisation");
      } else {
        require_launch(launch_quant(attention.chunks > 1 ? nullptr : runner.a_attention_out.get(),
                                    attention.chunks > 1 ? runner.a_attention_partials.get<float>()
                                                         : nullptr,
                                    attention.chunks,
                                    counted ? runner.request_chunks.get<int>() : nullptr, 1,
                                    target(word), requests, query_width, stream),
                       "assistant attention quantisation");
      }
      runner.launches += 1;
      const PartialSource o_source = run_linear(runner, plan.o, scales + word, w.o_scale,
                                                runner.a_linear_out.get(), true);
      require_launch(launch_post_attention_norms_quant(
                         runner.a_linear_out.get(), o_source, w.post_attention_norm, current,
                         w.pre_mlp_norm, runner.a_residual.get(), target(word + 1), requests,
                         a_hidden, epsilon, stream),
                     "assistant post-attention norms");
      runner.launches += 1;
      run_linear(runner, plan.gate_up, scales + word + 1, w.gate_up_scale, runner.a_gate_up.get(),
                 false);
      require_launch(launch_geglu_quant(runner.a_gate_up.get(), TailSource{}, target(word + 2), requests,
                                        assistant.intermediate_size, stream),
                     "assistant GeGLU");
      runner.launches += 1;
      const PartialSource down_source = run_linear(runner, plan.down, scales + word + 2,
                                                   w.down_scale, runner.a_linear_out.get(), true);
      const bool last = index + 1 == assistant.layer_count;
      const void *next_norm = last ? runner.assistant_weights.final_norm
                                   : runner.assistant_layers[static_cast<size_t>(index) + 1].input_norm;
      require_launch(launch_layer_output_norm_quant(
                         runner.a_linear_out.get(), down_source, w.post_mlp_norm,
                         runner.a_residual.get(), w.scalar, other, next_norm,
                         last ? runner.a_final_hidden.get() : nullptr, target(word + 3), requests,
                         a_hidden, epsilon, stream),
                     "assistant layer output");
      runner.launches += 1;
      input_word = word + 3;
      std::swap(current, other);
    }
    int *step_tokens = draft_tokens + draft_index * requests;
    if (draft_index == 0 && forced != nullptr) {
      // The target already produced this token; the drafter's LM head would be dead work
      // (cuda/assistant_runner.cu:306-312).
      require_cuda(cudaMemcpyAsync(step_tokens, device_forced, sizeof(int) * requests,
                                   cudaMemcpyDeviceToDevice, stream),
                   "select forced assistant first tokens");
    } else {
      require_launch(launch_linear_argmax(plans.head, scales + input_word,
                                          runner.assistant_weights.token_embedding_scale, best,
                                          runner.device_error, stream),
                     "assistant LM head");
      require_launch(launch_unpack_best(best, step_tokens, requests, stream), "assistant argmax");
      runner.launches += 2;
    }
    run_linear(runner, plans.post, scales + input_word,
               runner.assistant_weights.post_projection_scale, runner.a_previous_hidden.get(),
               false);
  }
  } else {
  // bf16 precision (the reference's default, and its lm_head mode): activations stay bf16 from
  // one linear to the next, so the row kernels stop after their bf16 rows and nothing is
  // quantised, except the final-normed hidden rows when the LM head alone runs in e4m3.
  const bool head_fp8 = runner.assistant_mode == CARAT_B200_ASSISTANT_FP8_LM_HEAD;
  StepPlans &wide = draft_plans_bf16_for(runner, requests);
  const auto rows_only = [](void *rows_out) {
    return QuantTarget{nullptr, nullptr, nullptr, nullptr, rows_out};
  };
  const int head_word = 0;
  for (int draft_index = 0; draft_index < depth; ++draft_index) {
    amax = scratch + draft_index * scratch_stride;
    best = reinterpret_cast<unsigned long long *>(amax + runner.a_amax_words);
    const int *input_tokens =
        draft_index == 0 ? device_tokens : draft_tokens + (draft_index - 1) * requests;
    require_launch(launch_embed_concat_quant(
                       runner.weights.token_embedding, input_tokens, config.vocabulary_size,
                       draft_index == 0 ? runner.hidden_by_slot.get()
                                        : runner.a_previous_hidden.get(),
                       draft_index == 0 ? device_slots : nullptr, rows_only(runner.a_concat.get()),
                       requests, hidden, stream),
                   "assistant input");
    runner.launches += 1;
    void *current = runner.a_hidden_a.get();
    void *other = runner.a_hidden_b.get();
    run_linear(runner, wide.pre, nullptr, nullptr, current, false);
    require_launch(launch_norm_quant(current, runner.assistant_layers[0].input_norm,
                                     runner.a_normed.get(), QuantTarget{}, requests, a_hidden,
                                     epsilon, stream),
                   "assistant input norm");
    runner.launches += 1;
    for (int index = 0; index < assistant.layer_count; ++index) {
      const auto &w = runner.assistant_layers[static_cast<size_t>(index)];
      const LayerPlans &plan = wide.layers[static_cast<size_t>(index)];
      const LayerState &shared = shared_layer(runner, index);
      const auto &shape = shared.shape;
      const int query_width = assistant.query_heads * shape.head_dim;
      const RopeTable &rope = *runner.rope_tables[static_cast<size_t>(shared.rope)];
      run_linear(runner, plan.qkv, nullptr, nullptr, runner.a_projected.get(), false);
      require_launch(launch_query_post(runner.a_projected.get(), w.q_norm, rope.cosine.get(),
                                       rope.sine.get(), runner.a_queries.get(), device_context,
                                       draft_index, requests, assistant.query_heads,
                                       shape.head_dim, runner.maximum_context, epsilon, stream,
                                       runner.early_keys),
                     "assistant query post-processing");
      runner.launches += 1;
      AttentionArguments attention{};
      attention.inputs_static = runner.early_keys ? 1 : 0;   // positions and slots: step inputs
      attention.queries = runner.a_queries.get();
      attention.key_cache = shared.keys();
      attention.value_cache = shared.values();
      attention.slot_stride = shared.slot_stride;
      attention.head_stride = shared.head_stride;
      attention.positions = device_context;
      attention.slots = device_slots;
      attention.scores = runner.a_scores.get();
      attention.output = runner.a_attention_out.get();
      attention.chunk_partials = runner.a_attention_partials.get<float>();
      attention.requests = requests;
      attention.depth = 1;
      attention.query_heads = assistant.query_heads;
      attention.kv_heads = shape.kv_heads;
      attention.head_dim = shape.head_dim;
      attention.capacity = shared.capacity;
      attention.window = shape.global_attention ? 0 : config.sliding_window;
      attention.draft = 1;
      // Drafting reads the target's caches and writes none.
      attention.cache_static = runner.early_keys ? 1 : 0;
      attention.max_cache_rows = std::min(longest, shared.capacity);
      attention.score_stride = runner.score_stride_global;
      attention.chunk_keys = global_chunk_keys;
      attention.chunks = attention_chunks(attention.max_cache_rows, global_chunk_keys);
      attention.stats = runner.attention_stats.get<float2>();
      attention.stats_stride = runner.stats_stride;
      attention.request_chunks = runner.request_chunks.get<int>();
      attention.maps = draft_attention_maps(runner, index);
      require_launch(attention.maps != nullptr ? launch_attention_tc(attention, stream)
                                               : launch_attention_simt(attention, stream),
                     "assistant attention");
      runner.launches += attention.maps != nullptr ? attention_tc_launches(attention) : 3;
      if (attention.chunks > 1) {
        // Key-chunk partial outputs: summed and rounded into the bf16 rows the O linear reads.
        const bool counted = attention.maps != nullptr;
        require_launch(launch_quant(nullptr, runner.a_attention_partials.get<float>(),
                                    attention.chunks,
                                    counted ? runner.request_chunks.get<int>() : nullptr, 1,
                                    rows_only(runner.a_attention_out.get()), requests,
                                    query_width, stream),
                       "assistant attention rows");
        runner.launches += 1;
      }
      const PartialSource o_source =
          run_linear(runner, plan.o, nullptr, nullptr, runner.a_linear_out.get(), true);
      require_launch(launch_post_attention_norms_quant(
                         runner.a_linear_out.get(), o_source, w.post_attention_norm, current,
                         w.pre_mlp_norm, runner.a_residual.get(),
                         rows_only(runner.a_pre_mlp.get()), requests, a_hidden, epsilon, stream),
                     "assistant post-attention norms");
      runner.launches += 1;
      run_linear(runner, plan.gate_up, nullptr, nullptr, runner.a_gate_up.get(), false);
      require_launch(launch_geglu_quant(runner.a_gate_up.get(), TailSource{},
                                        rows_only(runner.a_activated.get()), requests,
                                        assistant.intermediate_size, stream),
                     "assistant GeGLU");
      runner.launches += 1;
      const PartialSource down_source =
          run_linear(runner, plan.down, nullptr, nullptr, runner.a_linear_out.get(), true);
      const bool last = index + 1 == assistant.layer_count;
      const void *next_norm = last ? runner.assistant_weights.final_norm
                                   : runner.assistant_layers[static_cast<size_t>(index) + 1].input_norm;
      // The normed rows feed the next layer's Q linear, or (last layer) are the final hidden
      // rows; those are also quantised when the LM head runs in e4m3.
      const QuantTarget next_target = (last && head_fp8) ? target(head_word) : QuantTarget{};
      require_launch(launch_layer_output_norm_quant(
                         runner.a_linear_out.get(), down_source, w.post_mlp_norm,
                         runner.a_residual.get(), w.scalar, other, next_norm,
                         last ? runner.a_final_hidden.get() : runner.a_normed.get(), next_target,
                         requests, a_hidden, epsilon, stream),
                     "assistant layer output");
      runner.launches += 1;
      std::swap(current, other);
    }
    int *step_tokens = draft_tokens + draft_index * requests;
    if (draft_index == 0 && forced != nullptr) {
      require_cuda(cudaMemcpyAsync(step_tokens, device_forced, sizeof(int) * requests,
                                   cudaMemcpyDeviceToDevice, stream),
                   "select forced assistant first tokens");
    } else {
      if (head_fp8) {
        require_launch(launch_linear_argmax(plans.head, scales + head_word,
                                            runner.assistant_weights.token_embedding_scale, best,
                                            runner.device_error, stream),
                       "assistant LM head");
      } else {
        require_launch(launch_linear_argmax(wide.head, nullptr, nullptr, best,
                                            runner.device_error, stream),
                       "assistant LM head");
      }
      require_launch(launch_unpack_best(best, step_tokens, requests, stream), "assistant argmax");
      runner.launches += 2;
    }
    run_linear(runner, wide.post, nullptr, nullptr, runner.a_previous_hidden.get(), false);
  }
  }
  require_cuda(cudaEventRecord(runner.stop_event, stream), "record draft end");
  int *host_results = runner.host_results.get<int>();
  require_cuda(cudaMemcpyAsync(host_results, draft_tokens, sizeof(int) * depth * requests,
                               cudaMemcpyDeviceToHost, stream),
               "copy assistant proposals");
  require_cuda(cudaMemcpyAsync(host_results + depth * requests, runner.device_error, sizeof(int),
                               cudaMemcpyDeviceToHost, stream),
               "copy device error word");
  require_cuda(cudaStreamSynchronize(stream), "synchronize assistant draft");
  require_cuda(cudaEventElapsedTime(&runner.last_draft_ms, runner.start_event, runner.stop_event),
               "read draft time");
  runner.last_draft_launches = runner.launches;
  if (host_results[depth * requests] != 0) {
    const int code = host_results[depth * requests];
    cudaMemsetAsync(runner.device_error, 0, sizeof(int), stream);
    throw Failure{"a kernel wait ran out during assistant drafting (code " + std::to_string(code) +
                  ")"};
  }
  for (int draft_index = 0; draft_index < depth; ++draft_index)
    for (int row = 0; row < requests; ++row)
      proposals_out[row * depth + draft_index] = host_results[draft_index * requests + row];
}

template <typename Body> int guarded(Body &&body) {
  try {
    body();
    return 0;
  } catch (const Failure &failure) {
    set_last_error(failure.message);
    return -1;
  } catch (const std::exception &error) {
    set_last_error(error.what());
    return -2;
  }
}

} // namespace

extern "C" int carat_b200_runner_create(const carat_b200_model_config *config,
                                        const carat_b200_model_weights *weights, int batch,
                                        int maximum_context,
                                        const carat_b200_assistant_config *assistant,
                                        const carat_b200_assistant_weights *assistant_weights,
                                        carat_b200_runner **runner) {
  return guarded([&] {
    if (config == nullptr || weights == nullptr || runner == nullptr)
      throw Failure{"invalid batch model runner shape"};
    auto built = std::make_unique<carat_b200_runner>();
    build_runner(*built, *config, *weights, batch, maximum_context, assistant, assistant_weights);
    *runner = built.release();
  });
}

extern "C" void carat_b200_runner_destroy(carat_b200_runner *runner) { delete runner; }

extern "C" int carat_b200_runner_verify_greedy_proposals(
    carat_b200_runner *runner, const int *proposals, int requests, int depth,
    const int *target_first_tokens, const int *slots, const int *maximum_accepted_tokens,
    int flags, int *accepted_tokens, int *next_tokens) {
  return guarded([&] {
    if (runner == nullptr)
      throw Failure{"invalid greedy verification batch"};
    verify_step(*runner, proposals, requests, depth, target_first_tokens, slots,
                maximum_accepted_tokens, flags, false, accepted_tokens, next_tokens);
  });
}

extern "C" int carat_b200_runner_append_ragged(carat_b200_runner *runner, const int *token_ids,
                                               const int *slots, int count, int *next_tokens) {
  return guarded([&] {
    if (runner == nullptr || token_ids == nullptr || slots == nullptr || next_tokens == nullptr ||
        count <= 0 || count > runner->batch) {
      throw Failure{"invalid ragged token batch"};
    }
    std::vector<bool> seen(static_cast<size_t>(runner->batch), false);
    for (int row = 0; row < count; ++row) {
      const int slot = slots[row];
      if (slot < 0 || slot >= runner->batch || seen[static_cast<size_t>(slot)] ||
          token_ids[row] < 0 || token_ids[row] >= runner->config.vocabulary_size) {
        throw Failure{"invalid or repeated ragged slot"};
      }
      seen[static_cast<size_t>(slot)] = true;
      const int position = runner->slot_positions[static_cast<size_t>(slot)];
      if (position <= 0 || position >= runner->maximum_context)
        throw Failure{"ragged slot is empty or full"};
    }
    // One row per slot whose only proposal is the forced token: it is always accepted, its KV
    // rows are committed, the position advances by one and the prediction is the next token.
    std::vector<int> accepted(static_cast<size_t>(count));
    verify_step(*runner, token_ids, count, 1, token_ids, slots, nullptr, 0, false,
                accepted.data(), next_tokens);
  });
}

extern "C" int carat_b200_runner_draft(carat_b200_runner *runner, const int *last_tokens,
                                       const int *slots, const int *forced_first_tokens,
                                       int requests, int depth, int *proposals_out) {
  return guarded([&] {
    if (runner == nullptr)
      throw Failure{"assistant is not configured or draft batch is invalid"};
    draft_step(*runner, last_tokens, slots, forced_first_tokens, requests, depth, proposals_out);
  });
}

extern "C" int carat_b200_runner_prefill_slot_fp8(carat_b200_runner *runner, int slot,
                                                  const int *tokens, int count, int chunk,
                                                  int *next_token) {
  return guarded([&] {
    if (runner == nullptr || tokens == nullptr || count <= 0 || chunk <= 0 || chunk > 8 ||
        next_token == nullptr || slot < 0 || slot >= runner->batch) {
      throw Failure{"invalid slot prefill request"};
    }
    for (int start = 0; start < count; start += chunk) {
      const int part = std::min(chunk, count - start);
      int accepted = 0;
      int next = 0;
      verify_step(*runner, tokens + start, 1, part, tokens + start, &slot, nullptr,
                  CARAT_B200_VERIFY_ASSUME_MATCH, true, &accepted, &next);
      *next_token = next;
    }
  });
}

extern "C" int carat_b200_runner_set_bf16_weights(carat_b200_runner *runner,
                                                  const carat_b200_layer_bf16_weights *layers,
                                                  int layer_count) {
  return guarded([&] {
    if (runner == nullptr || layers == nullptr || layer_count != runner->config.layer_count)
      throw Failure{"invalid batch model runner shape"};
    for (int index = 0; index < layer_count; ++index) {
      if (layers[index].qkv == nullptr || layers[index].o == nullptr ||
          layers[index].gate_up == nullptr || layers[index].down == nullptr) {
        throw Failure{"invalid batch model runner shape"};
      }
    }
    runner->bf16_layers.assign(layers, layers + layer_count);
    runner->prefill_plans.clear();
    if (runner->p_normed.get() == nullptr) {
      const size_t rows = maximum_rows;
      runner->p_normed.allocate(rows * runner->config.hidden_size * 2);
      runner->p_pre_mlp.allocate(rows * runner->config.hidden_size * 2);
      runner->p_activated.allocate(rows * runner->config.intermediate_size * 2);
      runner->p_step_inputs.allocate(sizeof(int) * (rows + 4 * prefill_pieces), true);
      runner->p_host_inputs.allocate(sizeof(int) * (rows + 4 * prefill_pieces));
      runner->p_request_chunks.allocate(sizeof(int) * prefill_pieces, true);
    }
  });
}

extern "C" int carat_b200_runner_prefill_slots_chunks(
    carat_b200_runner *runner, const int *slots, const int *const *token_ids,
    const int *token_counts, int requests, int chunk_tokens, int *predictions,
    int *has_prediction) {
  return guarded([&] {
    if (runner == nullptr || slots == nullptr || token_ids == nullptr || token_counts == nullptr ||
        predictions == nullptr || has_prediction == nullptr || requests <= 0 ||
        requests > runner->batch || chunk_tokens <= 0) {
      throw Failure{"invalid batched chunk prefill shape"};
    }
    if (runner->bf16_layers.empty())
      throw Failure{"BF16 prefill needs the target's bf16 weights"};
    std::vector<bool> seen(static_cast<size_t>(runner->batch), false);
    std::vector<int> begin(static_cast<size_t>(requests));
    std::vector<int> end(static_cast<size_t>(requests));
    for (int request = 0; request < requests; ++request) {
      const int slot = slots[request];
      if (slot < 0 || slot >= runner->batch || seen[static_cast<size_t>(slot)] ||
          token_ids[request] == nullptr || token_counts[request] <= 0 ||
          token_counts[request] > runner->maximum_context) {
        throw Failure{"invalid batched chunk prefill request"};
      }
      seen[static_cast<size_t>(slot)] = true;
      const int position = runner->slot_positions[static_cast<size_t>(slot)];
      const int remaining = token_counts[request] - position;
      if (position < 0 || remaining <= 0)
        throw Failure{"batched chunk does not extend resident context"};
      begin[static_cast<size_t>(request)] = position;
      end[static_cast<size_t>(request)] = position + std::min(remaining, chunk_tokens);
      for (int index = position; index < end[static_cast<size_t>(request)]; ++index) {
        if (token_ids[request][index] < 0 ||
            token_ids[request][index] >= runner->config.vocabulary_size) {
          throw Failure{"batched chunk contains an invalid token id"};
        }
      }
      has_prediction[request] = 0;
      predictions[request] = -1;
    }
    // Walk the chunks in steps. A step is a list of (request, eight-token piece) entries of one
    // common depth (rows of different entries never mix in bf16, so the grouping does not change
    // any row). A request may put several consecutive pieces into one step (up to 64 entries and
    // 256 rows in all), so that the weights stream once per step instead of once per eight
    // tokens: freely while its sliding rings are still unwrapped (the rings are then linear
    // caches), up to 32 pieces past the first wrap (the sliding layers then go wave by wave, see
    // prefill_step). The two kinds do not share a step.
    constexpr int step_tokens = 8;
    const int window = runner->config.sliding_window;
    std::vector<int> cursor = begin;
    const size_t hidden_bytes = static_cast<size_t>(runner->config.hidden_size) * 2;
    for (;;) {
      std::vector<int> waiting;
      bool any_linear = false;
      for (int request = 0; request < requests; ++request) {
        if (end[static_cast<size_t>(request)] > cursor[static_cast<size_t>(request)])
          waiting.push_back(request);
      }
      if (waiting.empty())
        break;
      const auto stays_linear = [&](int request, int pieces, int depth) {
        return cursor[static_cast<size_t>(request)] + pieces * depth <= window;
      };
      for (const int request : waiting) {
        const int left = end[static_cast<size_t>(request)] - cursor[static_cast<size_t>(request)];
        any_linear = any_linear || stays_linear(request, 1, std::min(step_tokens, left));
      }
      // One kind of request per step: those whose rings stay linear, else the others.
      std::vector<int> active;
      int depth = step_tokens;
      for (const int request : waiting) {
        const int left = end[static_cast<size_t>(request)] - cursor[static_cast<size_t>(request)];
        if (any_linear && !stays_linear(request, 1, std::min(step_tokens, left)))
          continue;
        active.push_back(request);
        depth = std::min(depth, left);
      }
      if (any_linear) {
        // The common depth may have shrunk; drop whoever no longer stays linear at that depth.
        std::vector<int> kept;
        for (const int request : active) {
          if (stays_linear(request, 1, depth))
            kept.push_back(request);
        }
        active.swap(kept);
      }
      std::vector<int> pieces(active.size(), 1);
      {
        // Past the first wrap every extra piece costs three small launches per sliding layer, so
        // a slot takes at most `wave_limit` pieces there.
        constexpr int wave_limit = 32;
        const int most = std::min(prefill_pieces, maximum_rows / depth);
        int total = static_cast<int>(active.size());
        for (bool grew = true; grew && total < most;) {
          grew = false;
          for (size_t index = 0; index < active.size() && total < most; ++index) {
            const int request = active[index];
            const int left =
                end[static_cast<size_t>(request)] - cursor[static_cast<size_t>(request)];
            const bool allowed = any_linear ? stays_linear(request, pieces[index] + 1, depth)
                                            : pieces[index] < wave_limit;
            if ((pieces[index] + 1) * depth <= left && allowed) {
              ++pieces[index];
              ++total;
              grew = true;
            }
          }
        }
      }
      // Entry order: slot by slot while the rings are linear; wave by wave otherwise (wave w =
      // the w-th piece of every request that has one), because a wave is one attention launch.
      std::vector<int> step_slots;
      std::vector<int> step_ids;
      std::vector<int> last_entry(active.size(), 0);
      std::vector<int> waves;
      bool predict = false;
      if (any_linear) {
        for (size_t index = 0; index < active.size(); ++index) {
          const int request = active[index];
          const int from = cursor[static_cast<size_t>(request)];
          const int count = pieces[index] * depth;
          for (int piece = 0; piece < pieces[index]; ++piece)
            step_slots.push_back(slots[request]);
          step_ids.insert(step_ids.end(), token_ids[request] + from,
                          token_ids[request] + from + count);
          last_entry[index] = static_cast<int>(step_slots.size()) - 1;
        }
      } else {
        const int deepest = *std::max_element(pieces.begin(), pieces.end());
        for (int wave = 0; wave < deepest; ++wave) {
          int members = 0;
          for (size_t index = 0; index < active.size(); ++index) {
            if (pieces[index] <= wave)
              continue;
            const int request = active[index];
            const int from = cursor[static_cast<size_t>(request)] + wave * depth;
            step_slots.push_back(slots[request]);
            step_ids.insert(step_ids.end(), token_ids[request] + from,
                            token_ids[request] + from + depth);
            last_entry[index] = static_cast<int>(step_slots.size()) - 1;
            ++members;
          }
          waves.push_back(members);
        }
      }
      for (size_t index = 0; index < active.size(); ++index) {
        const int request = active[index];
        predict = predict || cursor[static_cast<size_t>(request)] + pieces[index] * depth ==
                                 token_counts[request];
      }
      const int entries = static_cast<int>(step_slots.size());
      std::vector<int> step_predictions(static_cast<size_t>(entries) * depth, -1);
      prefill_step(*runner, step_ids.data(), entries, depth, step_slots.data(), any_linear, waves,
                   predict, step_predictions.data());
      for (size_t index = 0; index < active.size(); ++index) {
        const int request = active[index];
        cursor[static_cast<size_t>(request)] += pieces[index] * depth;
        if (cursor[static_cast<size_t>(request)] != token_counts[request])
          continue;
        // The whole prompt is resident: its last row predicts the first generated token and its
        // final-normed hidden row goes to the drafter's table (cuda/batch_model_runner.cu:1106-1124).
        const size_t row = static_cast<size_t>(last_entry[index]) * depth + depth - 1;
        has_prediction[request] = 1;
        predictions[request] = step_predictions[row];
        require_cuda(cudaMemcpyAsync(
                         runner->hidden_by_slot.get<unsigned char>() + slots[request] * hidden_bytes,
                         runner->final_hidden.get<unsigned char>() + row * hidden_bytes,
                         hidden_bytes, cudaMemcpyDeviceToDevice, runner->stream),
                     "hand the prefill hidden row to the drafter");
      }
      require_cuda(cudaStreamSynchronize(runner->stream), "synchronize prefill hand-off");
    }
  });
}

extern "C" int carat_b200_runner_set_assistant_precision(
    carat_b200_runner *runner, int mode, const carat_b200_assistant_bf16_weights *bf16) {
  return guarded([&] {
    if (runner == nullptr || !runner->has_assistant)
      throw Failure{"assistant is not configured or draft batch is invalid"};
    if (mode != CARAT_B200_ASSISTANT_FP8_OFF && mode != CARAT_B200_ASSISTANT_FP8_LM_HEAD &&
        mode != CARAT_B200_ASSISTANT_FP8_ALL) {
      throw Failure{"CARAT_ASSISTANT_FP8_MODE must be off, lm_head or all"};
    }
    if (mode != CARAT_B200_ASSISTANT_FP8_OFF && !runner->assistant_has_fp8)
      throw Failure{"assistant FP8 mode requires quantized assistant weights"};
    if (mode != CARAT_B200_ASSISTANT_FP8_ALL) {
      if (bf16 == nullptr || bf16->layers == nullptr || bf16->token_embedding == nullptr ||
          bf16->pre_projection == nullptr || bf16->post_projection == nullptr) {
        throw Failure{"invalid assistant shape"};
      }
      for (int index = 0; index < runner->assistant.layer_count; ++index) {
        const carat_b200_assistant_bf16_layer &layer = bf16->layers[index];
        if (layer.q == nullptr || layer.o == nullptr || layer.gate_up == nullptr ||
            layer.down == nullptr) {
          throw Failure{"invalid assistant shape"};
        }
      }
      runner->assistant_bf16 = *bf16;
      runner->assistant_bf16_layers.assign(bf16->layers,
                                           bf16->layers + runner->assistant.layer_count);
      runner->assistant_bf16.layers = runner->assistant_bf16_layers.data();
      runner->draft_plans_bf16.clear();
    }
    runner->assistant_mode = mode;
  });
}

extern "C" int carat_b200_runner_use_int4_mlp(carat_b200_runner *runner,
                                              const carat_b200_int4_mlp_layer *layers,
                                              int layer_count, int group_width) {
  return guarded([&] {
    if (runner == nullptr)
      throw Failure{"invalid BF16 INT4 linear weight shape"};
    runner->verify_plans.clear();
    if (layers == nullptr) {
      runner->int4_layers.clear();
      return;
    }
    const int hidden = runner->config.hidden_size;
    const int intermediate = runner->config.intermediate_size;
    if (layer_count != runner->config.layer_count || (group_width != 128 && group_width != 256) ||
        hidden % group_width != 0 || intermediate % group_width != 0) {
      throw Failure{"invalid BF16 INT4 linear weight shape"};
    }
    for (int index = 0; index < layer_count; ++index) {
      const carat_b200_int4_mlp_layer &layer = layers[index];
      if (layer.gate_up_codes == nullptr || layer.gate_up_scales == nullptr ||
          layer.down_codes == nullptr || layer.down_scales == nullptr) {
        throw Failure{"invalid BF16 INT4 linear weight shape"};
      }
    }
    if (runner->pre_mlp.get() == nullptr) {
      runner->pre_mlp.allocate(static_cast<size_t>(128) * hidden * 2);
      runner->activated.allocate(static_cast<size_t>(128) * intermediate * 2);
      runner->unit_scale.allocate(sizeof(float));
      const float one = 1.0F;
      require_cuda(cudaMemcpy(runner->unit_scale.get(), &one, sizeof(float),
                              cudaMemcpyHostToDevice),
                   "store unit scale");
    }
    runner->int4_layers.assign(layers, layers + layer_count);
    runner->int4_group = group_width;
  });
}

extern "C" int carat_b200_runner_reset_slot(carat_b200_runner *runner, int slot) {
  return guarded([&] {
    if (runner == nullptr || slot < 0 || slot >= runner->batch)
      throw Failure{"invalid slot"};
    runner->slot_positions[static_cast<size_t>(slot)] = 0;
  });
}

extern "C" int carat_b200_runner_clone_slot(carat_b200_runner *runner, int source_slot,
                                            int destination_slot, uint64_t *copied_bytes) {
  return guarded([&] {
    if (runner == nullptr || source_slot < 0 || source_slot >= runner->batch ||
        destination_slot < 0 || destination_slot >= runner->batch ||
        source_slot == destination_slot) {
      throw Failure{"invalid cache slot clone"};
    }
    const int position = runner->slot_positions[static_cast<size_t>(source_slot)];
    if (position <= 0 || position >= runner->maximum_context)
      throw Failure{"source cache slot is empty or full"};
    uint64_t copied = 0;
    for (const LayerState &layer : runner->layers) {
      // The first min(position, capacity) physical rows of every KV head, keys and values.
      const int resident = std::min(position, layer.capacity);
      const size_t row_bytes = static_cast<size_t>(resident) * layer.shape.head_dim * 2;
      const size_t pitch = static_cast<size_t>(layer.head_stride) * 2;
      for (unsigned char *base : {static_cast<unsigned char *>(layer.keys()),
                                  static_cast<unsigned char *>(layer.values())}) {
        require_cuda(cudaMemcpy2DAsync(
                         base + static_cast<size_t>(destination_slot) * layer.slot_stride * 2,
                         pitch, base + static_cast<size_t>(source_slot) * layer.slot_stride * 2,
                         pitch, row_bytes, static_cast<size_t>(layer.shape.kv_heads),
                         cudaMemcpyDeviceToDevice, runner->stream),
                     "clone slot cache");
        copied += row_bytes * static_cast<uint64_t>(layer.shape.kv_heads);
      }
    }
    const size_t hidden_bytes = static_cast<size_t>(runner->config.hidden_size) * 2;
    require_cuda(cudaMemcpyAsync(
                     runner->hidden_by_slot.get<unsigned char>() + destination_slot * hidden_bytes,
                     runner->hidden_by_slot.get<unsigned char>() + source_slot * hidden_bytes,
                     hidden_bytes, cudaMemcpyDeviceToDevice, runner->stream),
                 "clone slot target hidden state");
    runner->slot_positions[static_cast<size_t>(destination_slot)] = position;
    require_cuda(cudaStreamSynchronize(runner->stream), "synchronize slot cache clone");
    if (copied_bytes != nullptr)
      *copied_bytes = copied;
  });
}

extern "C" int carat_b200_runner_seed_empty_cache_for_benchmark(carat_b200_runner *runner,
                                                                int position) {
  return guarded([&] {
    if (runner == nullptr || position < 0 || position >= runner->maximum_context)
      throw Failure{"invalid benchmark cache position"};
    for (LayerState &layer : runner->layers)
      require_cuda(cudaMemsetAsync(layer.kv.get(), 0, layer.kv.bytes(), runner->stream),
                   "clear KV arena");
    std::fill(runner->slot_positions.begin(), runner->slot_positions.end(), position);
    require_cuda(cudaStreamSynchronize(runner->stream), "seed benchmark cache");
  });
}

extern "C" int carat_b200_runner_seed_slot_positions(carat_b200_runner *runner,
                                                     const int *positions) {
  return guarded([&] {
    if (runner == nullptr || positions == nullptr)
      throw Failure{"invalid benchmark cache position"};
    for (int slot = 0; slot < runner->batch; ++slot) {
      if (positions[slot] < 0 || positions[slot] >= runner->maximum_context)
        throw Failure{"invalid benchmark cache position"};
    }
    for (LayerState &layer : runner->layers)
      require_cuda(cudaMemsetAsync(layer.kv.get(), 0, layer.kv.bytes(), runner->stream),
                   "clear KV arena");
    runner->slot_positions.assign(positions, positions + runner->batch);
    require_cuda(cudaStreamSynchronize(runner->stream), "seed benchmark cache");
  });
}

extern "C" int carat_b200_runner_batch(const carat_b200_runner *runner) {
  return runner == nullptr ? 0 : runner->batch;
}

extern "C" int carat_b200_runner_slot_position(const carat_b200_runner *runner, int slot,
                                               int *position) {
  return guarded([&] {
    if (runner == nullptr || position == nullptr || slot < 0 || slot >= runner->batch)
      throw Failure{"invalid slot"};
    *position = runner->slot_positions[static_cast<size_t>(slot)];
  });
}

extern "C" int carat_b200_runner_has_assistant(const carat_b200_runner *runner) {
  return runner != nullptr && runner->has_assistant ? 1 : 0;
}

extern "C" int carat_b200_runner_last_predictions(carat_b200_runner *runner, int *predictions,
                                                  int count) {
  return guarded([&] {
    if (runner == nullptr || predictions == nullptr || count <= 0 || count > runner->last_rows)
      throw Failure{"no predictions of that size are available"};
    std::memcpy(predictions, runner->last_predictions.data(),
                sizeof(int) * static_cast<size_t>(count));
  });
}

extern "C" int carat_b200_runner_device_pointer(carat_b200_runner *runner, int which, int layer,
                                                void **pointer, size_t *bytes) {
  return guarded([&] {
    if (runner == nullptr || pointer == nullptr || bytes == nullptr)
      throw Failure{"invalid inspection request"};
    if (which == 0 || which == 1) {
      if (layer < 0 || layer >= runner->config.layer_count)
        throw Failure{"invalid layer"};
      const LayerState &state = runner->layers[static_cast<size_t>(layer)];
      *pointer = which == 0 ? state.keys() : state.values();
      *bytes = static_cast<size_t>(runner->batch) * state.slot_stride * 2;
    } else if (which == 2) {
      *pointer = runner->hidden_by_slot.get();
      *bytes = static_cast<size_t>(runner->batch) * runner->config.hidden_size * 2;
    } else if (which == 3) {
      *pointer = runner->final_hidden.get();
      *bytes = static_cast<size_t>(runner->last_rows) * runner->config.hidden_size * 2;
    } else if (which >= 6 && which <= 12) {
      const DeviceBuffer *buffers[] = {&runner->packed,   &runner->queries,   &runner->attention_out,
                                       &runner->residual, &runner->gate_up,   &runner->quantized,
                                       &runner->scales};
      *pointer = buffers[which - 6]->get();
      *bytes = buffers[which - 6]->bytes();
    } else if (which == 4 && runner->has_assistant) {
      *pointer = runner->a_final_hidden.get();
      *bytes = runner->a_final_hidden.bytes();
    } else if (which == 5 && runner->has_assistant) {
      *pointer = runner->a_previous_hidden.get();
      *bytes = runner->a_previous_hidden.bytes();
    } else {
      throw Failure{"invalid inspection request"};
    }
  });
}

extern "C" int carat_b200_runner_read(carat_b200_runner *runner, int which, int layer,
                                      size_t offset, void *destination, size_t bytes) {
  void *base = nullptr;
  size_t available = 0;
  const int status = carat_b200_runner_device_pointer(runner, which, layer, &base, &available);
  if (status != 0)
    return status;
  return guarded([&] {
    if (destination == nullptr || offset + bytes > available)
      throw Failure{"inspection read exceeds the runner's buffer"};
    require_cuda(cudaStreamSynchronize(runner->stream), "drain runner stream");
    require_cuda(cudaMemcpy(destination, static_cast<unsigned char *>(base) + offset, bytes,
                            cudaMemcpyDefault),
                 "read runner buffer");
  });
}

extern "C" int carat_b200_runner_write(carat_b200_runner *runner, int which, int layer,
                                       size_t offset, const void *source, size_t bytes) {
  void *base = nullptr;
  size_t available = 0;
  const int status = carat_b200_runner_device_pointer(runner, which, layer, &base, &available);
  if (status != 0)
    return status;
  return guarded([&] {
    if (which < 0 || which > 2)
      throw Failure{"only the KV caches and the hidden-by-slot table can be written"};
    if (source == nullptr || offset + bytes > available)
      throw Failure{"write exceeds the runner's buffer"};
    require_cuda(cudaStreamSynchronize(runner->stream), "drain runner stream");
    require_cuda(cudaMemcpy(static_cast<unsigned char *>(base) + offset, source, bytes,
                            cudaMemcpyDefault),
                 "write runner buffer");
  });
}

extern "C" int carat_b200_runner_last_device_ms(const carat_b200_runner *runner, float *verify_ms,
                                                float *draft_ms) {
  if (runner == nullptr)
    return -1;
  if (verify_ms != nullptr)
    *verify_ms = runner->last_verify_ms;
  if (draft_ms != nullptr)
    *draft_ms = runner->last_draft_ms;
  return 0;
}

extern "C" int carat_b200_runner_last_launches(const carat_b200_runner *runner,
                                               int *verify_launches, int *draft_launches) {
  if (runner == nullptr)
    return -1;
  if (verify_launches != nullptr)
    *verify_launches = runner->last_verify_launches;
  if (draft_launches != nullptr)
    *draft_launches = runner->last_draft_launches;
  return 0;
}
