// Drop-in implementation of carat::Gemma4BatchModelRunner (include/carat/batch_model_runner.h in
// the Carat tree) over libcarat_b200's C ABI, for the speculative-decoding path:
// verify_greedy_proposals, draft_four, append_ragged, clone_slot, reset_slot,
// seed_empty_cache_for_benchmark and the accessors. Compile it inside the Carat build in place of cuda/batch_model_runner.cu and
// link libcarat_b200.so; the scheduler (src/native_runtime_main.cpp) is unchanged.
//
// Prompt prefill (prefill_slot, prefill_slot_from_prefix, prefill_slot_chunk,
// prefill_slots_chunks, prefill_slots_suffix) runs in BF16 on the bf16 matrices of the
// DeviceWeightArena, as in the reference (cuda/batch_model_runner.cu:1274-1275).
// prefill_slots_suffix_layer_slice finishes the whole suffix in its first call (it never leaves
// layer slices pending), and the lock-step `append` is append_ragged over every slot.
#include "carat/batch_model_runner.h"
#include "carat/device_weights.h"
#include "carat/gemma4_config.h"

#include "carat_b200.h"

#include <cstdlib>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

namespace carat {

namespace {

void check(int status) {
  // The library reports the reference's own exception texts.
  if (status != 0)
    throw std::runtime_error(carat_b200_last_error());
}

// Norm vectors only: a drafter that runs in bf16 may come without an Fp8WeightArena.
carat_b200_layer_weights norm_weights(const DeviceWeightArena &bf16, const std::string &prefix) {
  carat_b200_layer_weights weights{};
  weights.input_norm = bf16.at(prefix + "input_norm");
  weights.q_norm = bf16.at(prefix + "q_norm");
  weights.post_attention_norm = bf16.at(prefix + "post_attention_norm");
  weights.pre_mlp_norm = bf16.at(prefix + "pre_mlp_norm");
  weights.post_mlp_norm = bf16.at(prefix + "post_mlp_norm");
  weights.scalar = bf16.at(prefix + "scalar");
  return weights;
}

// CARAT_ASSISTANT_FP8_MODE, read where the reference reads it (cuda/assistant_runner.cu:31-43).
int assistant_fp8_mode(const Fp8WeightArena *weights) {
  const char *configured = std::getenv("CARAT_ASSISTANT_FP8_MODE");
  const std::string mode = configured == nullptr ? "off" : configured;
  if (mode == "off")
    return CARAT_B200_ASSISTANT_FP8_OFF;
  if (weights == nullptr)
    throw std::runtime_error("assistant FP8 mode requires quantized assistant weights");
  if (mode == "lm_head")
    return CARAT_B200_ASSISTANT_FP8_LM_HEAD;
  if (mode == "all")
    return CARAT_B200_ASSISTANT_FP8_ALL;
  throw std::runtime_error("CARAT_ASSISTANT_FP8_MODE must be off, lm_head or all");
}

carat_b200_layer_weights layer_weights(const DeviceWeightArena &bf16, const Fp8WeightArena &fp8,
                                       const std::string &prefix, bool assistant) {
  const std::string projection = prefix + (assistant ? "q" : "qkv");
  return carat_b200_layer_weights{
      bf16.at(prefix + "input_norm"),
      bf16.at(prefix + "q_norm"),
      assistant ? nullptr : bf16.at(prefix + "k_norm"),
      fp8.at(projection),
      fp8.scale(projection),
      fp8.at(prefix + "o"),
      fp8.scale(prefix + "o"),
      bf16.at(prefix + "post_attention_norm"),
      bf16.at(prefix + "pre_mlp_norm"),
      fp8.at(prefix + "gate_up"),
      fp8.scale(prefix + "gate_up"),
      fp8.at(prefix + "down"),
      fp8.scale(prefix + "down"),
      bf16.at(prefix + "post_mlp_norm"),
      bf16.at(prefix + "scalar")};
}

} // namespace

struct Gemma4BatchModelRunner::Implementation {
  carat_b200_runner *handle{nullptr};
  int batch{0};
  int maximum_context{0};
  int current_position{0};   // the lock-step position `append` and the benchmark seed keep

  // One prefill chunk per listed slot through the C ABI; an entry is set when the prompt is whole.
  std::vector<std::optional<int>> chunks(const std::vector<int> &slots,
                                         const std::vector<const std::vector<int> *> &token_ids,
                                         int chunk_tokens) {
    std::vector<const int *> pointers;
    std::vector<int> counts;
    for (const std::vector<int> *prompt : token_ids) {
      pointers.push_back(prompt != nullptr ? prompt->data() : nullptr);
      counts.push_back(prompt != nullptr ? static_cast<int>(prompt->size()) : 0);
    }
    std::vector<int> predictions(slots.size(), -1);
    std::vector<int> has_prediction(slots.size(), 0);
    check(carat_b200_runner_prefill_slots_chunks(handle, slots.data(), pointers.data(),
                                                 counts.data(), static_cast<int>(slots.size()),
                                                 chunk_tokens, predictions.data(),
                                                 has_prediction.data()));
    std::vector<std::optional<int>> result(slots.size());
    for (std::size_t request = 0; request < slots.size(); ++request) {
      if (has_prediction[request] != 0)
        result[request] = predictions[request];
    }
    return result;
  }
};

Gemma4BatchModelRunner::Gemma4BatchModelRunner(const Gemma4Config &config,
                                               const DeviceWeightArena &weights, int batch,
                                               int maximum_context,
                                               const Fp8WeightArena *fp8_weights,
                                               const DeviceWeightArena *assistant_weights,
                                               const Fp8WeightArena *assistant_fp8_weights)
    : implementation_(std::make_unique<Implementation>()) {
  if (fp8_weights == nullptr)
    throw std::runtime_error("carat-b200 runs the FP8 path: an Fp8WeightArena is required");
  std::vector<carat_b200_layer_shape> shapes;
  std::vector<carat_b200_layer_weights> layers;
  for (std::size_t index = 0; index < config.layers.size(); ++index) {
    const Gemma4LayerConfig &layer = config.layers[index];
    shapes.push_back({layer.attention == AttentionKind::global ? 1 : 0,
                      static_cast<int32_t>(layer.query_heads), static_cast<int32_t>(layer.kv_heads),
                      static_cast<int32_t>(layer.head_dimension),
                      static_cast<float>(layer.rope_theta), layer.key_equals_value ? 1 : 0});
    layers.push_back(layer_weights(weights, *fp8_weights,
                                   "layer." + std::to_string(index) + ".", false));
  }
  const carat_b200_model_config model{
      static_cast<int32_t>(config.hidden_size),     static_cast<int32_t>(config.intermediate_size),
      static_cast<int32_t>(config.vocabulary_size), static_cast<int32_t>(config.sliding_window),
      static_cast<float>(config.rms_norm_epsilon),  static_cast<int32_t>(shapes.size()),
      shapes.data()};
  const carat_b200_model_weights model_weights{
      weights.at("token_embedding"), fp8_weights->at("token_embedding"),
      fp8_weights->scale("token_embedding"), weights.at("final_norm"), layers.data()};

  // The drafter's shape is fixed in the reference (cuda/assistant_runner.cu:22-27,166-170).
  const int32_t assistant_layer_kinds[4] = {0, 0, 0, 1};
  const carat_b200_assistant_config assistant_config{1024, 8192, 32, 4, assistant_layer_kinds,
                                                     1.0e-6F};
  std::vector<carat_b200_layer_weights> assistant_layers;
  carat_b200_assistant_weights assistant{};
  const bool with_assistant = assistant_weights != nullptr;
  int assistant_mode = CARAT_B200_ASSISTANT_FP8_OFF;
  if (with_assistant) {
    assistant_mode = assistant_fp8_mode(assistant_fp8_weights);
    for (int index = 0; index < 4; ++index) {
      const std::string prefix = "layer." + std::to_string(index) + ".";
      assistant_layers.push_back(
          assistant_fp8_weights != nullptr
              ? layer_weights(*assistant_weights, *assistant_fp8_weights, prefix, true)
              : norm_weights(*assistant_weights, prefix));
    }
    assistant.final_norm = assistant_weights->at("final_norm");
    assistant.layers = assistant_layers.data();
    if (assistant_fp8_weights != nullptr) {
      assistant.token_embedding = assistant_fp8_weights->at("token_embedding");
      assistant.token_embedding_scale = assistant_fp8_weights->scale("token_embedding");
      assistant.pre_projection = assistant_fp8_weights->at("pre_projection");
      assistant.pre_projection_scale = assistant_fp8_weights->scale("pre_projection");
      assistant.post_projection = assistant_fp8_weights->at("post_projection");
      assistant.post_projection_scale = assistant_fp8_weights->scale("post_projection");
    }
  }
  check(carat_b200_runner_create(&model, &model_weights, batch, maximum_context,
                                 with_assistant ? &assistant_config : nullptr,
                                 with_assistant ? &assistant : nullptr,
                                 &implementation_->handle));
  implementation_->batch = batch;
  implementation_->maximum_context = maximum_context;
  {
    // BF16 prefill reads the target's bf16 matrices straight from the DeviceWeightArena.
    std::vector<carat_b200_layer_bf16_weights> bf16;
    for (std::size_t index = 0; index < config.layers.size(); ++index) {
      const std::string prefix = "layer." + std::to_string(index) + ".";
      bf16.push_back({weights.at(prefix + "qkv"), weights.at(prefix + "o"),
                      weights.at(prefix + "gate_up"), weights.at(prefix + "down")});
    }
    check(carat_b200_runner_set_bf16_weights(implementation_->handle, bf16.data(),
                                             static_cast<int>(bf16.size())));
  }
  if (with_assistant) {
    // The drafter's precision follows the reference's switch; its default runs every drafter
    // linear on the bf16 matrices of the assistant's DeviceWeightArena.
    std::vector<carat_b200_assistant_bf16_layer> bf16_layers;
    carat_b200_assistant_bf16_weights bf16{};
    if (assistant_mode != CARAT_B200_ASSISTANT_FP8_ALL) {
      for (int index = 0; index < 4; ++index) {
        const std::string prefix = "layer." + std::to_string(index) + ".";
        bf16_layers.push_back({assistant_weights->at(prefix + "q"),
                               assistant_weights->at(prefix + "o"),
                               assistant_weights->at(prefix + "gate_up"),
                               assistant_weights->at(prefix + "down")});
      }
      bf16.token_embedding = assistant_weights->at("token_embedding");
      bf16.pre_projection = assistant_weights->at("pre_projection");
      bf16.post_projection = assistant_weights->at("post_projection");
      bf16.layers = bf16_layers.data();
    }
    check(carat_b200_runner_set_assistant_precision(
        implementation_->handle, assistant_mode,
        assistant_mode != CARAT_B200_ASSISTANT_FP8_ALL ? &bf16 : nullptr));
  }
}

Gemma4BatchModelRunner::~Gemma4BatchModelRunner() {
  if (implementation_ != nullptr && implementation_->handle != nullptr)
    carat_b200_runner_destroy(implementation_->handle);
}

GreedyVerificationResult Gemma4BatchModelRunner::verify_greedy_proposals(
    const std::vector<std::vector<int>> &proposals, const std::vector<int> &target_first_tokens,
    const std::vector<int> &slots, const std::vector<int> &maximum_accepted_tokens) {
  const int requests = static_cast<int>(proposals.size());
  const int depth = requests > 0 ? static_cast<int>(proposals.front().size()) : 0;
  if (requests == 0 || target_first_tokens.size() != proposals.size() ||
      slots.size() != proposals.size()) {
    throw std::runtime_error("invalid greedy verification batch");
  }
  if (!maximum_accepted_tokens.empty() && maximum_accepted_tokens.size() != proposals.size())
    throw std::runtime_error("speculative acceptance caps do not match request count");
  std::vector<int> flat;
  flat.reserve(static_cast<std::size_t>(requests) * depth);
  for (const std::vector<int> &row : proposals) {
    if (static_cast<int>(row.size()) != depth)
      throw std::runtime_error("invalid or repeated speculative slot");
    flat.insert(flat.end(), row.begin(), row.end());
  }
  GreedyVerificationResult result;
  result.accepted_tokens.resize(proposals.size());
  result.next_tokens.resize(proposals.size());
  check(carat_b200_runner_verify_greedy_proposals(
      implementation_->handle, flat.data(), requests, depth, target_first_tokens.data(),
      slots.data(), maximum_accepted_tokens.empty() ? nullptr : maximum_accepted_tokens.data(), 0,
      result.accepted_tokens.data(), result.next_tokens.data()));
  return result;
}

bool Gemma4BatchModelRunner::has_assistant() const {
  return carat_b200_runner_has_assistant(implementation_->handle) != 0;
}

std::vector<std::vector<int>>
Gemma4BatchModelRunner::draft_four(const std::vector<int> &last_tokens,
                                   const std::vector<int> &slots,
                                   const std::vector<int> &forced_first_tokens, int depth) {
  if (last_tokens.empty() || slots.size() != last_tokens.size() || depth <= 0)
    throw std::runtime_error("assistant is not configured or draft batch is invalid");
  if (!forced_first_tokens.empty() && forced_first_tokens.size() != last_tokens.size())
    throw std::runtime_error("forced assistant first tokens do not match draft batch");
  std::vector<int> flat(last_tokens.size() * static_cast<std::size_t>(depth));
  check(carat_b200_runner_draft(implementation_->handle, last_tokens.data(), slots.data(),
                                forced_first_tokens.empty() ? nullptr : forced_first_tokens.data(),
                                static_cast<int>(last_tokens.size()), depth, flat.data()));
  std::vector<std::vector<int>> rows(last_tokens.size());
  for (std::size_t row = 0; row < rows.size(); ++row)
    rows[row].assign(flat.begin() + static_cast<std::ptrdiff_t>(row * depth),
                     flat.begin() + static_cast<std::ptrdiff_t>((row + 1) * depth));
  return rows;
}

std::vector<int> Gemma4BatchModelRunner::append_ragged(const std::vector<int> &token_ids,
                                                       const std::vector<int> &slots) {
  if (token_ids.empty() || slots.size() != token_ids.size())
    throw std::runtime_error("invalid ragged token batch");
  std::vector<int> next(token_ids.size());
  check(carat_b200_runner_append_ragged(implementation_->handle, token_ids.data(), slots.data(),
                                        static_cast<int>(token_ids.size()), next.data()));
  return next;
}

int Gemma4BatchModelRunner::prefill_slot(int slot, const std::vector<int> &token_ids,
                                         int chunk_tokens) {
  reset_slot(slot);
  return prefill_slot_from_prefix(slot, token_ids, 0, chunk_tokens);
}

int Gemma4BatchModelRunner::prefill_slot_from_prefix(int slot, const std::vector<int> &token_ids,
                                                     int cached_prefix_tokens, int chunk_tokens) {
  if (slot < 0 || slot >= implementation_->batch || token_ids.empty() ||
      token_ids.size() > static_cast<std::size_t>(implementation_->maximum_context) ||
      chunk_tokens <= 0 || chunk_tokens > implementation_->maximum_context ||
      cached_prefix_tokens < 0 || cached_prefix_tokens >= static_cast<int>(token_ids.size()) ||
      slot_position(slot) != cached_prefix_tokens) {
    throw std::runtime_error("invalid slot prefill shape");
  }
  std::optional<int> prediction;
  while (!prediction)
    prediction = prefill_slot_chunk(slot, token_ids, chunk_tokens);
  return *prediction;
}

std::optional<int> Gemma4BatchModelRunner::prefill_slot_chunk(int slot,
                                                              const std::vector<int> &token_ids,
                                                              int chunk_tokens) {
  if (slot < 0 || slot >= implementation_->batch || token_ids.empty() ||
      token_ids.size() > static_cast<std::size_t>(implementation_->maximum_context) ||
      chunk_tokens <= 0 || chunk_tokens > implementation_->maximum_context) {
    throw std::runtime_error("invalid slot prefill chunk shape");
  }
  if (slot_position(slot) >= static_cast<int>(token_ids.size()))
    throw std::runtime_error("slot prefill chunk does not extend resident context");
  return implementation_->chunks({slot}, {&token_ids}, chunk_tokens).front();
}

std::vector<std::optional<int>>
Gemma4BatchModelRunner::prefill_slots_chunks(const std::vector<int> &slots,
                                             const std::vector<const std::vector<int> *> &token_ids,
                                             int chunk_tokens) {
  if (slots.empty() || token_ids.size() != slots.size() || chunk_tokens <= 0)
    throw std::runtime_error("invalid batched chunk prefill shape");
  return implementation_->chunks(slots, token_ids, chunk_tokens);
}

std::vector<int>
Gemma4BatchModelRunner::prefill_slots_suffix(const std::vector<int> &slots,
                                             const std::vector<const std::vector<int> *> &token_ids) {
  if (slots.empty() || token_ids.size() != slots.size())
    throw std::runtime_error("invalid batched suffix prefill shape");
  std::vector<int> result;
  for (const std::optional<int> &entry :
       implementation_->chunks(slots, token_ids, implementation_->maximum_context)) {
    result.push_back(entry.value());   // one chunk as long as the context holds any suffix
  }
  return result;
}

LayerSlicedSuffixPrefillResult Gemma4BatchModelRunner::prefill_slots_suffix_layer_slice(
    const std::vector<int> &slots, const std::vector<const std::vector<int> *> &token_ids, int) {
  // All layers in this call: the result is complete at once and nothing stays pending.
  LayerSlicedSuffixPrefillResult result;
  result.predictions = prefill_slots_suffix(slots, token_ids);
  result.complete = true;
  return result;
}

void Gemma4BatchModelRunner::abort_suffix_layer_slices() {}
bool Gemma4BatchModelRunner::has_suffix_layer_slices() const { return false; }

std::vector<int> Gemma4BatchModelRunner::append(const std::vector<int> &token_ids) {
  if (token_ids.size() != static_cast<std::size_t>(implementation_->batch))
    throw std::runtime_error("token batch has the wrong size");
  if (implementation_->current_position >= implementation_->maximum_context)
    throw std::runtime_error("batch context is full");
  std::vector<int> slots(token_ids.size());
  for (std::size_t slot = 0; slot < slots.size(); ++slot)
    slots[slot] = static_cast<int>(slot);
  std::vector<int> next = append_ragged(token_ids, slots);
  ++implementation_->current_position;
  return next;
}

std::uint64_t Gemma4BatchModelRunner::clone_slot(int source_slot, int destination_slot) {
  std::uint64_t copied = 0;
  check(carat_b200_runner_clone_slot(implementation_->handle, source_slot, destination_slot,
                                     &copied));
  return copied;
}

void Gemma4BatchModelRunner::reset_slot(int slot) {
  check(carat_b200_runner_reset_slot(implementation_->handle, slot));
}

void Gemma4BatchModelRunner::seed_empty_cache_for_benchmark(int position) {
  check(carat_b200_runner_seed_empty_cache_for_benchmark(implementation_->handle, position));
  implementation_->current_position = position;
}

int Gemma4BatchModelRunner::batch() const { return implementation_->batch; }

int Gemma4BatchModelRunner::slot_position(int slot) const {
  int position = 0;
  check(carat_b200_runner_slot_position(implementation_->handle, slot, &position));
  return position;
}

int Gemma4BatchModelRunner::position() const { return implementation_->current_position; }

} // namespace carat
