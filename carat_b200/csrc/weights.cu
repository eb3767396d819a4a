// Weight pipeline: safetensors shards -> execution segments in one device arena -> e4m3 arena.
//
// Replaces, for the path's needs, src/safetensors.cpp (header parsing, shard index),
// src/weight_plan.cpp:37-128 (segment names, fused qkv / gate_up row stacking, 256-byte aligned
// arena offsets, the reference's validation and its error texts) and
// cuda/device_weights.cu:100-263 (upload, Fp8WeightArena::quantize with tensor scaling).
//
// Layout and flow are chosen for the B200 box rather than taken from the reference: every source
// tensor is read with pread() straight into one of two pinned staging buffers and copied to its
// place in the arena with cudaMemcpyAsync on a copy stream while the next read runs, and each
// two-dimensional segment is quantised on the device as soon as its last source has landed, on a
// second stream, so disk, PCIe and the quantiser overlap.
#include "../../include/carat_b200.h"
#include "context.cuh"
#include "int4_linear.cuh"
#include "row_ops.cuh"

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cctype>
#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

using namespace carat_b200;

namespace {

struct Failure {
  std::string message;
};

// ---------------------------------------------------------------- a JSON reader for two schemas
// Only what a safetensors header and a shard index need: objects, arrays, strings and
// non-negative integers; other scalars are skipped.
class JsonCursor {
public:
  explicit JsonCursor(const std::string &text) : text_(text) {}

  void skip_space() {
    while (position_ < text_.size() && std::isspace(static_cast<unsigned char>(text_[position_])))
      ++position_;
  }
  bool take(char expected) {
    skip_space();
    if (position_ < text_.size() && text_[position_] == expected) {
      ++position_;
      return true;
    }
    return false;
  }
  void expect(char expected) {
    if (!take(expected))
      throw Failure{std::string("malformed JSON: expected '") + expected + "'"};
  }
  char peek() {
    skip_space();
    return position_ < text_.size() ? text_[position_] : '\0';
  }
  std::string string() {
    expect('"');
    std::string value;
    while (position_ < text_.size() && text_[position_] != '"') {
      char character = text_[position_++];
      if (character == '\\' && position_ < text_.size()) {
        const char escaped = text_[position_++];
        switch (escaped) {
        case 'n': character = '\n'; break;
        case 't': character = '\t'; break;
        case 'u': position_ += 4; character = '?'; break;
        default: character = escaped; break;
        }
      }
      value.push_back(character);
    }
    expect('"');
    return value;
  }
  std::uint64_t integer() {
    skip_space();
    if (position_ >= text_.size() || !std::isdigit(static_cast<unsigned char>(text_[position_])))
      throw Failure{"malformed JSON: expected a non-negative integer"};
    std::uint64_t value = 0;
    while (position_ < text_.size() && std::isdigit(static_cast<unsigned char>(text_[position_])))
      value = value * 10 + static_cast<std::uint64_t>(text_[position_++] - '0');
    return value;
  }
  // Skips any value (used for __metadata__ and fields this reader has no use for).
  void skip_value() {
    const char next = peek();
    if (next == '"') {
      string();
    } else if (next == '{') {
      expect('{');
      if (!take('}')) {
        do {
          string();
          expect(':');
          skip_value();
        } while (take(','));
        expect('}');
      }
    } else if (next == '[') {
      expect('[');
      if (!take(']')) {
        do {
          skip_value();
        } while (take(','));
        expect(']');
      }
    } else {
      while (position_ < text_.size() && text_[position_] != ',' && text_[position_] != '}' &&
             text_[position_] != ']') {
        ++position_;
      }
    }
  }

private:
  const std::string &text_;
  size_t position_{0};
};

// ---------------------------------------------------------------- safetensors
struct Tensor {
  std::string shard_path;
  std::string dtype;
  std::vector<std::uint64_t> shape;
  std::uint64_t file_offset{0};
  std::uint64_t byte_size{0};
};

using TensorTable = std::map<std::string, Tensor, std::less<>>;

std::string read_file(const std::string &path) {
  const int descriptor = open(path.c_str(), O_RDONLY);
  if (descriptor < 0)
    throw Failure{"cannot open " + path};
  std::string text;
  char buffer[65536];
  ssize_t got = 0;
  while ((got = read(descriptor, buffer, sizeof(buffer))) > 0)
    text.append(buffer, static_cast<size_t>(got));
  close(descriptor);
  return text;
}

bool file_exists(const std::string &path) {
  struct stat info {};
  return stat(path.c_str(), &info) == 0;
}

std::uint64_t dtype_bytes(const std::string &dtype) {
  if (dtype == "BOOL" || dtype == "U8" || dtype == "I8")
    return 1;
  if (dtype == "U16" || dtype == "I16" || dtype == "F16" || dtype == "BF16")
    return 2;
  if (dtype == "U32" || dtype == "I32" || dtype == "F32")
    return 4;
  if (dtype == "U64" || dtype == "I64" || dtype == "F64")
    return 8;
  throw Failure{"unsupported safetensors dtype: " + dtype};
}

// One .safetensors file: 8-byte little-endian header length, a JSON header, then the data.
TensorTable open_safetensors(const std::string &path) {
  const int descriptor = open(path.c_str(), O_RDONLY);
  if (descriptor < 0)
    throw Failure{"cannot open safetensors file " + path};
  struct stat info {};
  fstat(descriptor, &info);
  const std::uint64_t file_bytes = static_cast<std::uint64_t>(info.st_size);
  unsigned char prefix[8];
  if (pread(descriptor, prefix, 8, 0) != 8) {
    close(descriptor);
    throw Failure{"cannot read safetensors header size from " + path};
  }
  std::uint64_t header_bytes = 0;
  for (int index = 0; index < 8; ++index)
    header_bytes |= static_cast<std::uint64_t>(prefix[index]) << (8 * index);
  if (header_bytes == 0 || header_bytes > file_bytes - 8 || header_bytes > (1ULL << 30)) {
    close(descriptor);
    throw Failure{"invalid safetensors header size in " + path};
  }
  std::string header(header_bytes, '\0');
  const ssize_t got = pread(descriptor, header.data(), header_bytes, 8);
  close(descriptor);
  if (got != static_cast<ssize_t>(header_bytes))
    throw Failure{"cannot read safetensors header from " + path};
  const std::uint64_t data_start = 8 + header_bytes;

  TensorTable tensors;
  JsonCursor cursor(header);
  cursor.expect('{');
  if (cursor.take('}'))
    return tensors;
  do {
    const std::string name = cursor.string();
    cursor.expect(':');
    if (name == "__metadata__") {
      cursor.skip_value();
      continue;
    }
    Tensor tensor;
    tensor.shard_path = path;
    std::uint64_t begin = 0;
    std::uint64_t end = 0;
    bool has_offsets = false;
    cursor.expect('{');
    do {
      const std::string field = cursor.string();
      cursor.expect(':');
      if (field == "dtype") {
        tensor.dtype = cursor.string();
      } else if (field == "shape") {
        cursor.expect('[');
        if (!cursor.take(']')) {
          do {
            tensor.shape.push_back(cursor.integer());
          } while (cursor.take(','));
          cursor.expect(']');
        }
      } else if (field == "data_offsets") {
        cursor.expect('[');
        begin = cursor.integer();
        cursor.expect(',');
        end = cursor.integer();
        cursor.expect(']');
        has_offsets = true;
      } else {
        cursor.skip_value();
      }
    } while (cursor.take(','));
    cursor.expect('}');
    if (!has_offsets || end < begin)
      throw Failure{"invalid offsets for tensor " + name};
    if (data_start + end > file_bytes)
      throw Failure{"out-of-range tensor " + name};
    std::uint64_t elements = 1;
    for (const std::uint64_t extent : tensor.shape)
      elements *= extent;
    if (elements * dtype_bytes(tensor.dtype) != end - begin)
      throw Failure{"byte-size mismatch for tensor " + name};
    tensor.file_offset = data_start + begin;
    tensor.byte_size = end - begin;
    tensors.emplace(name, std::move(tensor));
  } while (cursor.take(','));
  return tensors;
}

// A model directory: model.safetensors.index.json naming shards, or a single model.safetensors.
TensorTable open_model_directory(const std::string &directory) {
  const std::string index_path = directory + "/model.safetensors.index.json";
  if (!file_exists(index_path))
    return open_safetensors(directory + "/model.safetensors");
  const std::string index = read_file(index_path);
  std::map<std::string, std::string> weight_map;
  JsonCursor cursor(index);
  cursor.expect('{');
  do {
    const std::string field = cursor.string();
    cursor.expect(':');
    if (field != "weight_map") {
      cursor.skip_value();
      continue;
    }
    cursor.expect('{');
    if (!cursor.take('}')) {
      do {
        const std::string name = cursor.string();
        cursor.expect(':');
        weight_map[name] = cursor.string();
      } while (cursor.take(','));
      cursor.expect('}');
    }
  } while (cursor.take(','));
  std::map<std::string, TensorTable> shards;
  for (const auto &entry : weight_map) {
    if (shards.find(entry.second) == shards.end())
      shards.emplace(entry.second, open_safetensors(directory + "/" + entry.second));
  }
  TensorTable tensors;
  for (const auto &[name, shard] : weight_map) {
    const TensorTable &table = shards.at(shard);
    const auto found = table.find(name);
    if (found == table.end())
      throw Failure{"missing tensor " + name};
    tensors.emplace(name, found->second);
  }
  return tensors;
}

// ---------------------------------------------------------------- execution plan
struct Source {
  std::string tensor_name;
  std::uint64_t segment_offset;
  std::uint64_t byte_size;
};

struct Segment {
  std::string name;
  std::vector<std::uint64_t> shape;
  std::uint64_t arena_offset{0};
  std::uint64_t byte_size{0};
  std::vector<Source> sources;
};

struct SourceSpec {
  std::string tensor_name;
  std::vector<std::uint64_t> shape;
};

struct SegmentSpec {
  std::string name;
  std::vector<std::uint64_t> shape;
  std::vector<SourceSpec> sources;
};

constexpr std::uint64_t arena_alignment = 256;

std::uint64_t align_up(std::uint64_t value) {
  return (value + arena_alignment - 1) / arena_alignment * arena_alignment;
}

// Segment names and source tensors of the target (src/weight_plan.cpp:37-82): qkv stacks the
// q, k (and v) projection rows, gate_up the gate rows then the up rows.
std::vector<SegmentSpec> target_specs(const carat_b200_model_config &config) {
  const std::uint64_t hidden = static_cast<std::uint64_t>(config.hidden_size);
  const std::uint64_t intermediate = static_cast<std::uint64_t>(config.intermediate_size);
  const std::uint64_t vocabulary = static_cast<std::uint64_t>(config.vocabulary_size);
  std::vector<SegmentSpec> specs;
  specs.push_back({"token_embedding",
                   {vocabulary, hidden},
                   {{"model.language_model.embed_tokens.weight", {vocabulary, hidden}}}});
  for (int layer = 0; layer < config.layer_count; ++layer) {
    const carat_b200_layer_shape &shape = config.layers[layer];
    const std::uint64_t dim = static_cast<std::uint64_t>(shape.head_dim);
    const std::uint64_t query = static_cast<std::uint64_t>(shape.query_heads) * dim;
    const std::uint64_t kv = static_cast<std::uint64_t>(shape.kv_heads) * dim;
    const std::string source = "model.language_model.layers." + std::to_string(layer) + ".";
    const std::string prefix = "layer." + std::to_string(layer) + ".";
    const auto single = [&](const char *segment, const char *tensor,
                            std::vector<std::uint64_t> extents) {
      specs.push_back({prefix + segment, extents, {{source + tensor, extents}}});
    };
    SegmentSpec qkv{prefix + "qkv",
                    {query + kv, hidden},
                    {{source + "self_attn.q_proj.weight", {query, hidden}},
                     {source + "self_attn.k_proj.weight", {kv, hidden}}}};
    if (!shape.key_equals_value) {
      qkv.shape[0] += kv;
      qkv.sources.push_back({source + "self_attn.v_proj.weight", {kv, hidden}});
    }
    single("input_norm", "input_layernorm.weight", {hidden});
    single("q_norm", "self_attn.q_norm.weight", {dim});
    single("k_norm", "self_attn.k_norm.weight", {dim});
    specs.push_back(std::move(qkv));
    single("o", "self_attn.o_proj.weight", {hidden, query});
    single("post_attention_norm", "post_attention_layernorm.weight", {hidden});
    single("pre_mlp_norm", "pre_feedforward_layernorm.weight", {hidden});
    specs.push_back({prefix + "gate_up",
                     {2 * intermediate, hidden},
                     {{source + "mlp.gate_proj.weight", {intermediate, hidden}},
                      {source + "mlp.up_proj.weight", {intermediate, hidden}}}});
    single("down", "mlp.down_proj.weight", {hidden, intermediate});
    single("post_mlp_norm", "post_feedforward_layernorm.weight", {hidden});
    single("scalar", "layer_scalar", {1});
  }
  specs.push_back({"final_norm", {hidden}, {{"model.language_model.norm.weight", {hidden}}}});
  return specs;
}

// The drafter's segments (src/weight_plan.cpp:84-128); its shape is fixed in the reference
// (include/carat/weight_plan.h:25-35) and taken from `assistant` and the target config here.
std::vector<SegmentSpec> assistant_specs(const carat_b200_assistant_config &assistant,
                                         std::uint64_t backbone_hidden, std::uint64_t vocabulary) {
  const std::uint64_t hidden = static_cast<std::uint64_t>(assistant.hidden_size);
  const std::uint64_t intermediate = static_cast<std::uint64_t>(assistant.intermediate_size);
  std::vector<SegmentSpec> specs{
      {"token_embedding", {vocabulary, hidden}, {{"model.embed_tokens.weight", {vocabulary, hidden}}}},
      {"pre_projection",
       {hidden, 2 * backbone_hidden},
       {{"pre_projection.weight", {hidden, 2 * backbone_hidden}}}},
      {"post_projection",
       {backbone_hidden, hidden},
       {{"post_projection.weight", {backbone_hidden, hidden}}}},
  };
  for (int layer = 0; layer < assistant.layer_count; ++layer) {
    const std::uint64_t dim = assistant.layer_global[layer] ? 512 : 256;
    const std::uint64_t query = static_cast<std::uint64_t>(assistant.query_heads) * dim;
    const std::string source = "model.layers." + std::to_string(layer) + ".";
    const std::string prefix = "layer." + std::to_string(layer) + ".";
    const auto single = [&](const char *segment, const char *tensor,
                            std::vector<std::uint64_t> extents) {
      specs.push_back({prefix + segment, extents, {{source + tensor, extents}}});
    };
    single("input_norm", "input_layernorm.weight", {hidden});
    single("q_norm", "self_attn.q_norm.weight", {dim});
    single("q", "self_attn.q_proj.weight", {query, hidden});
    single("o", "self_attn.o_proj.weight", {hidden, query});
    single("post_attention_norm", "post_attention_layernorm.weight", {hidden});
    single("pre_mlp_norm", "pre_feedforward_layernorm.weight", {hidden});
    specs.push_back({prefix + "gate_up",
                     {2 * intermediate, hidden},
                     {{source + "mlp.gate_proj.weight", {intermediate, hidden}},
                      {source + "mlp.up_proj.weight", {intermediate, hidden}}}});
    single("down", "mlp.down_proj.weight", {hidden, intermediate});
    single("post_mlp_norm", "post_feedforward_layernorm.weight", {hidden});
    single("scalar", "layer_scalar", {1});
  }
  specs.push_back({"final_norm", {hidden}, {{"model.norm.weight", {hidden}}}});
  return specs;
}

struct Plan {
  std::vector<Segment> segments;
  std::uint64_t arena_bytes{0};
};

// Builds the plan with the reference's checks and messages (src/weight_plan.cpp:130-196).
Plan build_plan(const std::vector<SegmentSpec> &specs, const TensorTable &tensors,
                const std::string &label, const std::string &required_prefix) {
  Plan plan;
  std::set<std::string> used;
  std::uint64_t offset = 0;
  for (const SegmentSpec &spec : specs) {
    Segment segment;
    segment.name = spec.name;
    segment.shape = spec.shape;
    segment.arena_offset = align_up(offset);
    for (const SourceSpec &source : spec.sources) {
      const auto found = tensors.find(source.tensor_name);
      if (found == tensors.end())
        throw Failure{"missing tensor " + source.tensor_name};
      if (found->second.dtype != "BF16")
        throw Failure{label + "execution weights must be BF16: " + source.tensor_name};
      if (!used.insert(source.tensor_name).second)
        throw Failure{label + "weight source used twice: " + source.tensor_name};
      segment.sources.push_back({source.tensor_name, segment.byte_size, found->second.byte_size});
      segment.byte_size += found->second.byte_size;
    }
    std::uint64_t elements = 1;
    for (const std::uint64_t extent : segment.shape)
      elements *= extent;
    if (segment.byte_size % 2 != 0 || elements != segment.byte_size / 2) {
      throw Failure{label + "packed execution shape does not match source bytes: " + segment.name};
    }
    for (const SourceSpec &source : spec.sources) {
      if (tensors.find(source.tensor_name)->second.shape != source.shape) {
        throw Failure{label + "source shape does not match execution plan: " +
                      source.tensor_name};
      }
    }
    offset = segment.arena_offset + segment.byte_size;
    plan.segments.push_back(std::move(segment));
  }
  for (const auto &entry : tensors) {
    if (entry.first.compare(0, required_prefix.size(), required_prefix) == 0 &&
        used.find(entry.first) == used.end()) {
      throw Failure{label + "tensor absent from execution plan: " + entry.first};
    }
  }
  plan.arena_bytes = align_up(offset);
  return plan;
}

Plan plan_for(const std::string &directory, const carat_b200_model_config *config,
              const carat_b200_assistant_config *assistant, TensorTable *tensors_out) {
  if (config == nullptr || config->layers == nullptr || config->layer_count <= 0)
    throw Failure{"invalid batch model runner shape"};
  TensorTable tensors = open_model_directory(directory);
  Plan plan;
  if (assistant == nullptr) {
    plan = build_plan(target_specs(*config), tensors, "", "model.language_model.");
  } else {
    if (assistant->layer_global == nullptr || assistant->layer_count <= 0)
      throw Failure{"invalid assistant shape"};
    plan = build_plan(assistant_specs(*assistant, static_cast<std::uint64_t>(config->hidden_size),
                                      static_cast<std::uint64_t>(config->vocabulary_size)),
                      tensors, "assistant ", "");
  }
  if (tensors_out != nullptr)
    *tensors_out = std::move(tensors);
  return plan;
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

void require_cuda(cudaError_t status, const char *operation) {
  if (status != cudaSuccess)
    throw Failure{std::string(operation) + ": " + cudaGetErrorString(status)};
}

} // namespace

struct carat_b200_weights {
  Plan plan;
  std::map<std::string, size_t, std::less<>> by_name;
  unsigned char *arena{nullptr};       // bf16 segments at plan offsets
  unsigned char *fp8_arena{nullptr};   // e4m3 bytes of the two-dimensional segments
  float *scales{nullptr};              // one fp32 per two-dimensional segment
  std::vector<std::uint64_t> fp8_offsets;   // per segment; ~0 when it has no e4m3 form
  std::uint64_t fp8_bytes{0};
  // INT4 form of the MLP matrices (carat_b200_weights_quantize_int4_mlp): per layer the reordered
  // codes and group scales of gate_up and down, in one allocation.
  unsigned char *int4_arena{nullptr};
  std::vector<carat_b200_int4_mlp_layer> int4_layers;
  int int4_group_width{0};

  ~carat_b200_weights() {
    cudaFree(int4_arena);
    cudaFree(scales);
    cudaFree(fp8_arena);
    cudaFree(arena);
  }
};

namespace {

constexpr std::uint64_t no_fp8 = ~0ULL;
constexpr size_t staging_bytes = 64u << 20;

// Reads every source into its place in the arena through two pinned buffers (read k+1 overlaps
// the copy of k), and quantises a segment once its last byte is on the device.
void upload_and_quantize(carat_b200_weights &weights, const TensorTable &tensors, bool quantize) {
  const Plan &plan = weights.plan;
  require_cuda(cudaMalloc(&weights.arena, plan.arena_bytes), "allocate weight arena");
  weights.fp8_offsets.assign(plan.segments.size(), no_fp8);
  if (quantize) {
    std::uint64_t offset = 0;
    size_t matrices = 0;
    for (size_t index = 0; index < plan.segments.size(); ++index) {
      if (plan.segments[index].shape.size() != 2)
        continue;
      weights.fp8_offsets[index] = align_up(offset);
      offset = weights.fp8_offsets[index] + plan.segments[index].byte_size / 2;
      ++matrices;
    }
    weights.fp8_bytes = align_up(offset);
    if (matrices == 0)
      throw Failure{"empty FP8 weight plan"};
    require_cuda(cudaMalloc(&weights.fp8_arena, weights.fp8_bytes), "allocate FP8 weight arena");
    require_cuda(cudaMalloc(&weights.scales, sizeof(float) * plan.segments.size()),
                 "allocate FP8 scale arena");
  }
  cudaStream_t copy_stream = nullptr;
  cudaStream_t quantize_stream = nullptr;
  unsigned char *staging[2] = {nullptr, nullptr};
  cudaEvent_t staged[2] = {nullptr, nullptr};
  cudaEvent_t landed = nullptr;
  unsigned int *amax_words = nullptr;
  std::map<std::string, int> descriptors;
  const auto release = [&] {
    for (auto &entry : descriptors)
      close(entry.second);
    cudaFree(amax_words);
    if (landed != nullptr)
      cudaEventDestroy(landed);
    for (int index = 0; index < 2; ++index) {
      if (staged[index] != nullptr)
        cudaEventDestroy(staged[index]);
      cudaFreeHost(staging[index]);
    }
    if (quantize_stream != nullptr)
      cudaStreamDestroy(quantize_stream);
    if (copy_stream != nullptr)
      cudaStreamDestroy(copy_stream);
  };
  try {
    require_cuda(cudaStreamCreateWithFlags(&copy_stream, cudaStreamNonBlocking), "create stream");
    require_cuda(cudaStreamCreateWithFlags(&quantize_stream, cudaStreamNonBlocking),
                 "create stream");
    for (int index = 0; index < 2; ++index) {
      require_cuda(cudaMallocHost(&staging[index], staging_bytes), "allocate pinned staging");
      require_cuda(cudaEventCreateWithFlags(&staged[index], cudaEventDisableTiming),
                   "create event");
    }
    require_cuda(cudaEventCreateWithFlags(&landed, cudaEventDisableTiming), "create event");
    require_cuda(cudaMalloc(&amax_words, sizeof(unsigned int) * plan.segments.size()),
                 "allocate amax words");
    require_cuda(cudaMemsetAsync(amax_words, 0, sizeof(unsigned int) * plan.segments.size(),
                                 quantize_stream),
                 "clear amax words");
    int buffer = 0;
    for (size_t index = 0; index < plan.segments.size(); ++index) {
      const Segment &segment = plan.segments[index];
      for (const Source &source : segment.sources) {
        const Tensor &tensor = tensors.find(source.tensor_name)->second;
        auto opened = descriptors.find(tensor.shard_path);
        if (opened == descriptors.end()) {
          const int descriptor = open(tensor.shard_path.c_str(), O_RDONLY);
          if (descriptor < 0)
            throw Failure{"cannot open safetensors file " + tensor.shard_path};
          opened = descriptors.emplace(tensor.shard_path, descriptor).first;
        }
        for (std::uint64_t done = 0; done < source.byte_size; done += staging_bytes) {
          const size_t part =
              static_cast<size_t>(std::min<std::uint64_t>(staging_bytes, source.byte_size - done));
          // The buffer is free again once the copy that last used it has finished.
          require_cuda(cudaEventSynchronize(staged[buffer]), "wait for staging buffer");
          size_t filled = 0;
          while (filled < part) {
            const ssize_t got = pread(opened->second, staging[buffer] + filled, part - filled,
                                      static_cast<off_t>(tensor.file_offset + done + filled));
            if (got <= 0)
              throw Failure{"cannot read tensor " + source.tensor_name};
            filled += static_cast<size_t>(got);
          }
          require_cuda(cudaMemcpyAsync(weights.arena + segment.arena_offset +
                                           source.segment_offset + done,
                                       staging[buffer], part, cudaMemcpyHostToDevice, copy_stream),
                       "copy weights to the device");
          require_cuda(cudaEventRecord(staged[buffer], copy_stream), "record staging event");
          buffer ^= 1;
        }
      }
      if (quantize && weights.fp8_offsets[index] != no_fp8) {
        // Tensor-scale e4m3 of the whole segment (cuda/device_weights.cu:246-249).
        require_cuda(cudaEventRecord(landed, copy_stream), "record segment event");
        require_cuda(cudaStreamWaitEvent(quantize_stream, landed, 0), "order quantiser");
        if (launch_quant_tensor(weights.arena + segment.arena_offset,
                                weights.fp8_arena + weights.fp8_offsets[index],
                                weights.scales + index, amax_words + index,
                                static_cast<size_t>(segment.byte_size / 2), quantize_stream) != 0) {
          throw Failure{"FP8 weight quantisation launch failed"};
        }
      }
    }
    require_cuda(cudaStreamSynchronize(copy_stream), "finish weight upload");
    require_cuda(cudaStreamSynchronize(quantize_stream), "finish FP8 weight quantization");
  } catch (...) {
    release();
    throw;
  }
  release();
}

void describe(const carat_b200_weights &weights, size_t index, carat_b200_weight_segment *out) {
  const Segment &segment = weights.plan.segments[index];
  std::memset(out, 0, sizeof(*out));
  std::strncpy(out->name, segment.name.c_str(), sizeof(out->name) - 1);
  out->rank = static_cast<int32_t>(segment.shape.size());
  for (size_t axis = 0; axis < segment.shape.size() && axis < 2; ++axis)
    out->shape[axis] = segment.shape[axis];
  out->arena_offset = segment.arena_offset;
  out->byte_size = segment.byte_size;
  out->bf16 = weights.arena != nullptr ? weights.arena + segment.arena_offset : nullptr;
  if (weights.fp8_arena != nullptr && weights.fp8_offsets[index] != no_fp8) {
    out->fp8 = weights.fp8_arena + weights.fp8_offsets[index];
    out->fp8_scale = weights.scales + index;
  }
}

} // namespace

extern "C" int carat_b200_weights_plan_text(const char *model_directory,
                                            const carat_b200_model_config *config,
                                            const carat_b200_assistant_config *assistant,
                                            char *buffer, size_t buffer_bytes, size_t *needed) {
  return guarded([&] {
    if (model_directory == nullptr || needed == nullptr)
      throw Failure{"invalid weight plan request"};
    const Plan plan = plan_for(model_directory, config, assistant, nullptr);
    std::string text = "arena_bytes " + std::to_string(plan.arena_bytes) + "\n";
    for (const Segment &segment : plan.segments) {
      text += segment.name + " shape";
      for (const std::uint64_t extent : segment.shape)
        text += " " + std::to_string(extent);
      text += " offset " + std::to_string(segment.arena_offset) + " bytes " +
              std::to_string(segment.byte_size) + " sources";
      for (const Source &source : segment.sources)
        text += " " + source.tensor_name + "@" + std::to_string(source.segment_offset);
      text += "\n";
    }
    *needed = text.size() + 1;
    if (buffer != nullptr && buffer_bytes >= text.size() + 1)
      std::memcpy(buffer, text.c_str(), text.size() + 1);
  });
}

extern "C" int carat_b200_weights_load(const char *model_directory,
                                       const carat_b200_model_config *config,
                                       const carat_b200_assistant_config *assistant,
                                       int quantize_fp8, carat_b200_weights **weights) {
  return guarded([&] {
    if (model_directory == nullptr || weights == nullptr)
      throw Failure{"invalid weight plan request"};
    auto made = std::make_unique<carat_b200_weights>();
    TensorTable tensors;
    made->plan = plan_for(model_directory, config, assistant, &tensors);
    for (size_t index = 0; index < made->plan.segments.size(); ++index)
      made->by_name.emplace(made->plan.segments[index].name, index);
    upload_and_quantize(*made, tensors, quantize_fp8 != 0);
    *weights = made.release();
  });
}

extern "C" void carat_b200_weights_destroy(carat_b200_weights *weights) { delete weights; }

extern "C" int carat_b200_weights_segment_count(const carat_b200_weights *weights) {
  return weights == nullptr ? 0 : static_cast<int>(weights->plan.segments.size());
}

extern "C" int carat_b200_weights_segment(const carat_b200_weights *weights, int index,
                                          carat_b200_weight_segment *segment) {
  return guarded([&] {
    if (weights == nullptr || segment == nullptr || index < 0 ||
        index >= static_cast<int>(weights->plan.segments.size())) {
      throw Failure{"invalid weight segment index"};
    }
    describe(*weights, static_cast<size_t>(index), segment);
  });
}

extern "C" int carat_b200_weights_find(const carat_b200_weights *weights, const char *name,
                                       carat_b200_weight_segment *segment) {
  return guarded([&] {
    if (weights == nullptr || name == nullptr || segment == nullptr)
      throw Failure{"invalid weight segment index"};
    const auto found = weights->by_name.find(std::string_view(name));
    if (found == weights->by_name.end())
      throw Failure{std::string("missing execution weight ") + name};
    describe(*weights, found->second, segment);
  });
}

extern "C" int carat_b200_weights_quantize_int4_mlp(carat_b200_weights *weights,
                                                    int group_width) {
  return guarded([&] {
    if (weights == nullptr || (group_width != 128 && group_width != 256))
      throw Failure{"invalid BF16 INT4 linear weight shape"};
    // Layers are the segments "layer.N.gate_up" / "layer.N.down", N = 0, 1, ... without a gap.
    struct Matrix {
      size_t segment;
      std::uint64_t rows, cols;
    };
    std::vector<std::pair<Matrix, Matrix>> layers;
    for (int layer = 0;; ++layer) {
      const std::string prefix = "layer." + std::to_string(layer) + ".";
      const auto gate_up = weights->by_name.find(prefix + "gate_up");
      const auto down = weights->by_name.find(prefix + "down");
      if (gate_up == weights->by_name.end() || down == weights->by_name.end())
        break;
      const Segment &a = weights->plan.segments[gate_up->second];
      const Segment &b = weights->plan.segments[down->second];
      if (a.shape.size() != 2 || b.shape.size() != 2 || a.shape[1] % group_width != 0 ||
          b.shape[1] % group_width != 0 || a.shape[0] % 8 != 0 || b.shape[0] % 8 != 0) {
        throw Failure{"invalid BF16 INT4 linear weight shape"};
      }
      layers.push_back({{gate_up->second, a.shape[0], a.shape[1]},
                        {down->second, b.shape[0], b.shape[1]}});
    }
    if (layers.empty())
      throw Failure{"missing execution weight layer.0.gate_up"};
    const auto codes_bytes = [](const Matrix &m) { return align_up(m.rows * m.cols / 2); };
    const auto scales_bytes = [&](const Matrix &m) {
      return align_up(m.cols / static_cast<std::uint64_t>(group_width) * m.rows * 2);
    };
    std::uint64_t total = 0;
    std::uint64_t largest = 0;
    for (const auto &layer : layers) {
      for (const Matrix *m : {&layer.first, &layer.second}) {
        total += codes_bytes(*m) + scales_bytes(*m);
        largest = std::max(largest, codes_bytes(*m));
      }
    }
    cudaFree(weights->int4_arena);
    weights->int4_arena = nullptr;
    weights->int4_layers.clear();
    require_cuda(cudaMalloc(&weights->int4_arena, total), "allocate INT4 weight arena");
    unsigned char *row_major = nullptr;   // the reference-layout codes, before reordering
    require_cuda(cudaMalloc(&row_major, largest), "allocate INT4 staging");
    std::uint64_t offset = 0;
    int status = 0;
    for (const auto &layer : layers) {
      carat_b200_int4_mlp_layer out{};
      int index = 0;
      for (const Matrix *m : {&layer.first, &layer.second}) {
        unsigned char *codes = weights->int4_arena + offset;
        offset += codes_bytes(*m);
        unsigned char *scales = weights->int4_arena + offset;
        offset += scales_bytes(*m);
        const void *source = weights->arena + weights->plan.segments[m->segment].arena_offset;
        if (status == 0) {
          status = launch_int4_quantize(source, row_major, scales, static_cast<int>(m->rows),
                                        static_cast<int>(m->cols), group_width, nullptr);
        }
        if (status == 0)
          status = launch_int4_reorder(row_major, codes, m->rows * m->cols / 2, nullptr);
        if (index++ == 0) {
          out.gate_up_codes = codes;
          out.gate_up_scales = scales;
        } else {
          out.down_codes = codes;
          out.down_scales = scales;
        }
      }
      weights->int4_layers.push_back(out);
    }
    const cudaError_t finished = cudaDeviceSynchronize();
    cudaFree(row_major);
    if (status != 0 || finished != cudaSuccess) {
      weights->int4_layers.clear();
      throw Failure{"INT4 weight quantization failed"};
    }
    weights->int4_group_width = group_width;
  });
}

extern "C" int carat_b200_weights_int4_mlp_layers(const carat_b200_weights *weights,
                                                  carat_b200_int4_mlp_layer *layers, int capacity,
                                                  int *layer_count, int *group_width) {
  return guarded([&] {
    if (weights == nullptr || layer_count == nullptr)
      throw Failure{"invalid weight segment index"};
    *layer_count = static_cast<int>(weights->int4_layers.size());
    if (group_width != nullptr)
      *group_width = weights->int4_group_width;
    if (layers != nullptr) {
      if (capacity < *layer_count)
        throw Failure{"invalid weight segment index"};
      std::copy(weights->int4_layers.begin(), weights->int4_layers.end(), layers);
    }
  });
}
