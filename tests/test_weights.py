"""The weight pipeline (carat_b200_weights_*): safetensors model directory -> execution plan ->
device arenas. The plan checks mirror tests/weight_plan_tests.cpp of the reference (same tiny
model, same expectations and error texts; the fixtures are sparse files like the reference's,
tests/support/model_fixtures.cpp:84-97); the GPU test loads real bytes and compares the arenas
with the source tensors and the oracle's quantiser."""
import ctypes
import json
import os
import struct

import pytest
import torch

import carat_b200
from carat_b200 import capi

DTYPE_BYTES = {"BF16": 2, "F32": 4, "F16": 2, "U8": 1}


def write_safetensors(path, tensors, data=None):
    """tensors: [(name, dtype, shape)]. Without `data` the file is sparse (offsets only)."""
    header = {"__metadata__": {"format": "pt"}}
    offset = 0
    for name, dtype, shape in tensors:
        size = DTYPE_BYTES[dtype]
        for extent in shape:
            size *= extent
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [offset, offset + size]}
        offset += size
    text = json.dumps(header, separators=(",", ":"))
    text += " " * (-len(text) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(text)))
        handle.write(text.encode())
        if data is not None:
            for name, _, _ in tensors:
                handle.write(data[name])
        else:
            handle.truncate(8 + len(text) + offset)


def tiny_layer(tensors, layer, query, kv, dim, has_value):
    prefix = f"model.language_model.layers.{layer}."
    tensors += [(prefix + "input_layernorm.weight", "BF16", (8,)),
                (prefix + "self_attn.q_norm.weight", "BF16", (dim,)),
                (prefix + "self_attn.k_norm.weight", "BF16", (dim,)),
                (prefix + "self_attn.q_proj.weight", "BF16", (query, 8)),
                (prefix + "self_attn.k_proj.weight", "BF16", (kv, 8))]
    if has_value:
        tensors.append((prefix + "self_attn.v_proj.weight", "BF16", (kv, 8)))
    tensors += [(prefix + "self_attn.o_proj.weight", "BF16", (8, query)),
                (prefix + "post_attention_layernorm.weight", "BF16", (8,)),
                (prefix + "pre_feedforward_layernorm.weight", "BF16", (8,)),
                (prefix + "mlp.gate_proj.weight", "BF16", (16, 8)),
                (prefix + "mlp.up_proj.weight", "BF16", (16, 8)),
                (prefix + "mlp.down_proj.weight", "BF16", (8, 16)),
                (prefix + "post_feedforward_layernorm.weight", "BF16", (8,)),
                (prefix + "layer_scalar", "BF16", (1,))]


def tiny_tensors():
    tensors = [("model.language_model.embed_tokens.weight", "BF16", (32, 8)),
               ("model.language_model.norm.weight", "BF16", (8,))]
    tiny_layer(tensors, 0, 512, 256, 256, True)
    tiny_layer(tensors, 1, 1024, 512, 512, False)
    return tensors


def with_tensor(tensors, name, dtype, shape):
    changed = [(n, dtype, tuple(shape)) if n == name else (n, d, s) for n, d, s in tensors]
    if all(n != name for n, _, _ in tensors):
        changed.append((name, dtype, tuple(shape)))
    return changed


def tiny_config():
    layers = [carat_b200.Gemma4LayerConfig("sliding", 2, 1, 256, 1e4, False),
              carat_b200.Gemma4LayerConfig("global", 2, 1, 512, 1e6, True)]
    return carat_b200.Gemma4Config(8, 16, 32, 4, 1e-6, layers)


def plan_of(directory, config=None, assistant=None):
    """Parses carat_b200_weights_plan_text into (arena_bytes, [segment dicts])."""
    library = carat_b200.library()
    model_config, keep = carat_b200.runner.model_config_struct(config or tiny_config())
    assistant_struct, keep2 = (None, None)
    if assistant is not None:
        assistant_struct, keep2 = carat_b200.runner.assistant_config_struct(assistant)
    needed = ctypes.c_size_t(0)
    arguments = (str(directory).encode(), ctypes.byref(model_config),
                 ctypes.byref(assistant_struct) if assistant_struct is not None else None)
    capi.check(library.carat_b200_weights_plan_text(*arguments, None, 0, ctypes.byref(needed)))
    buffer = ctypes.create_string_buffer(needed.value)
    capi.check(library.carat_b200_weights_plan_text(*arguments, buffer, needed.value,
                                                    ctypes.byref(needed)))
    lines = buffer.value.decode().splitlines()
    arena_bytes = int(lines[0].split()[1])
    segments = []
    for line in lines[1:]:
        words = line.split()
        shape_end = words.index("offset")
        sources = words[words.index("sources") + 1:]
        segments.append({"name": words[0], "shape": [int(w) for w in words[2:shape_end]],
                         "offset": int(words[shape_end + 1]), "bytes": int(words[shape_end + 3]),
                         "sources": [(s.rsplit("@", 1)[0], int(s.rsplit("@", 1)[1]))
                                     for s in sources]})
    return arena_bytes, segments


def by_name(segments, name):
    return next(segment for segment in segments if segment["name"] == name)


def test_plan_packs_value_projection_only_without_key_value_sharing(tmp_path):
    write_safetensors(tmp_path / "model.safetensors", tiny_tensors())
    _, segments = plan_of(tmp_path)
    sliding = by_name(segments, "layer.0.qkv")
    assert sliding["shape"] == [1024, 8]
    assert [name for name, _ in sliding["sources"]] == [
        "model.language_model.layers.0.self_attn.q_proj.weight",
        "model.language_model.layers.0.self_attn.k_proj.weight",
        "model.language_model.layers.0.self_attn.v_proj.weight"]
    global_ = by_name(segments, "layer.1.qkv")
    assert global_["shape"] == [1536, 8]
    assert [name for name, _ in global_["sources"]] == [
        "model.language_model.layers.1.self_attn.q_proj.weight",
        "model.language_model.layers.1.self_attn.k_proj.weight"]
    assert by_name(segments, "layer.1.gate_up")["shape"] == [32, 8]
    assert len(segments) == 2 + 2 * 11


def test_arena_segments_are_aligned_contiguous_and_disjoint(tmp_path):
    write_safetensors(tmp_path / "model.safetensors", tiny_tensors())
    arena_bytes, segments = plan_of(tmp_path)
    previous_end = 0
    for segment in segments:
        assert segment["offset"] % 256 == 0 and segment["offset"] >= previous_end
        source_offset = 0
        sizes = {name: DTYPE_BYTES[d] * int(torch.tensor(s).prod()) for name, d, s in tiny_tensors()}
        for name, offset in segment["sources"]:
            assert offset == source_offset
            source_offset += sizes[name]
        assert source_offset == segment["bytes"]
        previous_end = segment["offset"] + segment["bytes"]
    assert arena_bytes >= previous_end and arena_bytes % 256 == 0
    assert segments[0]["name"] == "token_embedding" and segments[-1]["name"] == "final_norm"


def test_sharded_directory_and_tensors_outside_the_language_model(tmp_path):
    tensors = with_tensor(tiny_tensors(), "model.vision_tower.patch.weight", "F32", (4,))
    middle = len(tensors) // 2
    shards = {"model-1.safetensors": tensors[:middle], "model-2.safetensors": tensors[middle:]}
    weight_map = {}
    for shard, part in shards.items():
        write_safetensors(tmp_path / shard, part)
        weight_map.update({name: shard for name, _, _ in part})
    (tmp_path / "model.safetensors.index.json").write_text(
        json.dumps({"metadata": {}, "weight_map": weight_map}))
    assert len(plan_of(tmp_path)[1]) == 24


def failing(tmp_path, tensors, message):
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(carat_b200.CaratError) as error:
        plan_of(tmp_path)
    assert message in str(error.value), str(error.value)


def test_plan_rejects_invalid_sources(tmp_path):
    o_proj = "model.language_model.layers.1.self_attn.o_proj.weight"
    without_norm = [t for t in tiny_tensors() if t[0] != "model.language_model.norm.weight"]
    failing(tmp_path, without_norm, "missing tensor model.language_model.norm.weight")
    failing(tmp_path, with_tensor(tiny_tensors(), o_proj, "F32", (8, 1024)),
            "execution weights must be BF16: " + o_proj)
    failing(tmp_path, with_tensor(tiny_tensors(), o_proj, "BF16", (8, 8)),
            "packed execution shape does not match source bytes: layer.1.o")
    failing(tmp_path, with_tensor(tiny_tensors(), o_proj, "BF16", (1024, 8)),
            "source shape does not match execution plan: " + o_proj)
    failing(tmp_path, with_tensor(tiny_tensors(), "model.language_model.extra.weight", "BF16", (2,)),
            "tensor absent from execution plan: model.language_model.extra.weight")


def test_a_directory_without_weights_is_reported(tmp_path):
    with pytest.raises(carat_b200.CaratError, match="cannot open safetensors file"):
        plan_of(tmp_path)


def test_malformed_headers_are_rejected(tmp_path):
    path = tmp_path / "model.safetensors"
    path.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(carat_b200.CaratError, match="invalid safetensors header size"):
        plan_of(tmp_path)
    header = json.dumps({"a": {"dtype": "BF16", "shape": [4], "data_offsets": [0, 6]}})
    path.write_bytes(struct.pack("<Q", len(header)) + header.encode() + b"\0" * 8)
    with pytest.raises(carat_b200.CaratError, match="byte-size mismatch for tensor a"):
        plan_of(tmp_path)
    header = json.dumps({"a": {"dtype": "BF16", "shape": [4], "data_offsets": [0, 8]}})
    path.write_bytes(struct.pack("<Q", len(header)) + header.encode() + b"\0" * 4)
    with pytest.raises(carat_b200.CaratError, match="out-of-range tensor a"):
        plan_of(tmp_path)


def test_assistant_plan_packs_the_fixed_architecture(tmp_path):
    tensors = [("model.embed_tokens.weight", "BF16", (262144, 1024)),
               ("pre_projection.weight", "BF16", (1024, 10752)),
               ("post_projection.weight", "BF16", (5376, 1024)),
               ("model.norm.weight", "BF16", (1024,))]
    for layer in range(4):
        dim = 512 if layer == 3 else 256
        prefix = f"model.layers.{layer}."
        tensors += [(prefix + "input_layernorm.weight", "BF16", (1024,)),
                    (prefix + "self_attn.q_norm.weight", "BF16", (dim,)),
                    (prefix + "self_attn.q_proj.weight", "BF16", (32 * dim, 1024)),
                    (prefix + "self_attn.o_proj.weight", "BF16", (1024, 32 * dim)),
                    (prefix + "post_attention_layernorm.weight", "BF16", (1024,)),
                    (prefix + "pre_feedforward_layernorm.weight", "BF16", (1024,)),
                    (prefix + "mlp.gate_proj.weight", "BF16", (8192, 1024)),
                    (prefix + "mlp.up_proj.weight", "BF16", (8192, 1024)),
                    (prefix + "mlp.down_proj.weight", "BF16", (1024, 8192)),
                    (prefix + "post_feedforward_layernorm.weight", "BF16", (1024,)),
                    (prefix + "layer_scalar", "BF16", (1,))]
    write_safetensors(tmp_path / "model.safetensors", tensors)      # sparse: 2 GB of nothing
    target = carat_b200.Gemma4Config(5376, 21504, 262144, 1024, 1e-6, tiny_config().layers)
    _, segments = plan_of(tmp_path, target, carat_b200.Gemma4AssistantConfig())
    assert len(segments) == 3 + 4 * 10 + 1
    assert by_name(segments, "layer.0.q")["shape"] == [8192, 1024]
    assert by_name(segments, "layer.3.q")["shape"] == [16384, 1024]
    assert by_name(segments, "layer.3.q_norm")["shape"] == [512]
    assert len(by_name(segments, "layer.2.gate_up")["sources"]) == 2
    write_safetensors(tmp_path / "model.safetensors", tensors + [("stray.weight", "BF16", (2,))])
    with pytest.raises(carat_b200.CaratError,
                       match="assistant tensor absent from execution plan: stray.weight"):
        plan_of(tmp_path, target, carat_b200.Gemma4AssistantConfig())


@pytest.mark.gpu
def test_load_uploads_and_quantises_like_the_oracle(cuda_device, tmp_path):
    """Real bytes through the pipeline: two shards, fused segments stacked from their sources,
    e4m3 bytes and scales equal to the oracle's tensor-scale quantiser (cuda/linear.cu:76-153)."""
    from oracle import carat_semantics as cs
    tensors = tiny_tensors()
    generator = torch.Generator().manual_seed(0)
    values = {name: cs.bf16(torch.randn(shape, generator=generator) * 0.05)
              for name, _, shape in tensors}
    data = {name: values[name].to(torch.bfloat16).view(torch.int16).numpy().tobytes()
            for name in values}
    middle = len(tensors) // 2
    weight_map = {}
    for shard, part in (("model-1.safetensors", tensors[:middle]),
                        ("model-2.safetensors", tensors[middle:])):
        write_safetensors(tmp_path / shard, part, data)
        weight_map.update({name: shard for name, _, _ in part})
    (tmp_path / "model.safetensors.index.json").write_text(
        json.dumps({"metadata": {}, "weight_map": weight_map}))
    loaded = carat_b200.LoadedWeights(str(tmp_path), tiny_config())
    try:
        layer0 = "model.language_model.layers.0."
        qkv = torch.cat([values[layer0 + "self_attn.q_proj.weight"],
                         values[layer0 + "self_attn.k_proj.weight"],
                         values[layer0 + "self_attn.v_proj.weight"]])
        assert torch.equal(loaded.bf16.at("layer.0.qkv").float().cpu(), qkv)
        gate_up = torch.cat([values[layer0 + "mlp.gate_proj.weight"],
                             values[layer0 + "mlp.up_proj.weight"]])
        assert torch.equal(loaded.bf16.at("layer.0.gate_up").float().cpu(), gate_up)
        assert torch.equal(loaded.bf16.at("final_norm").float().cpu(),
                           values["model.language_model.norm.weight"])
        for name, source in (("layer.0.qkv", qkv), ("layer.0.gate_up", gate_up),
                             ("token_embedding",
                              values["model.language_model.embed_tokens.weight"])):
            want, want_scale = cs.quantize_e4m3(source)
            assert torch.equal(loaded.fp8.scale(name).cpu(), want_scale.reshape(1))
            assert torch.equal(loaded.fp8.at(name).view(torch.float8_e4m3fn).float().cpu(), want)
        with pytest.raises(carat_b200.CaratError, match="missing execution weight layer.2.qkv"):
            loaded.find("layer.2.qkv")
    finally:
        loaded.close()


@pytest.mark.gpu
def test_int4_mlp_form_comes_out_of_the_pipeline(cuda_device, tmp_path):
    """carat_b200_weights_quantize_int4_mlp on a loaded model (hidden 256, FFN 512, one layer):
    the codes and scales are the bytes of the two calls a caller would otherwise make on the bf16
    segment (quantise in the reference's layout, cuda/int4_bf16_linear.cu:95-136, then reorder),
    and a runner takes the result as it is."""
    hidden, inter = 256, 512
    prefix = "model.language_model.layers.0."
    tensors = [("model.language_model.embed_tokens.weight", "BF16", (64, hidden)),
               ("model.language_model.norm.weight", "BF16", (hidden,)),
               (prefix + "input_layernorm.weight", "BF16", (hidden,)),
               (prefix + "self_attn.q_norm.weight", "BF16", (64,)),
               (prefix + "self_attn.k_norm.weight", "BF16", (64,)),
               (prefix + "self_attn.q_proj.weight", "BF16", (4 * 64, hidden)),
               (prefix + "self_attn.k_proj.weight", "BF16", (2 * 64, hidden)),
               (prefix + "self_attn.v_proj.weight", "BF16", (2 * 64, hidden)),
               (prefix + "self_attn.o_proj.weight", "BF16", (hidden, 4 * 64)),
               (prefix + "post_attention_layernorm.weight", "BF16", (hidden,)),
               (prefix + "pre_feedforward_layernorm.weight", "BF16", (hidden,)),
               (prefix + "mlp.gate_proj.weight", "BF16", (inter, hidden)),
               (prefix + "mlp.up_proj.weight", "BF16", (inter, hidden)),
               (prefix + "mlp.down_proj.weight", "BF16", (hidden, inter)),
               (prefix + "post_feedforward_layernorm.weight", "BF16", (hidden,)),
               (prefix + "layer_scalar", "BF16", (1,))]
    generator = torch.Generator().manual_seed(3)
    data = {name: (torch.randn(shape, generator=generator) * 0.05).to(torch.bfloat16)
            .view(torch.int16).numpy().tobytes() for name, _, shape in tensors}
    write_safetensors(tmp_path / "model.safetensors", tensors, data)
    config = carat_b200.Gemma4Config(hidden, inter, 64, 128, 1e-6, [
        carat_b200.Gemma4LayerConfig("sliding", 4, 2, 64, 1e4, False)])
    loaded = carat_b200.LoadedWeights(str(tmp_path), config)
    library = carat_b200.library()
    try:
        layers = loaded.int4_mlp_layers(128)
        assert len(layers) == 1
        for name, codes_pointer, scales_pointer in (
                ("gate_up", layers[0].gate_up_codes, layers[0].gate_up_scales),
                ("down", layers[0].down_codes, layers[0].down_scales)):
            weight = loaded.bf16.at(f"layer.0.{name}")
            rows, cols = weight.shape
            packed = torch.empty(rows, cols // 2, dtype=torch.uint8, device="cuda")
            scales = torch.empty(cols // 128, rows, dtype=torch.bfloat16, device="cuda")
            reordered = torch.empty_like(packed)
            capi.check(library.carat_b200_int4_quantize_weight(
                ctypes.c_void_p(weight.data_ptr()), ctypes.c_void_p(packed.data_ptr()),
                ctypes.c_void_p(scales.data_ptr()), rows, cols, 128, None))
            capi.check(library.carat_b200_int4_reorder_weight(
                ctypes.c_void_p(packed.data_ptr()), ctypes.c_void_p(reordered.data_ptr()), rows,
                cols, None))
            torch.cuda.synchronize()
            got_codes = torch.as_tensor(carat_b200.runner._DeviceView(
                codes_pointer, [rows, cols // 2], "|u1"), device="cuda")
            got_scales = torch.as_tensor(carat_b200.runner._DeviceView(
                scales_pointer, [cols // 128, rows], "<i2"), device="cuda")
            assert torch.equal(got_codes, reordered), name
            assert torch.equal(got_scales, scales.view(torch.int16)), name
        runner = carat_b200.Gemma4BatchModelRunner(config, loaded.bf16, 2, 256, loaded.fp8)
        runner.use_int4_mlp(loaded)
        tokens = torch.randint(3, 64, (8,), generator=generator).tolist()
        first = runner.prefill_slot_fp8(0, tokens, 8)
        assert 0 <= first < 64 and runner.slot_position(0) == 8
        runner.close()
        with pytest.raises(carat_b200.CaratError, match="invalid BF16 INT4 linear weight shape"):
            loaded.int4_mlp_layers(64)
    finally:
        loaded.close()
