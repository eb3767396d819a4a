"""Host-side mirror of the reference's runner interface for the speculative-decoding path.

Class and method names follow include/carat/batch_model_runner.h, include/carat/device_weights.h and
include/carat/gemma4_config.h of the reference so that callers (and the parity tests) read like the
reference's own code; every call goes through the C ABI in include/carat_b200.h. PyTorch is used
here only to own device memory.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from . import capi
from .capi import CaratError, check, int_array

VERIFY_ASSUME_MATCH = 1
ASSISTANT_FP8_MODES = {"off": 0, "lm_head": 1, "all": 2}   # CARAT_ASSISTANT_FP8_MODE values


# --------------------------------------------------------------------------- configuration
@dataclass
class Gemma4LayerConfig:
    """include/carat/gemma4_config.h:14-26."""

    attention: str  # "sliding" | "global"
    query_heads: int
    kv_heads: int
    head_dimension: int
    rope_theta: float
    key_equals_value: bool

    def query_width(self) -> int:
        return self.query_heads * self.head_dimension

    def kv_width(self) -> int:
        return self.kv_heads * self.head_dimension

    def packed_width(self) -> int:
        return self.query_width() + self.kv_width() * (1 if self.key_equals_value else 2)


@dataclass
class Gemma4Config:
    """include/carat/gemma4_config.h:28-43 (the fields the path reads)."""

    hidden_size: int
    intermediate_size: int
    vocabulary_size: int
    sliding_window: int
    rms_norm_epsilon: float
    layers: List[Gemma4LayerConfig] = field(default_factory=list)

    @staticmethod
    def gemma4_31b() -> "Gemma4Config":
        """Gemma-4-31B text shapes (reference: src/fp8_linear_benchmark.cu:346-351,
        cuda/layer_runner.cu:162-176). The layer order is assumed to repeat 5 sliding : 1 global."""
        layers = []
        for index in range(60):
            if index % 6 == 5:
                layers.append(Gemma4LayerConfig("global", 32, 4, 512, 1e6, True))
            else:
                layers.append(Gemma4LayerConfig("sliding", 32, 16, 256, 1e4, False))
        return Gemma4Config(5376, 21504, 262144, 1024, 1e-6, layers)

    @staticmethod
    def tiny() -> "Gemma4Config":
        """The CPU-runnable plumbing case: 3 sliding (window 128) + 1 global layer, hidden 256,
        4 query / 2 KV heads, head_dim 64, FFN 1024, vocab 4096."""
        layers = [Gemma4LayerConfig("sliding", 4, 2, 64, 1e4, False) for _ in range(3)]
        layers.append(Gemma4LayerConfig("global", 4, 2, 64, 1e6, True))
        return Gemma4Config(256, 1024, 4096, 128, 1e-6, layers)


@dataclass
class Gemma4AssistantConfig:
    """Drafter shape (reference constants: cuda/assistant_runner.cu:22-27,166-170)."""

    hidden_size: int = 1024
    intermediate_size: int = 8192
    query_heads: int = 32
    layers: List[str] = field(default_factory=lambda: ["sliding", "sliding", "sliding", "global"])
    rms_norm_epsilon: float = 1e-6


def model_config_struct(config: "Gemma4Config"):
    """capi.ModelConfig for `config`, plus the layer array it points into (keep both alive)."""
    shapes = (capi.LayerShape * len(config.layers))()
    for index, layer in enumerate(config.layers):
        shapes[index] = capi.LayerShape(1 if layer.attention == "global" else 0, layer.query_heads,
                                        layer.kv_heads, layer.head_dimension, layer.rope_theta,
                                        1 if layer.key_equals_value else 0)
    return capi.ModelConfig(config.hidden_size, config.intermediate_size, config.vocabulary_size,
                            config.sliding_window, config.rms_norm_epsilon, len(config.layers),
                            shapes), shapes


def assistant_config_struct(config: "Gemma4AssistantConfig"):
    kinds = (ctypes.c_int32 * len(config.layers))(
        *[1 if kind == "global" else 0 for kind in config.layers])
    return capi.AssistantConfig(config.hidden_size, config.intermediate_size, config.query_heads,
                                len(config.layers), kinds, config.rms_norm_epsilon), kinds


# --------------------------------------------------------------------------- weights
class DeviceWeightArena:
    """BF16 segments by name (include/carat/device_weights.h DeviceWeightArena::at)."""

    def __init__(self, tensors: Dict[str, torch.Tensor]):
        self.tensors = {}
        for name, tensor in tensors.items():
            if not tensor.is_cuda or tensor.dtype != torch.bfloat16:
                raise CaratError(f"weight segment {name} must be a CUDA bf16 tensor")
            self.tensors[name] = tensor.contiguous()

    @staticmethod
    def from_host(tensors: Dict[str, torch.Tensor], device="cuda") -> "DeviceWeightArena":
        return DeviceWeightArena({name: value.to(device=device, dtype=torch.bfloat16)
                                  for name, value in tensors.items()})

    def at(self, name: str) -> torch.Tensor:
        return self.tensors[name]

    def names(self):
        return self.tensors.keys()


def quantize_tensor_to_fp8(tensor: torch.Tensor):
    """Tensor-scale e4m3 quantisation on the device through the C ABI; returns (bytes, scale)."""
    library = capi.library()
    tensor = tensor.contiguous()
    output = torch.empty(tensor.shape, dtype=torch.uint8, device=tensor.device)
    scale = torch.zeros(1, dtype=torch.float32, device=tensor.device)
    scratch = torch.zeros(1, dtype=torch.int32, device=tensor.device)
    stream = torch.cuda.current_stream(tensor.device).cuda_stream
    check(library.carat_b200_quantize_bf16_tensor_to_fp8(
        tensor.data_ptr(), output.data_ptr(), scale.data_ptr(), scratch.data_ptr(),
        tensor.numel(), stream))
    return output, scale


class Int4Bf16Linear:
    """Weight-only INT4 linear with bf16 activations (include/carat/linear.h:70-90 Int4Bf16Linear).

    Like the reference's class, the constructor quantises a row-major bf16 [output_width,
    input_width] weight in K-local groups (scale = bf16(max / 7), codes clamped to [-7, 7]) and
    reorders the codes once for the kernel; `run` multiplies up to 128 bf16 rows with it."""

    def __init__(self, row_major_weight: torch.Tensor, input_width: int, output_width: int,
                 group_width: int = 256):
        library = capi.library()
        if (row_major_weight.dtype != torch.bfloat16 or input_width <= 0 or output_width <= 0
                or row_major_weight.numel() != input_width * output_width
                or group_width not in (128, 256) or input_width % group_width != 0
                or output_width % 8 != 0):
            raise CaratError("invalid BF16 INT4 linear weight shape")
        device = row_major_weight.device
        weight = row_major_weight.contiguous()
        self.input_width = input_width
        self.output_width = output_width
        self.group_width = group_width
        self.packed = torch.empty(output_width, input_width // 2, dtype=torch.uint8, device=device)
        self.scales = torch.empty(input_width // group_width, output_width, dtype=torch.bfloat16,
                                  device=device)
        self.reordered = torch.empty_like(self.packed)
        stream = torch.cuda.current_stream(device).cuda_stream
        check(library.carat_b200_int4_quantize_weight(
            weight.data_ptr(), self.packed.data_ptr(), self.scales.data_ptr(), output_width,
            input_width, group_width, stream))
        check(library.carat_b200_int4_reorder_weight(
            self.packed.data_ptr(), self.reordered.data_ptr(), output_width, input_width, stream))
        self._workspaces: Dict[int, torch.Tensor] = {}

    @staticmethod
    def supports_rows(rows: int) -> bool:
        return 0 < rows <= 128

    def run(self, bf16_input: torch.Tensor, bf16_output: Optional[torch.Tensor] = None):
        library = capi.library()
        rows = bf16_input.shape[0] if bf16_input.dim() == 2 else 0
        if (bf16_input.dtype != torch.bfloat16 or not self.supports_rows(rows)
                or bf16_input.shape[1] != self.input_width):
            raise CaratError("invalid BF16 INT4 linear activation shape")
        bf16_input = bf16_input.contiguous()
        if bf16_output is None:
            bf16_output = torch.empty(rows, self.output_width, dtype=torch.bfloat16,
                                      device=bf16_input.device)
        needed = library.carat_b200_int4_linear_workspace_bytes(rows, self.input_width,
                                                                self.output_width)
        workspace = self._workspaces.get(rows)
        if workspace is None:
            workspace = torch.empty(max(needed, 16), dtype=torch.uint8, device=bf16_input.device)
            self._workspaces[rows] = workspace
        stream = torch.cuda.current_stream(bf16_input.device).cuda_stream
        check(library.carat_b200_int4_linear(
            bf16_input.data_ptr(), self.reordered.data_ptr(), self.scales.data_ptr(),
            bf16_output.data_ptr(), rows, self.input_width, self.output_width, self.group_width,
            workspace.data_ptr(), needed, stream))
        return bf16_output

    def allocated_bytes(self) -> int:
        return self.reordered.numel() + self.scales.numel() * 2


class Fp8WeightArena:
    """e4m3 bytes + one fp32 scale per 2-D segment (include/carat/device_weights.h Fp8WeightArena,
    cuda/device_weights.cu:200-263)."""

    def __init__(self):
        self.bytes: Dict[str, torch.Tensor] = {}
        self.scales: Dict[str, torch.Tensor] = {}

    @staticmethod
    def quantize(weights: DeviceWeightArena) -> "Fp8WeightArena":
        arena = Fp8WeightArena()
        for name in weights.names():
            tensor = weights.at(name)
            if tensor.dim() == 2:
                arena.bytes[name], arena.scales[name] = quantize_tensor_to_fp8(tensor)
        torch.cuda.synchronize()
        return arena

    def add(self, name: str, fp8_bytes: torch.Tensor, scale: torch.Tensor) -> None:
        self.bytes[name] = fp8_bytes
        self.scales[name] = scale

    def at(self, name: str) -> torch.Tensor:
        return self.bytes[name]

    def scale(self, name: str) -> torch.Tensor:
        return self.scales[name]


class _DeviceView:
    """Lets torch wrap device memory the C library owns (no copy)."""

    def __init__(self, pointer: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr,
                                         "data": (pointer, False), "version": 2}


class LoadedWeights:
    """A model directory loaded through the weight pipeline of the library
    (carat_b200_weights_load: safetensors shards -> execution plan -> bf16 arena -> e4m3 arena;
    ShardedSafetensors::open + WeightPlan::gemma4 + DeviceWeightArena::load +
    Fp8WeightArena::quantize in the reference). `.bf16` and `.fp8` are the two arenas as the
    runner's constructor takes them; their tensors view the library's device memory."""

    def __init__(self, model_directory: str, config: Gemma4Config,
                 assistant_config: Optional[Gemma4AssistantConfig] = None,
                 quantize_fp8: bool = True):
        self._library = capi.library()
        self._handle = ctypes.c_void_p()
        model_config, self._shapes = model_config_struct(config)
        assistant = None
        if assistant_config is not None:
            assistant, self._kinds = assistant_config_struct(assistant_config)
        check(self._library.carat_b200_weights_load(
            model_directory.encode(), ctypes.byref(model_config),
            ctypes.byref(assistant) if assistant is not None else None,
            1 if quantize_fp8 else 0, ctypes.byref(self._handle)))
        tensors, self.fp8 = {}, Fp8WeightArena()
        for index in range(self._library.carat_b200_weights_segment_count(self._handle)):
            segment = capi.WeightSegment()
            check(self._library.carat_b200_weights_segment(self._handle, index,
                                                           ctypes.byref(segment)))
            name = segment.name.decode()
            shape = [int(segment.shape[axis]) for axis in range(segment.rank)]
            tensors[name] = torch.as_tensor(_DeviceView(segment.bf16, shape, "<u2"),
                                            device="cuda").view(torch.bfloat16)
            if segment.fp8:
                self.fp8.add(name,
                             torch.as_tensor(_DeviceView(segment.fp8, shape, "|u1"), device="cuda"),
                             torch.as_tensor(_DeviceView(segment.fp8_scale, [1], "<f4"),
                                             device="cuda"))
        self.bf16 = DeviceWeightArena(tensors)

    def int4_mlp_layers(self, group_width: int = 128):
        """Quantises every layer's gate_up and down matrices to weight-only INT4 on the device
        (carat_b200_weights_quantize_int4_mlp) and returns the per-layer array that
        carat_b200_runner_use_int4_mlp takes; the buffers belong to this object."""
        check(self._library.carat_b200_weights_quantize_int4_mlp(self._handle, group_width))
        count = ctypes.c_int(0)
        check(self._library.carat_b200_weights_int4_mlp_layers(self._handle, None, 0,
                                                               ctypes.byref(count), None))
        layers = (capi.Int4MlpLayer * count.value)()
        check(self._library.carat_b200_weights_int4_mlp_layers(self._handle, layers, count.value,
                                                               ctypes.byref(count), None))
        return layers

    def find(self, name: str) -> capi.WeightSegment:
        segment = capi.WeightSegment()
        check(self._library.carat_b200_weights_find(self._handle, name.encode(),
                                                    ctypes.byref(segment)))
        return segment

    def close(self) -> None:
        if self._handle:
            self.bf16 = None
            self.fp8 = None
            self._library.carat_b200_weights_destroy(self._handle)
            self._handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown
            pass


@dataclass
class GreedyVerificationResult:
    """include/carat/batch_model_runner.h:10-15."""

    accepted_tokens: List[int]
    next_tokens: List[int]


def _pointer(tensor: Optional[torch.Tensor]):
    return None if tensor is None else ctypes.c_void_p(tensor.data_ptr())


class Gemma4BatchModelRunner:
    """include/carat/batch_model_runner.h:22-77, the methods on the speculative-decoding path."""

    def __init__(self, config: Gemma4Config, weights: DeviceWeightArena, batch: int,
                 maximum_context: int, fp8_weights: Optional[Fp8WeightArena] = None,
                 assistant_weights: Optional[DeviceWeightArena] = None,
                 assistant_fp8_weights: Optional[Fp8WeightArena] = None,
                 assistant_config: Optional[Gemma4AssistantConfig] = None,
                 assistant_fp8_mode: Optional[str] = None):
        """assistant_fp8_mode: "off" (every drafter linear in bf16), "lm_head" or "all"; None reads
        CARAT_ASSISTANT_FP8_MODE like the reference does and falls back to its default, "off"
        (cuda/assistant_runner.cu:29-43)."""
        self._library = capi.library()
        self._handle = ctypes.c_void_p()
        if fp8_weights is None:
            raise CaratError("invalid greedy verification batch")  # FP8 weights are required
        self.config = config
        self._keep = [weights, fp8_weights, assistant_weights, assistant_fp8_weights]
        shapes = (capi.LayerShape * len(config.layers))()
        layer_weights = (capi.LayerWeights * len(config.layers))()
        for index, layer in enumerate(config.layers):
            shapes[index] = capi.LayerShape(1 if layer.attention == "global" else 0,
                                            layer.query_heads, layer.kv_heads,
                                            layer.head_dimension, layer.rope_theta,
                                            1 if layer.key_equals_value else 0)
            layer_weights[index] = self._layer_weights(weights, fp8_weights, f"layer.{index}.",
                                                       "qkv", True)
        model_config = capi.ModelConfig(config.hidden_size, config.intermediate_size,
                                        config.vocabulary_size, config.sliding_window,
                                        config.rms_norm_epsilon, len(config.layers), shapes)
        model_weights = capi.ModelWeights(
            weights.at("token_embedding").data_ptr(), fp8_weights.at("token_embedding").data_ptr(),
            fp8_weights.scale("token_embedding").data_ptr(), weights.at("final_norm").data_ptr(),
            layer_weights)
        assistant_struct = None
        assistant_weight_struct = None
        if assistant_fp8_mode is None:
            assistant_fp8_mode = os.environ.get("CARAT_ASSISTANT_FP8_MODE", "off")
        if assistant_fp8_mode not in ASSISTANT_FP8_MODES:
            raise CaratError("CARAT_ASSISTANT_FP8_MODE must be off, lm_head or all")
        if assistant_weights is not None:
            if assistant_fp8_mode != "off" and assistant_fp8_weights is None:
                raise CaratError("assistant FP8 mode requires quantized assistant weights")
            assistant_config = assistant_config or Gemma4AssistantConfig()
            kinds = (ctypes.c_int32 * len(assistant_config.layers))(
                *[1 if kind == "global" else 0 for kind in assistant_config.layers])
            a_layers = (capi.LayerWeights * len(assistant_config.layers))()
            for index in range(len(assistant_config.layers)):
                a_layers[index] = self._layer_weights(assistant_weights, assistant_fp8_weights,
                                                      f"layer.{index}.", "q", False)
            assistant_struct = capi.AssistantConfig(
                assistant_config.hidden_size, assistant_config.intermediate_size,
                assistant_config.query_heads, len(assistant_config.layers), kinds,
                assistant_config.rms_norm_epsilon)
            fp8 = assistant_fp8_weights
            if fp8 is not None:
                assistant_weight_struct = capi.AssistantWeights(
                    fp8.at("token_embedding").data_ptr(), fp8.scale("token_embedding").data_ptr(),
                    fp8.at("pre_projection").data_ptr(), fp8.scale("pre_projection").data_ptr(),
                    fp8.at("post_projection").data_ptr(), fp8.scale("post_projection").data_ptr(),
                    assistant_weights.at("final_norm").data_ptr(), a_layers)
            else:
                assistant_weight_struct = capi.AssistantWeights(
                    None, None, None, None, None, None,
                    assistant_weights.at("final_norm").data_ptr(), a_layers)
            self._keep += [kinds, a_layers]
        self._keep += [shapes, layer_weights]
        check(self._library.carat_b200_runner_create(
            ctypes.byref(model_config), ctypes.byref(model_weights), batch, maximum_context,
            ctypes.byref(assistant_struct) if assistant_struct is not None else None,
            ctypes.byref(assistant_weight_struct) if assistant_weight_struct is not None else None,
            ctypes.byref(self._handle)))
        self._assistant_weights = assistant_weights
        self._assistant_layer_count = len(assistant_config.layers) if assistant_config else 0
        if assistant_weights is not None:
            self.set_assistant_fp8_mode(assistant_fp8_mode)

    def set_assistant_fp8_mode(self, mode: str) -> None:
        """Drafter precision, the reference's CARAT_ASSISTANT_FP8_MODE: "off" and "lm_head" run the
        drafter's linears on the bf16 matrices of the assistant's DeviceWeightArena."""
        if mode not in ASSISTANT_FP8_MODES:
            raise CaratError("CARAT_ASSISTANT_FP8_MODE must be off, lm_head or all")
        bf16 = None
        if mode != "all":
            arena = self._assistant_weights
            layers = (capi.AssistantBf16Layer * self._assistant_layer_count)()
            for index in range(self._assistant_layer_count):
                prefix = f"layer.{index}."
                layers[index] = capi.AssistantBf16Layer(
                    arena.at(prefix + "q").data_ptr(), arena.at(prefix + "o").data_ptr(),
                    arena.at(prefix + "gate_up").data_ptr(), arena.at(prefix + "down").data_ptr())
            bf16 = capi.AssistantBf16Weights(arena.at("token_embedding").data_ptr(),
                                             arena.at("pre_projection").data_ptr(),
                                             arena.at("post_projection").data_ptr(), layers)
            self._keep.append(layers)
        check(self._library.carat_b200_runner_set_assistant_precision(
            self._handle, ASSISTANT_FP8_MODES[mode],
            ctypes.byref(bf16) if bf16 is not None else None))
        self.assistant_fp8_mode = mode

    @staticmethod
    def _layer_weights(weights, fp8, prefix, projection, has_key_norm) -> capi.LayerWeights:
        def bf16(name):
            return weights.at(prefix + name).data_ptr()

        if fp8 is None:     # a drafter without e4m3 matrices: norms only
            return capi.LayerWeights(
                bf16("input_norm"), bf16("q_norm"), bf16("k_norm") if has_key_norm else None,
                None, None, None, None, bf16("post_attention_norm"), bf16("pre_mlp_norm"),
                None, None, None, None, bf16("post_mlp_norm"), bf16("scalar"))
        return capi.LayerWeights(
            bf16("input_norm"), bf16("q_norm"), bf16("k_norm") if has_key_norm else None,
            fp8.at(prefix + projection).data_ptr(), fp8.scale(prefix + projection).data_ptr(),
            fp8.at(prefix + "o").data_ptr(), fp8.scale(prefix + "o").data_ptr(),
            bf16("post_attention_norm"), bf16("pre_mlp_norm"),
            fp8.at(prefix + "gate_up").data_ptr(), fp8.scale(prefix + "gate_up").data_ptr(),
            fp8.at(prefix + "down").data_ptr(), fp8.scale(prefix + "down").data_ptr(),
            bf16("post_mlp_norm"), bf16("scalar"))

    def close(self) -> None:
        if self._handle:
            self._library.carat_b200_runner_destroy(self._handle)
            self._handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown
            pass

    # ---- the speculative-decoding path
    def verify_greedy_proposals(self, proposals: Sequence[Sequence[int]],
                                target_first_tokens: Sequence[int], slots: Sequence[int],
                                maximum_accepted_tokens: Sequence[int] = (),
                                flags: int = 0) -> GreedyVerificationResult:
        requests = len(proposals)
        depth = len(proposals[0]) if requests else 0
        if requests == 0 or len(target_first_tokens) != requests or len(slots) != requests:
            raise CaratError("invalid greedy verification batch")
        if maximum_accepted_tokens and len(maximum_accepted_tokens) != requests:
            raise CaratError("speculative acceptance caps do not match request count")
        if any(len(row) != depth for row in proposals):
            raise CaratError("invalid or repeated speculative slot")
        flat = int_array([token for row in proposals for token in row])
        accepted = (ctypes.c_int * requests)()
        next_tokens = (ctypes.c_int * requests)()
        caps = int_array(maximum_accepted_tokens) if maximum_accepted_tokens else None
        check(self._library.carat_b200_runner_verify_greedy_proposals(
            self._handle, flat, requests, depth, int_array(target_first_tokens), int_array(slots),
            caps, flags, accepted, next_tokens))
        return GreedyVerificationResult(list(accepted), list(next_tokens))

    def append_ragged(self, token_ids: Sequence[int], slots: Sequence[int]) -> List[int]:
        """Plain decode, one token per listed slot; returns the greedy next tokens
        (Gemma4BatchModelRunner::append_ragged, cuda/batch_model_runner.cu:1544-1615)."""
        active = len(token_ids)
        if active == 0 or len(slots) != active:
            raise CaratError("invalid ragged token batch")
        next_tokens = (ctypes.c_int * active)()
        check(self._library.carat_b200_runner_append_ragged(
            self._handle, int_array(token_ids), int_array(slots), active, next_tokens))
        return list(next_tokens)

    def clone_slot(self, source_slot: int, destination_slot: int) -> int:
        """Copies a slot's resident KV rows, hand-off hidden row and position to another slot and
        returns the KV bytes copied (Gemma4BatchModelRunner::clone_slot,
        cuda/batch_model_runner.cu:1507-1542)."""
        copied = ctypes.c_uint64(0)
        check(self._library.carat_b200_runner_clone_slot(self._handle, source_slot,
                                                         destination_slot, ctypes.byref(copied)))
        return copied.value

    def has_assistant(self) -> bool:
        return bool(self._library.carat_b200_runner_has_assistant(self._handle))

    def draft_four(self, last_tokens: Sequence[int], slots: Sequence[int],
                   forced_first_tokens: Sequence[int] = (), depth: int = 4) -> List[List[int]]:
        requests = len(last_tokens)
        if requests == 0 or len(slots) != requests:
            raise CaratError("assistant is not configured or draft batch is invalid")
        if forced_first_tokens and len(forced_first_tokens) != requests:
            raise CaratError("forced assistant first tokens do not match draft batch")
        output = (ctypes.c_int * (requests * max(depth, 1)))()
        forced = int_array(forced_first_tokens) if forced_first_tokens else None
        check(self._library.carat_b200_runner_draft(self._handle, int_array(last_tokens),
                                                    int_array(slots), forced, requests, depth,
                                                    output))
        return [list(output[row * depth:(row + 1) * depth]) for row in range(requests)]

    # ---- BF16 prefill (cuda/batch_model_runner.cu:1048-1355)
    def set_bf16_weights(self, weights: Optional[DeviceWeightArena] = None) -> None:
        """Hands the target's bf16 matrices (layer.N.qkv / o / gate_up / down of the
        DeviceWeightArena the runner was built with, unless another arena is given) to the runner;
        BF16 prefill runs on them."""
        arena = weights or self._keep[0]
        layers = (capi.LayerBf16Weights * len(self.config.layers))()
        for index in range(len(self.config.layers)):
            prefix = f"layer.{index}."
            layers[index] = capi.LayerBf16Weights(
                arena.at(prefix + "qkv").data_ptr(), arena.at(prefix + "o").data_ptr(),
                arena.at(prefix + "gate_up").data_ptr(), arena.at(prefix + "down").data_ptr())
        check(self._library.carat_b200_runner_set_bf16_weights(self._handle, layers, len(layers)))
        self._keep.append(layers)
        self._has_bf16 = True

    def prefill_slots_chunks(self, slots: Sequence[int], token_ids: Sequence[Sequence[int]],
                             chunk_tokens: int) -> List[Optional[int]]:
        """One BF16 prefill chunk per listed slot; an entry holds the greedy next token only when
        that request's whole prompt became resident (Gemma4BatchModelRunner::prefill_slots_chunks)."""
        requests = len(slots)
        if requests == 0 or len(token_ids) != requests:
            raise CaratError("invalid batched chunk prefill shape")
        if not getattr(self, "_has_bf16", False):
            self.set_bf16_weights()
        arrays = [int_array(tokens) for tokens in token_ids]
        pointers = (ctypes.POINTER(ctypes.c_int) * requests)(*[
            ctypes.cast(array, ctypes.POINTER(ctypes.c_int)) for array in arrays])
        counts = int_array([len(tokens) for tokens in token_ids])
        predictions = (ctypes.c_int * requests)()
        has_prediction = (ctypes.c_int * requests)()
        check(self._library.carat_b200_runner_prefill_slots_chunks(
            self._handle, int_array(slots), pointers, counts, requests, chunk_tokens, predictions,
            has_prediction))
        return [predictions[r] if has_prediction[r] else None for r in range(requests)]

    def prefill_slot_chunk(self, slot: int, token_ids: Sequence[int],
                           chunk_tokens: int) -> Optional[int]:
        """Gemma4BatchModelRunner::prefill_slot_chunk (cuda/batch_model_runner.cu:1066-1125)."""
        if not token_ids or chunk_tokens <= 0:
            raise CaratError("invalid slot prefill chunk shape")
        return self.prefill_slots_chunks([slot], [token_ids], chunk_tokens)[0]

    def prefill_slot(self, slot: int, token_ids: Sequence[int], chunk_tokens: int = 1024) -> int:
        """Gemma4BatchModelRunner::prefill_slot (:1048-1052): reset the slot, prefill in BF16."""
        self.reset_slot(slot)
        return self.prefill_slot_from_prefix(slot, token_ids, 0, chunk_tokens)

    def prefill_slot_from_prefix(self, slot: int, token_ids: Sequence[int],
                                 cached_prefix_tokens: int, chunk_tokens: int = 1024) -> int:
        """:1054-1064: the first cached_prefix_tokens of token_ids are already resident."""
        if (not token_ids or chunk_tokens <= 0 or cached_prefix_tokens < 0
                or cached_prefix_tokens >= len(token_ids)
                or self.slot_position(slot) != cached_prefix_tokens):
            raise CaratError("invalid slot prefill shape")
        prediction = None
        while prediction is None:
            prediction = self.prefill_slot_chunk(slot, token_ids, chunk_tokens)
        return prediction

    def prefill_slots_suffix(self, slots: Sequence[int],
                             token_ids: Sequence[Sequence[int]]) -> List[int]:
        """Gemma4BatchModelRunner::prefill_slots_suffix (:1127-1228) for BF16 suffixes: whatever of
        each prompt is not resident yet, in one call."""
        if not slots or len(token_ids) != len(slots):
            raise CaratError("invalid batched suffix prefill shape")
        longest = max(len(tokens) for tokens in token_ids)
        return self.prefill_slots_chunks(slots, token_ids, max(longest, 1))

    def prefill_slot_fp8(self, slot: int, token_ids: Sequence[int], chunk_tokens: int = 8) -> int:
        next_token = ctypes.c_int(0)
        check(self._library.carat_b200_runner_prefill_slot_fp8(
            self._handle, slot, int_array(token_ids), len(token_ids), chunk_tokens,
            ctypes.byref(next_token)))
        return next_token.value

    def reset_slot(self, slot: int) -> None:
        check(self._library.carat_b200_runner_reset_slot(self._handle, slot))

    def seed_empty_cache_for_benchmark(self, position: int) -> None:
        check(self._library.carat_b200_runner_seed_empty_cache_for_benchmark(self._handle,
                                                                             position))

    def seed_slot_positions(self, positions: Sequence[int]) -> None:
        """Benchmark helper: zero KV and one context length per slot."""
        if len(positions) != self.batch():
            raise CaratError("invalid benchmark cache position")
        check(self._library.carat_b200_runner_seed_slot_positions(self._handle,
                                                                  int_array(positions)))

    def batch(self) -> int:
        return self._library.carat_b200_runner_batch(self._handle)

    def slot_position(self, slot: int) -> int:
        position = ctypes.c_int(0)
        check(self._library.carat_b200_runner_slot_position(self._handle, slot,
                                                            ctypes.byref(position)))
        return position.value

    # ---- inspection
    def last_predictions(self, count: int) -> List[int]:
        output = (ctypes.c_int * count)()
        check(self._library.carat_b200_runner_last_predictions(self._handle, output, count))
        return list(output)

    def device_pointer(self, which: int, layer: int = 0):
        """(address, bytes) of a runner-owned device buffer (carat_b200_runner_device_pointer)."""
        pointer = ctypes.c_void_p()
        size = ctypes.c_size_t(0)
        check(self._library.carat_b200_runner_device_pointer(self._handle, which, layer,
                                                             ctypes.byref(pointer),
                                                             ctypes.byref(size)))
        return pointer.value, size.value

    def _device_view(self, which: int, layer: int, shape) -> torch.Tensor:
        elements = 1
        for extent in shape:
            elements *= extent
        holder = torch.empty(elements, dtype=torch.bfloat16, device="cuda")
        check(self._library.carat_b200_runner_read(self._handle, which, layer, 0,
                                                   holder.data_ptr(), elements * 2))
        return holder.reshape(shape)

    def use_int4_mlp(self, weights: Optional[DeviceWeightArena], group_width: int = 128) -> None:
        """Switches the target's gate_up and down projections to weight-only INT4 linears built
        from the bf16 segments of `weights` (None switches back to the e4m3 linears). A step then
        takes at most 128 rows."""
        if weights is None:
            check(self._library.carat_b200_runner_use_int4_mlp(self._handle, None, 0, 0))
            self._int4 = None
            return
        if isinstance(weights, LoadedWeights):
            # The weight pipeline quantises on the device and keeps the buffers.
            layers = weights.int4_mlp_layers(group_width)
            check(self._library.carat_b200_runner_use_int4_mlp(self._handle, layers, len(layers),
                                                               group_width))
            self._int4 = (layers, weights)
            return
        hidden = self.config.hidden_size
        intermediate = self.config.intermediate_size
        layers = (capi.Int4MlpLayer * len(self.config.layers))()
        linears = []
        for index in range(len(self.config.layers)):
            gate_up = Int4Bf16Linear(weights.at(f"layer.{index}.gate_up"), hidden,
                                     2 * intermediate, group_width)
            down = Int4Bf16Linear(weights.at(f"layer.{index}.down"), intermediate, hidden,
                                  group_width)
            linears += [gate_up, down]
            layers[index].gate_up_codes = gate_up.reordered.data_ptr()
            layers[index].gate_up_scales = gate_up.scales.data_ptr()
            layers[index].down_codes = down.reordered.data_ptr()
            layers[index].down_scales = down.scales.data_ptr()
        torch.cuda.synchronize()
        check(self._library.carat_b200_runner_use_int4_mlp(self._handle, layers, len(layers),
                                                           group_width))
        self._int4 = (layers, linears)

    def write_cache(self, which: int, layer: int, values: torch.Tensor) -> None:
        """Overwrites a whole key (which = 0) or value (1) cache of `layer`, or the hidden-by-slot
        table (2), with bf16 `values` laid out like the runner's buffer."""
        data = values.to(dtype=torch.bfloat16).contiguous()
        check(self._library.carat_b200_runner_write(self._handle, which, layer, 0, data.data_ptr(),
                                                    data.numel() * 2))

    def key_cache(self, layer: int, capacity: int) -> torch.Tensor:
        shape = self.config.layers[layer]
        return self._device_view(0, layer, (self.batch(), shape.kv_heads, capacity,
                                            shape.head_dimension))

    def value_cache(self, layer: int, capacity: int) -> torch.Tensor:
        shape = self.config.layers[layer]
        return self._device_view(1, layer, (self.batch(), shape.kv_heads, capacity,
                                            shape.head_dimension))

    def target_hidden_slots(self) -> torch.Tensor:
        return self._device_view(2, 0, (self.batch(), self.config.hidden_size))

    def last_final_hidden(self, rows: int) -> torch.Tensor:
        return self._device_view(3, 0, (rows, self.config.hidden_size))

    def last_logits(self, rows: int) -> torch.Tensor:
        """bf16 logits [rows, vocabulary] of the last verify call. The step never stores logits
        (the LM head's epilogue keeps only the argmax), so they are recomputed here from the
        call's final-normed hidden rows with the same tensor-scale quantiser and FP8 linear
        (run_decode_lm_head, cuda/batch_model_runner.cu:840-853). Inspection only."""
        library = self._library
        hidden = self.last_final_hidden(rows)
        width, vocabulary = self.config.hidden_size, self.config.vocabulary_size
        fp8 = self._keep[1]
        quantised = torch.empty(rows, width, dtype=torch.uint8, device="cuda")
        scale = torch.zeros(1, dtype=torch.float32, device="cuda")
        scratch = torch.zeros(1, dtype=torch.int32, device="cuda")
        logits = torch.empty(rows, vocabulary, dtype=torch.bfloat16, device="cuda")
        needed = library.carat_b200_fp8_linear_workspace_bytes(rows, width, vocabulary)
        workspace = torch.empty(max(needed, 16), dtype=torch.uint8, device="cuda")
        stream = torch.cuda.current_stream().cuda_stream
        # The any-size form of the quantiser (same tensor-wide scale): more rows than the device
        # holds row CTAs at once (k = 8: 216 rows) do not fit the one-launch form.
        check(library.carat_b200_quantize_bf16_tensor_to_fp8(
            hidden.data_ptr(), quantised.data_ptr(), scale.data_ptr(), scratch.data_ptr(),
            rows * width, stream))
        check(library.carat_b200_fp8_linear(
            quantised.data_ptr(), scale.data_ptr(), fp8.at("token_embedding").data_ptr(),
            fp8.scale("token_embedding").data_ptr(), logits.data_ptr(), rows, width, vocabulary,
            workspace.data_ptr(), needed, stream))
        torch.cuda.synchronize()
        return logits

    def assistant_final_hidden(self, rows: int, width: int) -> torch.Tensor:
        return self._device_view(4, 0, (rows, width))

    def assistant_previous_hidden(self, rows: int) -> torch.Tensor:
        return self._device_view(5, 0, (rows, self.config.hidden_size))

    def last_device_ms(self):
        verify = ctypes.c_float(0)
        draft = ctypes.c_float(0)
        check(self._library.carat_b200_runner_last_device_ms(self._handle, ctypes.byref(verify),
                                                             ctypes.byref(draft)))
        return verify.value, draft.value

    def last_launches(self):
        verify = ctypes.c_int(0)
        draft = ctypes.c_int(0)
        check(self._library.carat_b200_runner_last_launches(self._handle, ctypes.byref(verify),
                                                            ctypes.byref(draft)))
        return verify.value, draft.value
