"""ctypes binding of libcarat_b200.so (the C ABI declared in include/carat_b200.h).

Loading fails loudly when the library has not been built: there is no fallback path.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_size_t, c_void_p

_PACKAGE = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(_PACKAGE, "libcarat_b200.so")


class CaratError(RuntimeError):
    """A C entry point returned a failure; the text is carat_b200_last_error()."""


class LayerShape(Structure):
    _fields_ = [("global_attention", c_int32), ("query_heads", c_int32), ("kv_heads", c_int32),
                ("head_dim", c_int32), ("rope_theta", c_float), ("key_equals_value", c_int32)]


class ModelConfig(Structure):
    _fields_ = [("hidden_size", c_int32), ("intermediate_size", c_int32),
                ("vocabulary_size", c_int32), ("sliding_window", c_int32),
                ("rms_norm_epsilon", c_float), ("layer_count", c_int32),
                ("layers", POINTER(LayerShape))]


class LayerWeights(Structure):
    _fields_ = [("input_norm", c_void_p), ("q_norm", c_void_p), ("k_norm", c_void_p),
                ("qkv", c_void_p), ("qkv_scale", c_void_p), ("o", c_void_p), ("o_scale", c_void_p),
                ("post_attention_norm", c_void_p), ("pre_mlp_norm", c_void_p),
                ("gate_up", c_void_p), ("gate_up_scale", c_void_p), ("down", c_void_p),
                ("down_scale", c_void_p), ("post_mlp_norm", c_void_p), ("scalar", c_void_p)]


class Int4MlpLayer(Structure):
    _fields_ = [("gate_up_codes", c_void_p), ("gate_up_scales", c_void_p),
                ("down_codes", c_void_p), ("down_scales", c_void_p)]


class SlotView(Structure):
    _fields_ = [("cached_tokens", POINTER(c_int)), ("cached_count", c_int32),
                ("occupied", c_int32), ("age", ctypes.c_uint64), ("prefilling", c_int32)]


class ReplicaView(Structure):
    _fields_ = [("slots", POINTER(SlotView)), ("slot_count", c_int32),
                ("queued_requests", c_int32), ("alive", c_int32)]


class Placement(Structure):
    _fields_ = [("decision", c_int32), ("replica", c_int32), ("destination", c_int32),
                ("source", c_int32), ("prefix_tokens", ctypes.c_uint64)]


class WeightSegment(Structure):
    _fields_ = [("name", ctypes.c_char * 96), ("rank", c_int32),
                ("shape", ctypes.c_uint64 * 2), ("arena_offset", ctypes.c_uint64),
                ("byte_size", ctypes.c_uint64), ("bf16", c_void_p), ("fp8", c_void_p),
                ("fp8_scale", c_void_p)]


class LayerBf16Weights(Structure):
    _fields_ = [("qkv", c_void_p), ("o", c_void_p), ("gate_up", c_void_p), ("down", c_void_p)]


class AssistantBf16Layer(Structure):
    _fields_ = [("q", c_void_p), ("o", c_void_p), ("gate_up", c_void_p), ("down", c_void_p)]


class AssistantBf16Weights(Structure):
    _fields_ = [("token_embedding", c_void_p), ("pre_projection", c_void_p),
                ("post_projection", c_void_p), ("layers", POINTER(AssistantBf16Layer))]


class ModelWeights(Structure):
    _fields_ = [("token_embedding", c_void_p), ("token_embedding_fp8", c_void_p),
                ("token_embedding_scale", c_void_p), ("final_norm", c_void_p),
                ("layers", POINTER(LayerWeights))]


class AssistantConfig(Structure):
    _fields_ = [("hidden_size", c_int32), ("intermediate_size", c_int32), ("query_heads", c_int32),
                ("layer_count", c_int32), ("layer_global", POINTER(c_int32)),
                ("rms_norm_epsilon", c_float)]


class AssistantWeights(Structure):
    _fields_ = [("token_embedding", c_void_p), ("token_embedding_scale", c_void_p),
                ("pre_projection", c_void_p), ("pre_projection_scale", c_void_p),
                ("post_projection", c_void_p), ("post_projection_scale", c_void_p),
                ("final_norm", c_void_p), ("layers", POINTER(LayerWeights))]


# name -> (restype, argtypes); every symbol include/carat_b200.h declares.
_P = c_void_p
_I = c_int
_F = c_float
_IP = POINTER(c_int)
SIGNATURES = {
    "carat_b200_last_error": (c_char_p, []),
    "carat_b200_abi_version": (_I, []),
    "carat_b200_device_error": (_I, [_IP]),
    "carat_b200_selftest_bounded_wait": (_I, [_P, _P]),
    "carat_b200_fp8_linear": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _P, c_size_t, _P]),
    "carat_b200_fp8_linear_workspace_bytes": (c_size_t, [_I, _I, _I]),
    "carat_b200_fp8_linear_geglu": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P, c_size_t, _P]),
    "carat_b200_fp8_linear_geglu_workspace_bytes": (c_size_t, [_I, _I, _I]),
    "carat_b200_fp8_linear_static": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _P]),
    "carat_b200_fp8_linear_argmax": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _P]),
    "carat_b200_fp8_linear_check": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _P]),
    "carat_b200_bf16_linear": (_I, [_P, _P, _P, _I, _I, _I, _P, c_size_t, _P]),
    "carat_b200_bf16_linear_workspace_bytes": (c_size_t, [_I, _I, _I]),
    "carat_b200_bf16_linear_argmax": (_I, [_P, _P, _P, _P, _I, _I, _I, _P]),
    "carat_b200_int4_quantize_weight": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "carat_b200_int4_reorder_weight": (_I, [_P, _P, _I, _I, _P]),
    "carat_b200_int4_linear": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _P, c_size_t, _P]),
    "carat_b200_int4_linear_workspace_bytes": (c_size_t, [_I, _I, _I]),
    "carat_b200_int4_linear_check": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "carat_b200_quantize_bf16_to_fp8": (_I, [_P, _P, _P, _P, _I, _I, _P]),
    "carat_b200_quantize_bf16_to_fp8_from_amax": (_I, [_P, _P, _P, _P, c_size_t, _P]),
    "carat_b200_quantize_bf16_tensor_to_fp8": (_I, [_P, _P, _P, _P, c_size_t, _P]),
    "carat_b200_rms_norm_quantize": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _F, _P]),
    "carat_b200_rms_norm_add_and_norm_quantize": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _F,
                                                      _P]),
    "carat_b200_gelu_gate_quantize": (_I, [_P, _P, _P, _P, _I, _I, _P]),
    "carat_b200_rms_norm_add_scale_then_norm_quantize": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P,
                                                             _P, _I, _I, _F, _P]),
    "carat_b200_rope_tables": (_I, [_P, _P, _I, _I, _F, _I, _P]),
    "carat_b200_qkv_postprocess": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I,
                                       _I, _F, _P]),
    "carat_b200_verify_attention": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I,
                                        _I, _I, _P]),
    "carat_b200_verify_attention_check": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I,
                                              _I, _I, _I, _I, _P]),
    "carat_b200_backup_kv_ring_spans": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "carat_b200_restore_kv_ring_suffixes": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "carat_b200_argmax_bf16_rows": (_I, [_P, _I, _I, _P, _P]),
    "carat_b200_greedy_prefix_accept": (_I, [_P, _P, _P, _P, _I, _I, _P, _P, _P]),
    "carat_b200_runner_create": (_I, [POINTER(ModelConfig), POINTER(ModelWeights), _I, _I,
                                     POINTER(AssistantConfig), POINTER(AssistantWeights),
                                     POINTER(c_void_p)]),
    "carat_b200_runner_destroy": (None, [_P]),
    "carat_b200_select_placement": (_I, [_IP, _I, POINTER(SlotView), _I, _I, POINTER(Placement)]),
    "carat_b200_route_request": (_I, [_IP, _I, POINTER(ReplicaView), _I, _I, POINTER(Placement)]),
    "carat_b200_weights_quantize_int4_mlp": (_I, [_P, _I]),
    "carat_b200_weights_int4_mlp_layers": (_I, [_P, POINTER(Int4MlpLayer), _I, _IP, _IP]),
    "carat_b200_weights_load": (_I, [c_char_p, POINTER(ModelConfig), POINTER(AssistantConfig), _I,
                                    POINTER(c_void_p)]),
    "carat_b200_weights_destroy": (None, [_P]),
    "carat_b200_weights_segment_count": (_I, [_P]),
    "carat_b200_weights_segment": (_I, [_P, _I, POINTER(WeightSegment)]),
    "carat_b200_weights_find": (_I, [_P, c_char_p, POINTER(WeightSegment)]),
    "carat_b200_weights_plan_text": (_I, [c_char_p, POINTER(ModelConfig), POINTER(AssistantConfig),
                                         c_char_p, c_size_t, POINTER(c_size_t)]),
    "carat_b200_runner_set_bf16_weights": (_I, [_P, POINTER(LayerBf16Weights), _I]),
    "carat_b200_runner_prefill_slots_chunks": (_I, [_P, _IP, POINTER(_IP), _IP, _I, _I, _IP, _IP]),
    "carat_b200_runner_set_assistant_precision": (_I, [_P, _I, POINTER(AssistantBf16Weights)]),
    "carat_b200_runner_use_int4_mlp": (_I, [_P, POINTER(Int4MlpLayer), _I, _I]),
    "carat_b200_runner_verify_greedy_proposals": (_I, [_P, _IP, _I, _I, _IP, _IP, _IP, _I, _IP,
                                                      _IP]),
    "carat_b200_runner_append_ragged": (_I, [_P, _IP, _IP, _I, _IP]),
    "carat_b200_runner_clone_slot": (_I, [_P, _I, _I, ctypes.POINTER(ctypes.c_uint64)]),
    "carat_b200_runner_draft": (_I, [_P, _IP, _IP, _IP, _I, _I, _IP]),
    "carat_b200_runner_prefill_slot_fp8": (_I, [_P, _I, _IP, _I, _I, _IP]),
    "carat_b200_runner_reset_slot": (_I, [_P, _I]),
    "carat_b200_runner_seed_empty_cache_for_benchmark": (_I, [_P, _I]),
    "carat_b200_runner_seed_slot_positions": (_I, [_P, _IP]),
    "carat_b200_runner_batch": (_I, [_P]),
    "carat_b200_runner_slot_position": (_I, [_P, _I, _IP]),
    "carat_b200_runner_has_assistant": (_I, [_P]),
    "carat_b200_runner_last_predictions": (_I, [_P, _IP, _I]),
    "carat_b200_runner_device_pointer": (_I, [_P, _I, _I, POINTER(c_void_p), POINTER(c_size_t)]),
    "carat_b200_runner_read": (_I, [_P, _I, _I, c_size_t, _P, c_size_t]),
    "carat_b200_runner_write": (_I, [_P, _I, _I, c_size_t, _P, c_size_t]),
    "carat_b200_runner_last_device_ms": (_I, [_P, POINTER(c_float), POINTER(c_float)]),
    "carat_b200_runner_last_launches": (_I, [_P, _IP, _IP]),
}

STATIC_SCRATCH_BYTES = 8 * 1024 * 1024  # CARAT_B200_STATIC_SCRATCH_BYTES

_library = None


def library() -> ctypes.CDLL:
    """The loaded shared library with argument types set. Raises when it is missing."""
    global _library
    if _library is None:
        if not os.path.exists(LIBRARY_PATH):
            raise CaratError(
                f"{LIBRARY_PATH} is missing: build it with `python -m carat_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        loaded = ctypes.CDLL(LIBRARY_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            function = getattr(loaded, name)
            function.restype = restype
            function.argtypes = argtypes
        _library = loaded
    return _library


def check(status: int) -> None:
    if status != 0:
        message = library().carat_b200_last_error()
        raise CaratError(message.decode() if message else f"carat_b200 call failed ({status})")


def int_array(values):
    """A C int array of the values; a ctypes int array is passed through as it is, so a caller
    that hands the same long sequence to many calls (a prompt, quantum after quantum) can convert
    it once."""
    if isinstance(values, ctypes.Array) and values._type_ is c_int:
        return values
    values = list(values)
    return (c_int * len(values))(*values)
