"""ctypes binding of oracle/_ref/libref_cuda.so: the reference's own CUDA operators and batch
runner, compiled unmodified for sm_100a by `make -C oracle ref_cuda` (test infrastructure only).

Tests that import this module skip when the library has not been built (it can only be built
where a checkout of the reference exists; the built file travels with the repository snapshot).
"""
import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_double, c_float, c_int, c_size_t, c_void_p

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBRARY_PATH = os.path.join(ROOT, "oracle", "_ref", "libref_cuda.so")
SHIM_LIBRARY_PATH = os.path.join(ROOT, "oracle", "_ref", "libshim_runner.so")

_P, _I, _F = c_void_p, c_int, c_float


class Segment(Structure):
    _fields_ = [("name", c_char_p), ("pointer", c_void_p), ("scale", c_void_p)]


class Layer(Structure):
    _fields_ = [("global_attention", c_int), ("query_heads", c_int), ("kv_heads", c_int),
                ("head_dimension", c_int), ("rotary_dimension", c_int), ("rope_theta", c_double),
                ("key_equals_value", c_int)]


SIGNATURES = {
    "ref_last_error": (c_char_p, []),
    "ref_quantize_bf16_to_fp8_e4m3": (_I, [_P, _P, _P, c_size_t]),
    "ref_quantize_bf16_to_fp8_e4m3_from_row_amax": (_I, [_P, _P, _P, _P, _I, _I]),
    "ref_quantize_bf16_to_fp8_e4m3_from_amax_values": (_I, [_P, _P, _P, _P, _I, _I, _I]),
    "ref_fp8_linear_run": (_I, [_P, _P, _P, _P, _P, _I, _I, _I]),
    "ref_fp8_linear_launch": (_I, [_P, _P, _P, _P, _P, _I, _I, _I]),
    "ref_quantize_argmax_launch": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I]),
    "ref_bf16_linear_run": (_I, [_P, _P, _P, _I, _I, _I]),
    "ref_rms_norm_bf16": (_I, [_P, _P, _P, c_size_t, c_size_t, _F]),
    "ref_rms_norm_bf16_with_row_amax": (_I, [_P, _P, _P, _P, c_size_t, c_size_t, _F]),
    "ref_rms_norm_add_and_norm_bf16": (_I, [_P, _P, _P, _P, _P, _P, c_size_t, c_size_t, _F]),
    "ref_rms_norm_add_and_norm_bf16_with_row_amax": (_I, [_P, _P, _P, _P, _P, _P, _P, c_size_t,
                                                         c_size_t, _F]),
    "ref_rms_norm_add_scale_bf16": (_I, [_P, _P, _P, _P, _P, c_size_t, c_size_t, _F]),
    "ref_gelu_tanh_gate_rows_bf16": (_I, [_P, _P, _I, _I]),
    "ref_gelu_tanh_gate_rows_bf16_with_block_amax": (_I, [_P, _P, _P, _I, _I]),
    "ref_reduce_block_amax_to_rows": (_I, [_P, _P, _I, _I]),
    "ref_embedding_batch_bf16": (_I, [_P, _P, _P, _I, _I, _I, _F]),
    "ref_token_to_head_batch_bf16": (_I, [_P, _P, _I, _I, _I, _I]),
    "ref_head_to_token_batch_bf16": (_I, [_P, _P, _I, _I, _I, _I]),
    "ref_head_to_token_batch_bf16_with_block_amax": (_I, [_P, _P, _P, _I, _I, _I, _I]),
    "ref_backup_kv_ring_spans_bf16": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I]),
    "ref_restore_kv_ring_suffixes_bf16": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I]),
    "ref_argmax_bf16_workspace_bytes": (c_size_t, [_I]),
    "ref_argmax_bf16_rows": (_I, [_P, _I, _I, _P, _P]),
    "ref_qkv_run_prefill_uniform_direct": (_I, [_I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I,
                                               _I, _I, _F]),
    "ref_qkv_run_prefill_uniform": (_I, [_I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I,
                                        _I, _F]),
    "ref_qkv_run_query_ragged": (_I, [_I, _P, _P, _P, _P, _I, _I, _I, _I, _F]),
    "ref_attention_run_uniform_batch": (_I, [_I, _I, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I,
                                            _I]),
    "ref_attention_run_uniform_ring_batch": (_I, [_I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _I, _I,
                                                 _I, _I, _I, _I]),
    "ref_decode_attention_run_ragged": (_I, [_I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I,
                                            _I, _I, _I]),
    "ref_runner_create": (c_void_p, [_I, _I, _I, _I, _I, c_double, POINTER(Layer), _I,
                                     POINTER(Segment), _I, POINTER(Segment), _I, _I, _I,
                                     POINTER(Segment), _I, POINTER(Segment), _I]),
    "ref_runner_destroy": (None, [_P]),
    "ref_runner_verify_greedy_proposals": (_I, [_P, POINTER(c_int), _I, _I, POINTER(c_int),
                                               POINTER(c_int), POINTER(c_int), POINTER(c_int),
                                               POINTER(c_int)]),
    "ref_runner_draft_four": (_I, [_P, POINTER(c_int), POINTER(c_int), POINTER(c_int), _I, _I,
                                   POINTER(c_int)]),
    "ref_runner_append_ragged": (_I, [_P, POINTER(c_int), POINTER(c_int), _I, POINTER(c_int)]),
    "ref_runner_clone_slot": (_I, [_P, _I, _I, POINTER(ctypes.c_ulonglong)]),
    "ref_runner_prefill_slot": (_I, [_P, _I, POINTER(c_int), _I, _I, POINTER(c_int)]),
    "ref_runner_prefill_slots_chunks": (_I, [_P, POINTER(c_int), POINTER(POINTER(c_int)),
                                            POINTER(c_int), _I, _I, POINTER(c_int),
                                            POINTER(c_int)]),
    "ref_runner_reset_slot": (_I, [_P, _I]),
    "ref_runner_seed_empty_cache_for_benchmark": (_I, [_P, _I]),
    "ref_runner_slot_position": (_I, [_P, _I, POINTER(c_int)]),
    "ref_assistant_create": (c_void_p, [POINTER(Segment), _I, POINTER(Segment), _I, _I, _I]),
    "ref_assistant_destroy": (None, [_P]),
    "ref_assistant_draft_four": (_I, [_P, _P, _P, POINTER(c_int), POINTER(c_int), POINTER(c_int),
                                      POINTER(c_int), _I, _I, _I, _P, _P, _I, _P, _P, _I,
                                      POINTER(c_int)]),
}

RUNNER_FACE = ("ref_last_error", "ref_runner_create", "ref_runner_destroy",
               "ref_runner_verify_greedy_proposals", "ref_runner_draft_four",
               "ref_runner_append_ragged", "ref_runner_clone_slot", "ref_runner_reset_slot",
               "ref_runner_prefill_slot", "ref_runner_prefill_slots_chunks",
               "ref_runner_seed_empty_cache_for_benchmark", "ref_runner_slot_position")

_library = None
_shim_library = None


def shim_library() -> ctypes.CDLL:
    """oracle/_ref/libshim_runner.so: this repository's drop-in C++ Gemma4BatchModelRunner
    (carat_b200/shim/) compiled against the reference's headers, behind the same C face."""
    global _shim_library
    if _shim_library is None:
        if not os.path.exists(SHIM_LIBRARY_PATH):
            pytest.skip("oracle/_ref/libshim_runner.so is not built (make -C oracle shim "
                        "REFERENCE=<carat checkout>)")
        loaded = ctypes.CDLL(SHIM_LIBRARY_PATH, mode=os.RTLD_NOW)
        for name in RUNNER_FACE:
            function = getattr(loaded, name)
            function.restype, function.argtypes = SIGNATURES[name]
        _shim_library = loaded
    return _shim_library


def available() -> bool:
    return os.path.exists(LIBRARY_PATH)


def library() -> ctypes.CDLL:
    """The loaded reference library; skips the calling test when it has not been built."""
    global _library
    if _library is None:
        if not available():
            pytest.skip("oracle/_ref/libref_cuda.so is not built (make -C oracle ref_cuda "
                        "REFERENCE=<carat checkout>)")
        loaded = ctypes.CDLL(LIBRARY_PATH, mode=os.RTLD_NOW)
        for name, (restype, argtypes) in SIGNATURES.items():
            function = getattr(loaded, name)
            function.restype = restype
            function.argtypes = argtypes
        _library = loaded
    return _library


class ReferenceError_(RuntimeError):
    """The reference threw; the text is its exception message."""


def check(status: int, loaded=None) -> None:
    if status != 0:
        message = (loaded or library()).ref_last_error()
        raise ReferenceError_(message.decode() if message else f"reference call failed ({status})")


def ints(values):
    values = list(values)
    return (c_int * len(values))(*values)


def _segments(table, scales=None):
    """name -> device tensor (and name -> scale tensor) as an array of Segment records."""
    names = sorted(table)
    array = (Segment * len(names))()
    for index, name in enumerate(names):
        array[index].name = name.encode()
        array[index].pointer = table[name].data_ptr()
        array[index].scale = scales[name].data_ptr() if scales is not None else None
    return array, len(names)


class ReferenceRunner:
    """carat::Gemma4BatchModelRunner itself (cuda/batch_model_runner.cu), fed device pointers the
    test owns through the reference's own arena interface."""

    def __init__(self, config, bf16, fp8, fp8_scales, batch, maximum_context, assistant_bf16=None,
                 assistant_fp8=None, assistant_fp8_scales=None, loaded=None):
        # `loaded` selects the implementation of the class behind the face: the reference's own
        # (default) or this repository's C++ shim (shim_library()).
        self._library = loaded or library()
        self._keep = (bf16, fp8, fp8_scales, assistant_bf16, assistant_fp8, assistant_fp8_scales)
        layers = (Layer * len(config.layers))()
        for index, layer in enumerate(config.layers):
            layers[index].global_attention = 1 if layer.attention == "global" else 0
            layers[index].query_heads = layer.query_heads
            layers[index].kv_heads = layer.kv_heads
            layers[index].head_dimension = layer.head_dimension
            layers[index].rotary_dimension = (layer.head_dimension // 4
                                              if layer.attention == "global"
                                              else layer.head_dimension)
            layers[index].rope_theta = layer.rope_theta
            layers[index].key_equals_value = 1 if layer.key_equals_value else 0
        bf16_array, bf16_count = _segments(bf16)
        fp8_array, fp8_count = _segments(fp8, fp8_scales)
        a_bf16_array, a_bf16_count = (None, 0)
        a_fp8_array, a_fp8_count = (None, 0)
        if assistant_bf16 is not None:
            a_bf16_array, a_bf16_count = _segments(assistant_bf16)
        if assistant_fp8 is not None:
            a_fp8_array, a_fp8_count = _segments(assistant_fp8, assistant_fp8_scales)
        self._arrays = (layers, bf16_array, fp8_array, a_bf16_array, a_fp8_array)
        self._handle = self._library.ref_runner_create(
            config.hidden_size, config.intermediate_size, config.vocabulary_size,
            config.sliding_window, maximum_context, config.rms_norm_epsilon, layers,
            len(config.layers), bf16_array, bf16_count, fp8_array, fp8_count, batch,
            maximum_context, a_bf16_array, a_bf16_count, a_fp8_array, a_fp8_count)
        if not self._handle:
            raise ReferenceError_(self._library.ref_last_error().decode())

    def _check(self, status):
        check(status, self._library)

    def close(self):
        if self._handle:
            self._library.ref_runner_destroy(self._handle)
            self._handle = None

    def __del__(self):
        self.close()

    def verify_greedy_proposals(self, proposals, target_first, slots, caps=None):
        requests, depth = len(proposals), len(proposals[0])
        flat = ints(token for row in proposals for token in row)
        accepted = (c_int * requests)()
        following = (c_int * requests)()
        self._check(self._library.ref_runner_verify_greedy_proposals(
            self._handle, flat, requests, depth, ints(target_first), ints(slots),
            ints(caps) if caps is not None else None, accepted, following))
        return list(accepted), list(following)

    def draft_four(self, last_tokens, slots, forced=None, depth=4):
        requests = len(last_tokens)
        out = (c_int * (requests * depth))()
        self._check(self._library.ref_runner_draft_four(
            self._handle, ints(last_tokens), ints(slots),
            ints(forced) if forced is not None else None, requests, depth, out))
        return [list(out[row * depth:(row + 1) * depth]) for row in range(requests)]

    def append_ragged(self, tokens, slots):
        out = (c_int * len(tokens))()
        self._check(self._library.ref_runner_append_ragged(self._handle, ints(tokens), ints(slots),
                                                     len(tokens), out))
        return list(out)

    def prefill_slot(self, slot, tokens, chunk_tokens=1024):
        out = c_int(0)
        self._check(self._library.ref_runner_prefill_slot(self._handle, slot, ints(tokens),
                                                          len(tokens), chunk_tokens,
                                                          ctypes.byref(out)))
        return out.value

    def prefill_slots_chunks(self, slots, token_ids, chunk_tokens):
        requests = len(slots)
        arrays = [ints(tokens) for tokens in token_ids]
        pointers = (POINTER(c_int) * requests)(*[ctypes.cast(a, POINTER(c_int)) for a in arrays])
        predictions = (c_int * requests)()
        has = (c_int * requests)()
        self._check(self._library.ref_runner_prefill_slots_chunks(
            self._handle, ints(slots), pointers, ints([len(t) for t in token_ids]), requests,
            chunk_tokens, predictions, has))
        return [predictions[r] if has[r] else None for r in range(requests)]

    def clone_slot(self, source, destination):
        copied = ctypes.c_ulonglong(0)
        self._check(self._library.ref_runner_clone_slot(self._handle, source, destination,
                                                  ctypes.byref(copied)))
        return copied.value

    def reset_slot(self, slot):
        self._check(self._library.ref_runner_reset_slot(self._handle, slot))

    def seed_empty_cache_for_benchmark(self, position):
        self._check(self._library.ref_runner_seed_empty_cache_for_benchmark(self._handle, position))

    def slot_position(self, slot):
        value = c_int(0)
        self._check(self._library.ref_runner_slot_position(self._handle, slot, ctypes.byref(value)))
        return value.value


class ReferenceAssistant:
    """carat::Gemma4AssistantRunner itself (cuda/assistant_runner.cu) over device memory the
    caller owns: the target embedding, the hidden-by-slot table and the two shared KV layers."""

    def __init__(self, bf16, fp8, fp8_scales, maximum_batch, maximum_context):
        self._library = library()
        self._keep = (bf16, fp8, fp8_scales)
        bf16_array, bf16_count = _segments(bf16)
        fp8_array, fp8_count = (None, 0)
        if fp8 is not None:
            fp8_array, fp8_count = _segments(fp8, fp8_scales)
        self._arrays = (bf16_array, fp8_array)
        self._handle = self._library.ref_assistant_create(bf16_array, bf16_count, fp8_array,
                                                          fp8_count, maximum_batch,
                                                          maximum_context)
        if not self._handle:
            raise ReferenceError_(self._library.ref_last_error().decode())

    def close(self):
        if self._handle:
            self._library.ref_assistant_destroy(self._handle)
            self._handle = None

    def __del__(self):
        self.close()

    def draft_four(self, target_embedding, hidden_by_slot, last_tokens, context_positions, slots,
                   forced, maximum_slots, depth, sliding_keys, sliding_values, sliding_capacity,
                   global_keys, global_values, global_capacity):
        requests = len(last_tokens)
        out = (c_int * (requests * depth))()
        check(self._library.ref_assistant_draft_four(
            self._handle, target_embedding, hidden_by_slot, ints(last_tokens),
            ints(context_positions), ints(slots), ints(forced) if forced is not None else None,
            requests, maximum_slots, depth, sliding_keys, sliding_values, sliding_capacity,
            global_keys, global_values, global_capacity, out))
        return [list(out[row * depth:(row + 1) * depth]) for row in range(requests)]
