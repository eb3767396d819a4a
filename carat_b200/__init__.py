"""carat_b200: the speculative-decoding step of the Carat Gemma-4 runtime for NVIDIA B200.

The product is libcarat_b200.so (hand-written sm_100a CUDA behind the C ABI of
include/carat_b200.h); this package holds its sources, its build recipe and a thin host-side
mirror of the reference's runner interface.
"""
from .capi import CaratError, library  # noqa: F401
from . import dispatcher, runner  # noqa: F401
from .runner import (DeviceWeightArena, Fp8WeightArena, Gemma4AssistantConfig,  # noqa: F401
                     Gemma4BatchModelRunner, Gemma4Config, Gemma4LayerConfig,
                     GreedyVerificationResult, Int4Bf16Linear, LoadedWeights, VERIFY_ASSUME_MATCH,
                     quantize_tensor_to_fp8)
