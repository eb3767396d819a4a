"""Shared pieces of the parity tests: moving oracle tensors to the device runner and comparing."""
import torch

import carat_b200
from oracle import carat_semantics as cs


def runner_config(config: cs.ModelConfig) -> carat_b200.Gemma4Config:
    layers = [carat_b200.Gemma4LayerConfig(layer.kind, layer.query_heads, layer.kv_heads,
                                           layer.head_dim, layer.rope_theta, layer.key_equals_value)
              for layer in config.layers]
    return carat_b200.Gemma4Config(config.hidden, config.intermediate, config.vocab, config.window,
                                   config.eps, layers)


def assistant_config(assistant: cs.AssistantConfig) -> carat_b200.Gemma4AssistantConfig:
    return carat_b200.Gemma4AssistantConfig(assistant.hidden, assistant.intermediate,
                                            assistant.query_heads, list(assistant.layers),
                                            assistant.eps)


def build_pair(config, weights, slots, assistant=None, assistant_weights=None):
    """An oracle runner and a device runner over the same weights."""
    oracle = cs.OracleRunner(config, weights, slots, assistant, assistant_weights)
    arena = carat_b200.DeviceWeightArena.from_host(weights)
    fp8 = carat_b200.Fp8WeightArena.quantize(arena)
    a_arena = a_fp8 = a_config = None
    if assistant is not None:
        a_arena = carat_b200.DeviceWeightArena.from_host(assistant_weights)
        a_fp8 = carat_b200.Fp8WeightArena.quantize(a_arena)
        a_config = assistant_config(assistant)
    device = carat_b200.Gemma4BatchModelRunner(runner_config(config), arena, slots,
                                               config.max_context, fp8, a_arena, a_fp8, a_config)
    return oracle, device, fp8


def relative_error(actual: torch.Tensor, expected: torch.Tensor) -> float:
    """Largest |a - e| relative to the tensor's own scale (max |e|)."""
    actual = actual.float().cpu()
    expected = expected.float().cpu()
    return float((actual - expected).abs().max() / expected.abs().max().clamp_min(1e-12))


def cosine(actual: torch.Tensor, expected: torch.Tensor) -> float:
    actual = actual.float().cpu().reshape(-1)
    expected = expected.float().cpu().reshape(-1)
    return float(torch.nn.functional.cosine_similarity(actual, expected, dim=0))


def rms_relative_error(actual: torch.Tensor, expected: torch.Tensor) -> float:
    """||a - e|| / ||e||: the norm-wise relative error of a tensor."""
    actual = actual.float().cpu().reshape(-1)
    expected = expected.float().cpu().reshape(-1)
    return float((actual - expected).norm() / expected.norm().clamp_min(1e-12))
