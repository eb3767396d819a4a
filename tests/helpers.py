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


def one_ulp_apart(got: torch.Tensor, want: torch.Tensor) -> bool:
    """Every element within one bf16 ulp of the reference. Near a cancellation (|value| far below
    the tensor's typical magnitude) an ulp of the value itself is meaningless, because the fp32
    partial sums that cancelled were rounded at their own, larger magnitude; the ulp of 1/16 of
    the tensor's rms is the floor there."""
    got = got.float()
    want = want.float()
    floor = want.pow(2).mean().sqrt() / 16
    allowed = torch.maximum(want.abs(), floor) * 2.0 ** -7
    return bool(((got - want).abs() <= allowed).all())


def int4_reference_test_case():
    """Weights and input of tests/cuda_ops_tests.cu:811-850, recomputed from their formulas."""
    rows, input_width, output_width = 17, 512, 256
    index = torch.arange(output_width * input_width, dtype=torch.float32)
    amplitude = torch.where(index % input_width < 256, 1.0, 16.0)
    weight = amplitude * (2.75 * torch.sin(index * 0.071) + 0.31 * torch.cos(index * 0.013))
    cell = torch.arange(rows * input_width, dtype=torch.float32)
    column = cell % input_width
    value = 0.75 * torch.sin(cell * 0.037) - 0.21 * torch.cos(column * 0.019)
    return (cs.bf16(weight).reshape(output_width, input_width),
            cs.bf16(value).reshape(rows, input_width))
