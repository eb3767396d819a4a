"""The FP8 linear (reference: Fp8Linear::run, cuda/linear.cu:645-803) through the C ABI, over every
scheduling shape the plan can choose: one piece per tile, uniform split-K (fewer tiles than SMs),
a K-cut tail round (more tiles than SMs with a short last round), ragged feature counts, and the
fused argmax epilogue of the LM head.

Products of e4m3 values are exact in fp32 and the sums here stay far below 2^24 ulps of trouble,
but the accumulation order of a tensor-core K loop (and of split pieces) is not the oracle's, so
the bar is: bit-exact for almost every element, the rest one bf16 ulp away (measured at a floor
magnitude where sums cancel), against both the oracle and the plain one-thread-per-output
cross-check kernel.
"""
import ctypes

import pytest
import torch

import carat_b200
from carat_b200.capi import check
from helpers import one_ulp_apart
from oracle import carat_semantics as cs

pytestmark = pytest.mark.gpu


def ptr(tensor):
    return ctypes.c_void_p(tensor.data_ptr())


def quantised(rows, cols, std, seed):
    generator = torch.Generator(device="cuda").manual_seed(seed)
    values = (torch.randn(rows, cols, device="cuda", generator=generator) * std).to(torch.bfloat16)
    return carat_b200.quantize_tensor_to_fp8(values)


SHAPES = [
    (120, 5376, 16384, "one piece per tile"),
    (120, 8192, 5376, "uniform split-K"),
    (120, 1024, 20480, "K-cut tail round"),          # 160 tiles on 148 SMs
    (24, 1024, 8192 + 64, "ragged feature count"),
    (5, 256, 384, "few rows"),
    (64, 2048, 19072 + 128 * 20, "tail round, 64 padded rows"),
    (192, 1024, 20480, "192 padded rows, K-cut tail round"),
    (160, 2048, 5376, "192 padded rows, uniform split-K"),
]


@pytest.mark.parametrize("rows,k,n,what", SHAPES)
def test_linear_matches_oracle_and_cross_check(cuda_device, rows, k, n, what):
    library = carat_b200.library()
    weight, weight_scale = quantised(n, k, 0.02, 1)
    activation, activation_scale = quantised(rows, k, 1.0, 2)
    needed = library.carat_b200_fp8_linear_workspace_bytes(rows, k, n)
    if "split-K" in what or "tail round" in what:
        assert needed > 0, what
    workspace = torch.empty(max(needed, 16), dtype=torch.uint8, device="cuda")
    got = torch.full((rows, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    plain = torch.empty_like(got)
    check(library.carat_b200_fp8_linear(ptr(activation), ptr(activation_scale), ptr(weight),
                                        ptr(weight_scale), ptr(got), rows, k, n, ptr(workspace),
                                        needed, None))
    check(library.carat_b200_fp8_linear_check(ptr(activation), ptr(activation_scale), ptr(weight),
                                              ptr(weight_scale), ptr(plain), rows, k, n, None))
    torch.cuda.synchronize()
    code = ctypes.c_int(0)
    check(library.carat_b200_device_error(ctypes.byref(code)))
    assert code.value == 0
    want = cs.fp8_linear(activation.view(torch.float8_e4m3fn).float().cpu(),
                         activation_scale.cpu(), weight.view(torch.float8_e4m3fn).float().cpu(),
                         weight_scale.cpu())
    got_host = got.cpu()
    assert not torch.isnan(got_host.float()).any()
    for reference in (want.to(torch.bfloat16), plain.cpu()):
        assert float((got_host != reference).float().mean()) < 2e-3, what
        assert one_ulp_apart(got_host, reference), what


def test_lm_head_argmax_epilogue(cuda_device):
    library = carat_b200.library()
    rows, k, n = 120, 1024, 40000            # ragged last tile, several rounds of tiles
    weight, weight_scale = quantised(n, k, 0.02, 3)
    activation, activation_scale = quantised(rows, k, 1.0, 4)
    tokens = torch.empty(rows, dtype=torch.int32, device="cuda")
    keys = torch.empty(rows, dtype=torch.int64, device="cuda")
    check(library.carat_b200_fp8_linear_argmax(ptr(activation), ptr(activation_scale), ptr(weight),
                                               ptr(weight_scale), ptr(tokens), ptr(keys), rows, k,
                                               n, None))
    torch.cuda.synchronize()
    logits = cs.fp8_linear(activation.view(torch.float8_e4m3fn).float().cpu(),
                           activation_scale.cpu(), weight.view(torch.float8_e4m3fn).float().cpu(),
                           weight_scale.cpu())
    want = cs.argmax_lowest_index(logits)
    got = tokens.cpu().long()
    # A differing choice must be a tie or a one-ulp near-tie in the oracle's bf16 logits.
    for row in range(rows):
        if int(got[row]) != int(want[row]):
            best = float(logits[row, want[row]])
            chosen = float(logits[row, got[row]])
            assert abs(best - chosen) <= abs(best) * 2 ** -7, (row, best, chosen)
    assert float((got != want).float().mean()) < 0.05


def test_argmax_ties_take_the_lowest_index(cuda_device):
    """Equal logits: the reference's argmax keeps the lowest index (cuda/ops.cu:890-981)."""
    library = carat_b200.library()
    rows, k, n = 8, 128, 1024
    weight = torch.zeros(n, k, dtype=torch.uint8, device="cuda")
    one = torch.tensor([1.0]).to(torch.float8_e4m3fn).view(torch.uint8).item()
    # Features 700 and 300 get identical weights: a tie between them in every row.
    weight[700, :4] = one
    weight[300, :4] = one
    activation = torch.full((rows, k), one, dtype=torch.uint8, device="cuda")
    scale = torch.ones(1, dtype=torch.float32, device="cuda")
    tokens = torch.empty(rows, dtype=torch.int32, device="cuda")
    keys = torch.empty(rows, dtype=torch.int64, device="cuda")
    check(library.carat_b200_fp8_linear_argmax(ptr(activation), ptr(scale), ptr(weight), ptr(scale),
                                               ptr(tokens), ptr(keys), rows, k, n, None))
    torch.cuda.synchronize()
    assert tokens.cpu().tolist() == [300] * rows


GATED_SHAPES = [
    (120, 5376, 21504, "31B gate_up: 336 tiles, K-cut tail finished by the last piece"),
    (24, 1024, 64 * 160, "160 tiles, tail round, 32 padded rows"),
    (5, 256, 192, "three tiles"),
    (64, 2048, 64 * 300, "300 tiles, 64 padded rows"),
    (200, 512, 64 * 150, "150 tiles, 256 padded rows"),
    (150, 512, 64 * 160, "160 tiles, 192 padded rows"),
]


@pytest.mark.parametrize("rows,k,width,what", GATED_SHAPES)
def test_gated_linear_equals_linear_then_geglu(cuda_device, rows, k, width, what):
    """GeGLU in the gate_up linear's epilogue (carat_b200_fp8_linear_geglu) against the two separate
    operations it replaces, byte for byte: the activated bf16 rows, the tensor maximum, and the
    e4m3 rows and scale after the quantisation that follows."""
    library = carat_b200.library()
    weight, weight_scale = quantised(2 * width, k, 0.05, 11)
    activation, activation_scale = quantised(rows, k, 1.0, 12)
    # Separate: linear -> [rows, 2 * width] -> GeGLU + quantise.
    needed = library.carat_b200_fp8_linear_workspace_bytes(rows, k, 2 * width)
    workspace = torch.empty(max(needed, 16), dtype=torch.uint8, device="cuda")
    packed = torch.empty(rows, 2 * width, dtype=torch.bfloat16, device="cuda")
    check(library.carat_b200_fp8_linear(ptr(activation), ptr(activation_scale), ptr(weight),
                                        ptr(weight_scale), ptr(packed), rows, k, 2 * width,
                                        ptr(workspace), needed, None))
    want_fp8 = torch.empty(rows, width, dtype=torch.uint8, device="cuda")
    want_scale = torch.zeros(1, device="cuda")
    scratch = torch.zeros(1, dtype=torch.int32, device="cuda")
    check(library.carat_b200_gelu_gate_quantize(ptr(packed), ptr(want_fp8), ptr(want_scale),
                                                ptr(scratch), rows, width, None))
    # Fused, twice over the same workspace (the barrier word must come back to zero), once with
    # the quantisation in the same launch and once with it as a separate call.
    bytes_needed = library.carat_b200_fp8_linear_geglu_workspace_bytes(rows, k, width)
    gated_workspace = torch.empty(bytes_needed, dtype=torch.uint8, device="cuda")
    for attempt in range(2):
        activated = torch.full((rows, width), float("nan"), dtype=torch.bfloat16, device="cuda")
        amax_bits = torch.full((1,), 12345, dtype=torch.int32, device="cuda")
        got_fp8 = torch.empty(rows, width, dtype=torch.uint8, device="cuda")
        got_scale = torch.zeros(1, device="cuda")
        same_launch = attempt == 0
        check(library.carat_b200_fp8_linear_geglu(
            ptr(activation), ptr(activation_scale), ptr(weight), ptr(weight_scale), ptr(activated),
            ptr(amax_bits), ptr(got_fp8) if same_launch else None,
            ptr(got_scale) if same_launch else None, rows, k, width, ptr(gated_workspace),
            bytes_needed, None))
        if not same_launch:
            check(library.carat_b200_quantize_bf16_to_fp8_from_amax(
                ptr(activated), ptr(amax_bits), ptr(got_fp8), ptr(got_scale), rows * width, None))
        torch.cuda.synchronize()
        assert not torch.isnan(activated.float()).any(), what
        assert amax_bits.view(torch.float32).item() == activated.float().abs().max().item(), what
        # The two paths cut K differently for some features (a tile that is whole here may sit in
        # the other schedule's K-cut tail), so a sum can land one bf16 ulp away now and then:
        # nearly every byte equal, the rest one e4m3 step apart.
        assert torch.equal(got_scale, want_scale), what
        differing = got_fp8 != want_fp8
        assert float(differing.float().mean()) < 1e-4, what
        if bool(differing.any()):
            a = got_fp8.view(torch.float8_e4m3fn).float()[differing]
            b = want_fp8.view(torch.float8_e4m3fn).float()[differing]
            assert float(((a - b).abs() / torch.maximum(a.abs(), b.abs()).clamp_min(2 ** -9)).max()) \
                <= 0.126, what
    code = ctypes.c_int(0)
    check(library.carat_b200_device_error(ctypes.byref(code)))
    assert code.value == 0
