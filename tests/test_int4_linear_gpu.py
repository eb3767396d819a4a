"""The weight-only INT4 linear (reference: Int4Bf16Linear, include/carat/linear.h:70-90,
cuda/int4_bf16_linear.cu) through the C ABI: the quantiser must reproduce the reference's rule bit
for bit (codes, bf16 group scales, both layouts), the linear must match the oracle's
bf16(X . bf16(code * scale)^T) over every scheduling shape, and the reference's own test case
(tests/cuda_ops_tests.cu:811-914: 17 rows, 512 -> 256, groups of 256, closed-form weights whose
second group is sixteen times larger) is held to that test's bar and to the tighter one used here.
"""
import ctypes
import math

import pytest
import torch

import carat_b200
from carat_b200.capi import check
from helpers import cosine, int4_reference_test_case, one_ulp_apart
from oracle import carat_semantics as cs

pytestmark = pytest.mark.gpu


def ptr(tensor):
    return ctypes.c_void_p(tensor.data_ptr())


def device_int4(weight, group_width):
    output_width, input_width = weight.shape
    return carat_b200.Int4Bf16Linear(weight.to(torch.bfloat16).cuda(), input_width, output_width,
                                     group_width)


@pytest.mark.parametrize("group_width", [128, 256])
def test_quantiser_matches_the_reference_rule(cuda_device, group_width):
    generator = torch.Generator().manual_seed(3)
    weight = cs.bf16(torch.randn(384, 1024, generator=generator) * 0.02)
    weight[5, :group_width] = 0                      # an all-zero group: scale 1, codes 0
    weight[7, group_width:2 * group_width] *= 40     # a group with a large range
    weight = cs.bf16(weight)
    linear = device_int4(weight, group_width)
    codes, scales = cs.int4_quantize(weight, group_width)
    assert torch.equal(linear.scales.float().cpu(), scales)
    assert torch.equal(linear.packed.cpu(), cs.int4_pack(codes))
    assert float(scales[0, 5]) == 1.0 and int(codes[5, :group_width].abs().max()) == 0
    assert int(codes.abs().max()) == 7


def run_both(linear, packed_input):
    library = carat_b200.library()
    rows = packed_input.shape[0]
    got = linear.run(packed_input)
    plain = torch.empty_like(got)
    check(library.carat_b200_int4_linear_check(
        ptr(packed_input), ptr(linear.packed), ptr(linear.scales), ptr(plain), rows,
        linear.input_width, linear.output_width, linear.group_width, None))
    torch.cuda.synchronize()
    code = ctypes.c_int(0)
    check(library.carat_b200_device_error(ctypes.byref(code)))
    assert code.value == 0
    return got.cpu(), plain.cpu()


def test_reference_test_case(cuda_device):
    weight, activation = int4_reference_test_case()
    linear = device_int4(weight, 256)
    got, plain = run_both(linear, activation.to(torch.bfloat16).cuda())
    codes, scales = cs.int4_quantize(weight, 256)
    want = cs.int4_bf16_linear(activation, codes, scales, 256)
    # The reference's bar: cosine >= 0.999 per row and at most one differing row argmax.
    for row in range(want.shape[0]):
        assert cosine(got[row].float(), want[row]) >= 0.999
    assert int((got.float().argmax(dim=1) != want.argmax(dim=1)).sum()) <= 1
    # This build's bar: same values up to the accumulation order.
    for reference in (want.to(torch.bfloat16), plain):
        assert float((got != reference).float().mean()) < 2e-3
        assert one_ulp_apart(got, reference)


SHAPES = [
    (120, 5376, 16384, 128, "one piece per tile"),
    (120, 21504, 5376, 128, "uniform split-K"),
    (120, 1024, 20480, 128, "K-cut tail round"),
    (24, 1024, 8192 + 64, 256, "ragged feature count, 32 padded rows"),
    (5, 256, 384, 128, "few rows"),
    (64, 2048, 4096, 256, "64 padded rows, groups of 256"),
    (128, 512, 1024, 128, "full 128 rows"),
]


@pytest.mark.parametrize("rows,k,n,group_width,what", SHAPES)
def test_linear_matches_oracle_and_cross_check(cuda_device, rows, k, n, group_width, what):
    library = carat_b200.library()
    generator = torch.Generator().manual_seed(11)
    weight = cs.bf16(torch.randn(n, k, generator=generator) * 0.02)
    activation = cs.bf16(torch.randn(rows, k, generator=generator))
    linear = device_int4(weight, group_width)
    needed = library.carat_b200_int4_linear_workspace_bytes(rows, k, n)
    if what in ("uniform split-K", "K-cut tail round"):
        assert needed > 0, what
    got, plain = run_both(linear, activation.to(torch.bfloat16).cuda())
    assert not torch.isnan(got.float()).any()
    codes, scales = cs.int4_quantize(weight, group_width)
    assert torch.equal(linear.packed.cpu(), cs.int4_pack(codes))
    want = cs.int4_bf16_linear(activation, codes, scales, group_width)
    for reference in (want.to(torch.bfloat16), plain):
        assert float((got != reference).float().mean()) < 4e-3, what
        assert one_ulp_apart(got, reference), what


def test_argument_errors_carry_the_reference_messages(cuda_device):
    weight = torch.zeros(256, 512, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(carat_b200.CaratError, match="invalid BF16 INT4 linear weight shape"):
        carat_b200.Int4Bf16Linear(weight, 512, 256, 64)
    linear = carat_b200.Int4Bf16Linear(weight, 512, 256, 256)
    with pytest.raises(carat_b200.CaratError, match="invalid BF16 INT4 linear activation shape"):
        linear.run(torch.zeros(129, 512, dtype=torch.bfloat16, device="cuda"))
    assert math.isclose(linear.allocated_bytes(), 256 * 512 / 2 + 2 * 256 * 2)
