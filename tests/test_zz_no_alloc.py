"""carat_b200_fp8_linear_static: the FP8 linear for hosts that may not allocate device memory
(frozen-allocator serving loops, fixed-budget plugins). Its split-K scratch is an array inside the
library, so it must give exactly what carat_b200_fp8_linear gives with a caller-provided
workspace, call after call, agree with the CPU oracle, allocate nothing, and refuse shapes the
array cannot hold.

This file is collected last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

import carat_b200
from carat_b200 import capi
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


def test_static_scratch_linear_matches_workspace_linear_twice(cuda_device):
    library = carat_b200.library()
    rows, k, n = 120, 8192, 5376            # split-K shape: 3 x 120 x 5376 fp32 partial sums
    needed = library.carat_b200_fp8_linear_workspace_bytes(rows, k, n)
    assert 0 < needed <= capi.STATIC_SCRATCH_BYTES
    weight, weight_scale = quantised(n, k, 0.02, 1)
    workspace = torch.empty(needed, dtype=torch.uint8, device="cuda")
    for call in range(2):                    # two calls in a row share the built-in array
        activation, activation_scale = quantised(rows, k, 1.0, 10 + call)
        want = torch.empty(rows, n, dtype=torch.bfloat16, device="cuda")
        got = torch.full((rows, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        check(library.carat_b200_fp8_linear(ptr(activation), ptr(activation_scale), ptr(weight),
                                            ptr(weight_scale), ptr(want), rows, k, n,
                                            ptr(workspace), needed, None))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        check(library.carat_b200_fp8_linear_static(ptr(activation), ptr(activation_scale),
                                                   ptr(weight), ptr(weight_scale), ptr(got), rows,
                                                   k, n, None))
        torch.cuda.synchronize()
        if call == 1:
            # Once warmed up the call leaves the device's free memory exactly where it was.
            assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))   # bit-exact
        assert float(want.float().abs().max()) > 0.0
        # And both agree with the CPU oracle's FP8 linear to one bf16 ulp.
        oracle = cs.fp8_linear(activation.view(torch.float8_e4m3fn).float().cpu(),
                               activation_scale.cpu(), weight.view(torch.float8_e4m3fn).float().cpu(),
                               weight_scale.cpu())
        assert one_ulp_apart(got.float().cpu(), oracle)
        code = ctypes.c_int(-1)
        check(library.carat_b200_device_error(ctypes.byref(code)))
        assert code.value == 0                # no bounded wait ran out, in either error word


def test_static_scratch_linear_without_split_and_oversize_rejection(cuda_device):
    library = carat_b200.library()
    rows, k, n = 24, 1024, 16384            # 128 feature tiles: no split-K, no scratch needed
    weight, weight_scale = quantised(n, k, 0.02, 2)
    activation, activation_scale = quantised(rows, k, 1.0, 3)
    want = torch.empty(rows, n, dtype=torch.bfloat16, device="cuda")
    got = torch.empty_like(want)
    check(library.carat_b200_fp8_linear(ptr(activation), ptr(activation_scale), ptr(weight),
                                        ptr(weight_scale), ptr(want), rows, k, n, None, 0, None))
    check(library.carat_b200_fp8_linear_static(ptr(activation), ptr(activation_scale), ptr(weight),
                                               ptr(weight_scale), ptr(got), rows, k, n, None))
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))

    rows, k, n = 128, 16384, 9216           # 2 x 128 x 9216 fp32 = 9.4 MB > the 8 MiB array
    assert (library.carat_b200_fp8_linear_workspace_bytes(rows, k, n) >
            capi.STATIC_SCRATCH_BYTES)
    weight = torch.zeros(n, k, dtype=torch.uint8, device="cuda")
    activation = torch.zeros(rows, k, dtype=torch.uint8, device="cuda")
    scale = torch.ones(1, dtype=torch.float32, device="cuda")
    out = torch.zeros(rows, n, dtype=torch.bfloat16, device="cuda")
    status = library.carat_b200_fp8_linear_static(ptr(activation), ptr(scale), ptr(weight),
                                                  ptr(scale), ptr(out), rows, k, n, None)
    assert status != 0
    assert b"more than the" in library.carat_b200_last_error()
