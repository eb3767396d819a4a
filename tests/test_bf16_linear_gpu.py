"""The BF16 weight-streaming linear (carat_b200_bf16_linear: the FP8 linear's kernel with 16-bit
operands) against a plain PyTorch fp32 reference of the same product and against the reference's
own Bf16Linear (cuBLAS, cuda/linear.cu:534-643) where oracle/_ref/libref_cuda.so is built.
Bar: one bf16 ulp (fp32 accumulation order differs between implementations)."""
import ctypes

import pytest
import torch

import carat_b200
import reference_cuda as ref
from carat_b200.capi import check
from helpers import one_ulp_apart

pytestmark = pytest.mark.gpu


def ptr(tensor):
    return ctypes.c_void_p(tensor.data_ptr()) if tensor is not None else None


def operands(rows, k, n, seed):
    generator = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, k, device="cuda", generator=generator).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda", generator=generator) * 0.02).to(torch.bfloat16)
    return x, w


def run(x, w):
    library = carat_b200.library()
    rows, k = x.shape
    n = w.shape[0]
    out = torch.full((rows, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    need = library.carat_b200_bf16_linear_workspace_bytes(rows, k, n)
    work = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    check(library.carat_b200_bf16_linear(ptr(x), ptr(w), ptr(out), rows, k, n, ptr(work), need,
                                         None))
    torch.cuda.synchronize()
    return out


# rows x K -> N: drafter shapes (split-K and not), ragged K / N, prefill-chunk rows, 256 rows
SHAPES = [(24, 1024, 8192), (24, 8192, 1024), (24, 10752, 1024), (24, 1024, 16384),
          (5, 1024, 5376), (120, 5376, 16384), (192, 5376, 18432), (256, 21504, 5376),
          (7, 1000, 520), (33, 264, 1032)]


@pytest.mark.parametrize("rows,k,n", SHAPES)
def test_bf16_linear_matches_fp32_reference(cuda_device, rows, k, n):
    x, w = operands(rows, k, n, rows + k + n)
    got = run(x, w)
    want = (x.float() @ w.float().t()).to(torch.bfloat16)
    assert one_ulp_apart(got, want)
    assert float((got.view(torch.int16) != want.view(torch.int16)).float().mean()) < 0.05


@pytest.mark.parametrize("rows,k,n", [(24, 1024, 8192), (24, 16384, 1024), (120, 5376, 43008)])
def test_bf16_linear_matches_the_reference_cublas_linear(cuda_device, rows, k, n):
    theirs = ref.library()
    x, w = operands(rows, k, n, 3)
    got = run(x, w)
    want = torch.empty(rows, n, dtype=torch.bfloat16, device="cuda")
    ref.check(theirs.ref_bf16_linear_run(ptr(x), ptr(w), ptr(want), rows, k, n))
    torch.cuda.synchronize()
    assert one_ulp_apart(got, want)


def test_bf16_lm_head_argmax(cuda_device):
    """The drafter's default LM head: 24 rows x 1024 -> 262144, ties to the lowest index."""
    library = carat_b200.library()
    rows, k, n = 24, 1024, 262144
    x, w = operands(rows, k, n, 11)
    w[70000] = w[5]                       # an exact duplicate row: equal logits, lower index wins
    tokens = torch.empty(rows, dtype=torch.int32, device="cuda")
    keys = torch.empty(rows, dtype=torch.int64, device="cuda")
    check(library.carat_b200_bf16_linear_argmax(ptr(x), ptr(w), ptr(tokens), ptr(keys), rows, k, n,
                                                None))
    torch.cuda.synchronize()
    logits = (x.float() @ w.float().t()).to(torch.bfloat16).float()
    best = logits.max(dim=1).values
    chosen = logits.gather(1, tokens.long()[:, None])[:, 0]
    # The chosen logit is the row maximum up to one bf16 ulp of accumulation-order difference.
    assert bool((best - chosen <= best.abs() * 2.0 ** -7).all())
    exact = (logits.argmax(dim=1).int() == tokens)
    assert int(exact.sum()) >= rows - 2
    assert not bool((tokens == 70000).any())


def test_rejects_what_it_cannot_take(cuda_device):
    library = carat_b200.library()
    x, w = operands(8, 64, 64, 1)
    out = torch.empty(8, 64, dtype=torch.bfloat16, device="cuda")
    assert library.carat_b200_bf16_linear(ptr(x), ptr(w), ptr(out), 257, 64, 64, None, 0, None) != 0
    assert library.carat_b200_bf16_linear(ptr(x), ptr(w), ptr(out), 8, 60, 64, None, 0, None) != 0
    assert b"invalid BF16 linear shape" in library.carat_b200_last_error()
