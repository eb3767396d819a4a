"""The new kernels beside the reference's own CUDA operators, on the same inputs, on the GPU.

The reference side is oracle/_ref/libref_cuda.so: cuda/ops.cu, linear.cu, qkv.cu,
prefill_gemm_attention.cu of the reference compiled unmodified for sm_100a (cuBLASLt carries its
FP8 linear). Bars: bytes and scale identical for quantisation and for pure copies; bf16 rows
identical or one ulp apart on rare elements where the two sides sum fp32 squares in a different
order; linears within one bf16 ulp of the cuBLASLt result; attention within bf16 relative 2e-2
(the reference's own bar against host math is 0.015, tests/cuda_ops_tests.cu:1630-1779).
"""
import ctypes

import pytest
import torch

import carat_b200
import reference_cuda as ref
from carat_b200.capi import check
from helpers import one_ulp_apart, relative_error

pytestmark = pytest.mark.gpu

_alive = []


@pytest.fixture(autouse=True)
def _release_device_tensors():
    yield
    _alive.clear()
    torch.cuda.synchronize()


def keep(tensor):
    _alive.append(tensor)
    return tensor


def randn(shape, seed, scale=1.0, dtype=torch.bfloat16):
    generator = torch.Generator(device="cuda").manual_seed(seed)
    return keep((torch.randn(shape, device="cuda", generator=generator) * scale).to(dtype))


def empty(shape, dtype=torch.bfloat16):
    return keep(torch.empty(shape, dtype=dtype, device="cuda"))


def zeros(shape, dtype=torch.float32):
    return keep(torch.zeros(shape, dtype=dtype, device="cuda"))


def ptr(tensor):
    return ctypes.c_void_p(tensor.data_ptr()) if tensor is not None else None


def pointer_table(tensors):
    """Device array of device pointers (the reference's per-request cache pointer tables)."""
    return keep(torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device="cuda"))


def flips(got, want):
    return float((got.view(torch.int16) != want.view(torch.int16)).float().mean())


def ulp_close(got, want):
    """bf16 rows equal except for rare last-bit flips (different fp32 summation order)."""
    assert flips(got, want) < 2e-3
    assert one_ulp_apart(got, want)


# ---------------------------------------------------------------- quantisers (a12)
@pytest.mark.parametrize("rows,width", [(5, 256), (120, 5376), (120, 21504), (128, 8192)])
def test_plain_quantise_bytes_and_scale_equal_the_reference(cuda_device, rows, width):
    ours, theirs = carat_b200.library(), ref.library()
    x = randn((rows, width), rows + width, 3.0)
    out_a, out_b = empty((rows, width), torch.uint8), empty((rows, width), torch.uint8)
    scale_a, scale_b = zeros(1), zeros(1)
    scratch = zeros(1, torch.int32)
    check(ours.carat_b200_quantize_bf16_to_fp8(ptr(x), ptr(out_a), ptr(scale_a), ptr(scratch), rows,
                                               width, None))
    ref.check(theirs.ref_quantize_bf16_to_fp8_e4m3(ptr(x), ptr(out_b), ptr(scale_b), rows * width))
    torch.cuda.synchronize()
    assert torch.equal(scale_a, scale_b)
    assert torch.equal(out_a, out_b)


def test_large_tensor_quantiser_equals_the_reference(cuda_device):
    ours, theirs = carat_b200.library(), ref.library()
    rows, width = 4096, 5376     # the reference's non-cooperative branch (weights at load time)
    x = randn((rows, width), 9, 0.02)
    out_a, out_b = empty((rows, width), torch.uint8), empty((rows, width), torch.uint8)
    scale_a, scale_b = zeros(1), zeros(1)
    scratch = zeros(1, torch.int32)
    check(ours.carat_b200_quantize_bf16_tensor_to_fp8(ptr(x), ptr(out_a), ptr(scale_a),
                                                      ptr(scratch), rows * width, None))
    ref.check(theirs.ref_quantize_bf16_to_fp8_e4m3(ptr(x), ptr(out_b), ptr(scale_b), rows * width))
    torch.cuda.synchronize()
    assert torch.equal(scale_a, scale_b)
    assert torch.equal(out_a, out_b)


# ---------------------------------------------------------------- fused row operators (a7, a11)
@pytest.mark.parametrize("rows,width", [(5, 1024), (120, 5376), (128, 5376)])
def test_rms_norm_quantise_against_the_reference_pair(cuda_device, rows, width):
    ours, theirs = carat_b200.library(), ref.library()
    x = randn((rows, width), 1 + rows, 1.0)
    w = keep((1.0 + 0.1 * randn((width,), 2, 1.0).float()).to(torch.bfloat16))
    norm_a, norm_b = empty((rows, width)), empty((rows, width))
    out_a, out_b = empty((rows, width), torch.uint8), empty((rows, width), torch.uint8)
    scale_a, scale_b = zeros(1), zeros(1)
    row_amax = zeros(rows)
    scratch = zeros(1, torch.int32)
    check(ours.carat_b200_rms_norm_quantize(ptr(x), ptr(w), ptr(norm_a), ptr(out_a), ptr(scale_a),
                                            ptr(scratch), rows, width, 1e-6, None))
    ref.check(theirs.ref_rms_norm_bf16_with_row_amax(ptr(x), ptr(w), ptr(norm_b), ptr(row_amax),
                                                     rows, width, 1e-6))
    ref.check(theirs.ref_quantize_bf16_to_fp8_e4m3_from_row_amax(ptr(norm_b), ptr(out_b),
                                                                 ptr(scale_b), ptr(row_amax), rows,
                                                                 width))
    torch.cuda.synchronize()
    ulp_close(norm_a, norm_b)
    # The reference's quantiser applied to this side's rows gives this side's bytes and scale.
    out_c, scale_c = empty((rows, width), torch.uint8), zeros(1)
    ref.check(theirs.ref_quantize_bf16_to_fp8_e4m3(ptr(norm_a), ptr(out_c), ptr(scale_c),
                                                   rows * width))
    torch.cuda.synchronize()
    assert torch.equal(scale_a, scale_c)
    assert torch.equal(out_a, out_c)
    if torch.equal(norm_a, norm_b):
        assert torch.equal(out_a, out_b) and torch.equal(scale_a, scale_b)


@pytest.mark.parametrize("rows", [24, 120])
def test_post_attention_norms_against_the_reference(cuda_device, rows):
    ours, theirs = carat_b200.library(), ref.library()
    width = 5376
    x = randn((rows, width), 3, 0.3)
    residual = randn((rows, width), 4, 1.0)
    w1 = keep((1.0 + 0.1 * randn((width,), 5).float()).to(torch.bfloat16))
    w2 = keep((1.0 + 0.1 * randn((width,), 6).float()).to(torch.bfloat16))
    first_a, first_b, second_b = empty((rows, width)), empty((rows, width)), empty((rows, width))
    out_a, out_b = empty((rows, width), torch.uint8), empty((rows, width), torch.uint8)
    scale_a, scale_b, row_amax = zeros(1), zeros(1), zeros(rows)
    scratch = zeros(1, torch.int32)
    check(ours.carat_b200_rms_norm_add_and_norm_quantize(
        ptr(x), ptr(w1), ptr(residual), ptr(w2), ptr(first_a), ptr(out_a), ptr(scale_a),
        ptr(scratch), rows, width, 1e-6, None))
    ref.check(theirs.ref_rms_norm_add_and_norm_bf16_with_row_amax(
        ptr(x), ptr(w1), ptr(residual), ptr(w2), ptr(first_b), ptr(second_b), ptr(row_amax), rows,
        width, 1e-6))
    ref.check(theirs.ref_quantize_bf16_to_fp8_e4m3_from_row_amax(ptr(second_b), ptr(out_b),
                                                                 ptr(scale_b), ptr(row_amax), rows,
                                                                 width))
    torch.cuda.synchronize()
    ulp_close(first_a, first_b)
    # e4m3 bytes: equal wherever the bf16 rows were equal and the scales agree.
    if torch.equal(scale_a, scale_b):
        assert float((out_a != out_b).float().mean()) < 5e-3
    values_a = out_a.view(torch.float8_e4m3fn).float() * scale_a
    values_b = out_b.view(torch.float8_e4m3fn).float() * scale_b
    assert relative_error(values_a, values_b) < 0.07     # one e4m3 step


@pytest.mark.parametrize("rows,width", [(16, 8192), (120, 21504)])
def test_geglu_quantise_against_the_reference_chain(cuda_device, rows, width):
    ours, theirs = carat_b200.library(), ref.library()
    packed = randn((rows, 2 * width), 7, 1.5)
    out_a, out_b = empty((rows, width), torch.uint8), empty((rows, width), torch.uint8)
    scale_a, scale_b = zeros(1), zeros(1)
    scratch = zeros(1, torch.int32)
    activated = empty((rows, width))
    blocks = (width + 255) // 256
    block_amax, row_amax = zeros(rows * blocks), zeros(rows)
    check(ours.carat_b200_gelu_gate_quantize(ptr(packed), ptr(out_a), ptr(scale_a), ptr(scratch),
                                             rows, width, None))
    # cuda/layer_runner.cu:331-347: GeGLU with block maxima -> row maxima -> quantiser.
    ref.check(theirs.ref_gelu_tanh_gate_rows_bf16_with_block_amax(ptr(packed), ptr(activated),
                                                                  ptr(block_amax), rows, width))
    ref.check(theirs.ref_reduce_block_amax_to_rows(ptr(block_amax), ptr(row_amax), rows, blocks))
    ref.check(theirs.ref_quantize_bf16_to_fp8_e4m3_from_row_amax(ptr(activated), ptr(out_b),
                                                                 ptr(scale_b), ptr(row_amax), rows,
                                                                 width))
    torch.cuda.synchronize()
    assert torch.equal(scale_a, scale_b)
    assert torch.equal(out_a, out_b)      # element-wise math: no reduction order to differ in


def test_layer_output_against_the_reference(cuda_device):
    ours, theirs = carat_b200.library(), ref.library()
    rows, width = 120, 5376
    x = randn((rows, width), 11, 0.4)
    residual = randn((rows, width), 12, 1.0)
    w = keep((1.0 + 0.1 * randn((width,), 13).float()).to(torch.bfloat16))
    w_next = keep((1.0 + 0.1 * randn((width,), 14).float()).to(torch.bfloat16))
    scalar = keep(torch.tensor([0.75], dtype=torch.bfloat16, device="cuda"))
    out_a, out_b = empty((rows, width)), empty((rows, width))
    next_a, next_b = empty((rows, width)), empty((rows, width))
    fp8_a, scale_a, scratch = empty((rows, width), torch.uint8), zeros(1), zeros(1, torch.int32)
    check(ours.carat_b200_rms_norm_add_scale_then_norm_quantize(
        ptr(x), ptr(w), ptr(residual), ptr(scalar), ptr(out_a), ptr(w_next), ptr(next_a),
        ptr(fp8_a), ptr(scale_a), ptr(scratch), rows, width, 1e-6, None))
    ref.check(theirs.ref_rms_norm_add_scale_bf16(ptr(x), ptr(w), ptr(residual), ptr(scalar),
                                                 ptr(out_b), rows, width, 1e-6))
    ref.check(theirs.ref_rms_norm_bf16(ptr(out_b), ptr(w_next), ptr(next_b), rows, width, 1e-6))
    torch.cuda.synchronize()
    ulp_close(out_a, out_b)
    assert flips(next_a, next_b) < 5e-3 and one_ulp_apart(next_a, next_b)


# ---------------------------------------------------------------- FP8 linear (a12)
SHAPES_31B = [(5376, 16384), (8192, 5376), (5376, 18432), (16384, 5376), (5376, 43008),
              (21504, 5376), (5376, 262144)]


@pytest.mark.parametrize("k,n", SHAPES_31B)
def test_fp8_linear_against_cublaslt_at_120_rows(cuda_device, k, n):
    ours, theirs = carat_b200.library(), ref.library()
    rows = 120
    generator = torch.Generator(device="cuda").manual_seed(k + n)
    x = keep((torch.randn(rows, k, device="cuda", generator=generator) * 100).clamp(-440, 440)
             .to(torch.float8_e4m3fn).view(torch.uint8))
    w = keep((torch.randn(n, k, device="cuda", generator=generator) * 100).clamp(-440, 440)
             .to(torch.float8_e4m3fn).view(torch.uint8))
    x_scale = keep(torch.tensor([0.01], dtype=torch.float32, device="cuda"))
    w_scale = keep(torch.tensor([0.0002], dtype=torch.float32, device="cuda"))
    out_a, out_b = empty((rows, n)), empty((rows, n))
    need = ours.carat_b200_fp8_linear_workspace_bytes(rows, k, n)
    work = empty((max(need, 16),), torch.uint8)
    check(ours.carat_b200_fp8_linear(ptr(x), ptr(x_scale), ptr(w), ptr(w_scale), ptr(out_a), rows,
                                     k, n, ptr(work), need, None))
    ref.check(theirs.ref_fp8_linear_run(ptr(x), ptr(x_scale), ptr(w), ptr(w_scale), ptr(out_b),
                                        rows, k, n))
    torch.cuda.synchronize()
    assert one_ulp_apart(out_a, out_b)
    assert flips(out_a, out_b) < 0.05


def test_fused_lm_head_argmax_against_the_reference_chain(cuda_device):
    """quantise -> cuBLASLt FP8 GEMM -> argmax_bf16_rows (cuda/batch_model_runner.cu:840-853,
    938-940) against the fused LM head: same token wherever the reference's own top-2 margin
    exceeds one bf16 ulp of the winning logit."""
    ours, theirs = carat_b200.library(), ref.library()
    rows, k, n = 120, 5376, 262144
    hidden = randn((rows, k), 21, 1.0)
    generator = torch.Generator(device="cuda").manual_seed(22)
    w = keep((torch.randn(n, k, device="cuda", generator=generator) * 100).clamp(-440, 440)
             .to(torch.float8_e4m3fn).view(torch.uint8))
    w_scale = keep(torch.tensor([0.0002], dtype=torch.float32, device="cuda"))
    fp8, scale, scratch = empty((rows, k), torch.uint8), zeros(1), zeros(1, torch.int32)
    check(ours.carat_b200_quantize_bf16_to_fp8(ptr(hidden), ptr(fp8), ptr(scale), ptr(scratch),
                                               rows, k, None))
    tokens_a = empty((rows,), torch.int32)
    keys = empty((rows,), torch.int64)
    check(ours.carat_b200_fp8_linear_argmax(ptr(fp8), ptr(scale), ptr(w), ptr(w_scale),
                                            ptr(tokens_a), ptr(keys), rows, k, n, None))
    logits = empty((rows, n))
    tokens_b = empty((rows,), torch.int32)
    fp8_b, scale_b = empty((rows, k), torch.uint8), zeros(1)
    workspace = empty((theirs.ref_argmax_bf16_workspace_bytes(n) * rows,), torch.uint8)
    ref.check(theirs.ref_quantize_argmax_launch(ptr(hidden), ptr(fp8_b), ptr(scale_b), ptr(w),
                                                ptr(w_scale), ptr(logits), ptr(tokens_b),
                                                ptr(workspace), rows, k, n))
    torch.cuda.synchronize()
    assert torch.equal(fp8, fp8_b) and torch.equal(scale, scale_b)
    top2 = logits.float().topk(2, dim=1).values
    margin = top2[:, 0] - top2[:, 1]
    ulp = top2[:, 0].abs() * 2.0 ** -7
    differing = (tokens_a != tokens_b)
    assert bool((margin[differing] <= ulp[differing]).all())
    assert int(differing.sum()) <= 4


# ---------------------------------------------------------------- argmax and rollback (a13, a5)
def test_row_argmax_equals_the_reference_including_ties(cuda_device):
    ours, theirs = carat_b200.library(), ref.library()
    rows, elements = 24, 262144
    values = randn((rows, elements), 31, 4.0)
    values[3, 100] = values[3, 200000] = 99.0        # tie: lowest index wins
    values[7, :] = 0.0                               # all equal
    values[9, elements - 1] = 120.0                  # maximum in the last column
    out_a, out_b = empty((rows,), torch.int32), empty((rows,), torch.int32)
    workspace = empty((theirs.ref_argmax_bf16_workspace_bytes(elements) * rows,), torch.uint8)
    check(ours.carat_b200_argmax_bf16_rows(ptr(values), rows, elements, ptr(out_a), None))
    ref.check(theirs.ref_argmax_bf16_rows(ptr(values), rows, elements, ptr(out_b), ptr(workspace)))
    torch.cuda.synchronize()
    assert torch.equal(out_a, out_b)
    assert out_a[3].item() == 100 and out_a[7].item() == 0 and out_a[9].item() == elements - 1


@pytest.mark.parametrize("depth", [1, 5, 8])
def test_backup_and_restore_bytes_equal_the_reference(cuda_device, depth):
    ours, theirs = carat_b200.library(), ref.library()
    requests, heads, dim, capacity = 6, 16, 256, 1024
    positions = [3, 1020, 1023, 1024, 5000, 8000][:requests]      # spans that wrap and that do not
    accepted = [0, 1, depth, depth // 2, 1, depth][:requests]
    caches_k = [randn((heads, capacity, dim), 40 + r) for r in range(requests)]
    caches_v = [randn((heads, capacity, dim), 60 + r) for r in range(requests)]
    key_table, value_table = pointer_table(caches_k), pointer_table(caches_v)
    device_positions = keep(torch.tensor(positions, dtype=torch.int32, device="cuda"))
    device_accepted = keep(torch.tensor(accepted, dtype=torch.int32, device="cuda"))
    backups = [[empty((requests, heads, depth, dim)) for _ in range(2)] for _ in range(2)]
    check(ours.carat_b200_backup_kv_ring_spans(ptr(key_table), ptr(value_table),
                                               ptr(backups[0][0]), ptr(backups[0][1]),
                                               ptr(device_positions), requests, heads, depth, dim,
                                               capacity, None))
    ref.check(theirs.ref_backup_kv_ring_spans_bf16(ptr(key_table), ptr(value_table),
                                                   ptr(backups[1][0]), ptr(backups[1][1]),
                                                   ptr(device_positions), requests, heads, depth,
                                                   dim, capacity))
    torch.cuda.synchronize()
    assert torch.equal(backups[0][0], backups[1][0]) and torch.equal(backups[0][1], backups[1][1])
    # Overwrite the spans, then restore the rejected suffixes on two copies of the caches.
    originals = [cache.clone() for cache in caches_k + caches_v]
    for cache, position in zip(caches_k + caches_v, positions + positions):
        for token in range(depth):
            cache[:, (position + token) % capacity, :] = 7.0
    copies_k = [keep(cache.clone()) for cache in caches_k]
    copies_v = [keep(cache.clone()) for cache in caches_v]
    copy_key_table, copy_value_table = pointer_table(copies_k), pointer_table(copies_v)
    check(ours.carat_b200_restore_kv_ring_suffixes(ptr(backups[0][0]), ptr(backups[0][1]),
                                                   ptr(key_table), ptr(value_table),
                                                   ptr(device_positions), ptr(device_accepted),
                                                   requests, heads, depth, dim, capacity, None))
    ref.check(theirs.ref_restore_kv_ring_suffixes_bf16(ptr(backups[1][0]), ptr(backups[1][1]),
                                                       ptr(copy_key_table), ptr(copy_value_table),
                                                       ptr(device_positions), ptr(device_accepted),
                                                       requests, heads, depth, dim, capacity))
    torch.cuda.synchronize()
    for mine, theirs_copy in zip(caches_k + caches_v, copies_k + copies_v):
        assert torch.equal(mine, theirs_copy)
    for request, (cache, original) in enumerate(zip(caches_k, originals[:requests])):
        for token in range(depth):
            row = (positions[request] + token) % capacity
            expected = original[:, row, :] if token >= accepted[request] else \
                torch.full_like(original[:, row, :], 7.0)
            assert torch.equal(cache[:, row, :], expected)


# ---------------------------------------------------------------- QKV post-processing (a8)
@pytest.mark.parametrize("kind", ["sliding", "global"])
def test_qkv_postprocess_against_the_reference(cuda_device, kind):
    ours, theirs = carat_b200.library(), ref.library()
    requests, depth, table_positions = 4, 5, 8192
    if kind == "sliding":
        heads, kv_heads, dim, theta, proportional, kev = 32, 16, 256, 1e4, 0, 0
    else:
        heads, kv_heads, dim, theta, proportional, kev = 32, 4, 512, 1e6, 1, 1
    packed_width = heads * dim + kv_heads * dim * (1 if kev else 2)
    packed = randn((requests * depth, packed_width), 70, 1.0)
    q_norm = keep((1.0 + 0.1 * randn((dim,), 71).float()).to(torch.bfloat16))
    k_norm = keep((1.0 + 0.1 * randn((dim,), 72).float()).to(torch.bfloat16))
    positions = keep(torch.tensor([0, 17, 1500, 8192 - depth], dtype=torch.int32, device="cuda"))
    cosine, sine = empty((table_positions, dim)), empty((table_positions, dim))
    check(ours.carat_b200_rope_tables(ptr(cosine), ptr(sine), table_positions, dim, theta,
                                      proportional, None))
    q_a, k_a, v_a = (empty((requests, heads, depth, dim)), empty((requests, kv_heads, depth, dim)),
                     empty((requests, kv_heads, depth, dim)))
    check(ours.carat_b200_qkv_postprocess(ptr(packed), ptr(q_norm), ptr(k_norm), ptr(cosine),
                                          ptr(sine), ptr(q_a), ptr(k_a), ptr(v_a), ptr(positions),
                                          requests, depth, heads, kv_heads, dim, kev,
                                          table_positions, 1e-6, None))
    # Reference: token-major queries [requests * depth, heads, dim]; K/V staged
    # [requests, kv_heads, staged_capacity, dim] from row staged_position_start on.
    q_b = empty((requests * depth, heads, dim))
    k_b, v_b = zeros((requests, kv_heads, depth, dim), torch.bfloat16), \
        zeros((requests, kv_heads, depth, dim), torch.bfloat16)
    ref.check(theirs.ref_qkv_run_prefill_uniform(table_positions, ptr(packed), ptr(q_norm),
                                                 ptr(k_norm), ptr(q_b), ptr(k_b), ptr(v_b),
                                                 ptr(positions), requests, depth, heads, kv_heads,
                                                 dim, kev, 0, depth, 1e-6))
    torch.cuda.synchronize()
    q_b_head_major = q_b.view(requests, depth, heads, dim).permute(0, 2, 1, 3).contiguous()
    ulp_close(q_a, q_b_head_major)
    ulp_close(k_a, k_b)
    ulp_close(v_a, v_b)


# ---------------------------------------------------------------- verify attention (a9)
@pytest.mark.parametrize("depth", [5, 8])
def test_ring_attention_against_the_reference(cuda_device, depth):
    """Wrapped sliding ring: the reference writes the proposals into the ring and repairs the
    scores / outputs of later proposal slots from the backup (cuda/prefill_gemm_attention.cu:
    657-730); this side leaves the ring alone and reads the proposals from staging."""
    ours, theirs = carat_b200.library(), ref.library()
    requests, heads, kv_heads, dim, capacity = 3, 32, 16, 256, 1024
    positions = [1024, 3000, 8100]
    queries = randn((requests, heads, depth, dim), 80, 0.08)
    ring_k = randn((requests, kv_heads, capacity, dim), 81, 1.0)
    ring_v = randn((requests, kv_heads, capacity, dim), 82, 1.0)
    new_k = randn((requests, kv_heads, depth, dim), 83, 1.0)
    new_v = randn((requests, kv_heads, depth, dim), 84, 1.0)
    device_positions = keep(torch.tensor(positions, dtype=torch.int32, device="cuda"))
    stride = 16 + capacity
    scores = empty((requests * heads * depth * stride,))
    out_a = empty((requests * depth, heads * dim))
    check(ours.carat_b200_verify_attention(ptr(queries), ptr(ring_k), ptr(ring_v), ptr(new_k),
                                           ptr(new_v), ptr(device_positions), ptr(out_a),
                                           ptr(scores), stride, requests, depth, heads, kv_heads,
                                           dim, capacity, capacity, max(positions), None))
    written_k, written_v = keep(ring_k.clone()), keep(ring_v.clone())
    backup_k, backup_v = empty((requests, kv_heads, depth, dim)), empty((requests, kv_heads, depth, dim))
    for request, position in enumerate(positions):
        for token in range(depth):
            row = (position + token) % capacity
            backup_k[request, :, token] = ring_k[request, :, row]
            backup_v[request, :, token] = ring_v[request, :, row]
            written_k[request, :, row] = new_k[request, :, token]
            written_v[request, :, row] = new_v[request, :, token]
    key_table = pointer_table([written_k[r] for r in range(requests)])
    value_table = pointer_table([written_v[r] for r in range(requests)])
    out_b = empty((requests, heads, depth, dim))
    ref.check(theirs.ref_attention_run_uniform_ring_batch(
        2048, 32, 24, ptr(queries), ptr(key_table), ptr(value_table), ptr(backup_k), ptr(backup_v),
        ptr(out_b), ptr(device_positions), requests, heads, kv_heads, depth, capacity, dim))
    torch.cuda.synchronize()
    token_major = out_b.permute(0, 2, 1, 3).reshape(requests * depth, heads * dim)
    assert relative_error(out_a, token_major) < 2e-2


def test_global_attention_against_the_reference(cuda_device):
    ours, theirs = carat_b200.library(), ref.library()
    requests, depth, heads, kv_heads, dim, capacity = 3, 5, 32, 4, 512, 4096
    positions = [1, 700, 2100]
    queries = randn((requests, heads, depth, dim), 90, 0.06)
    cache_k = randn((requests, kv_heads, capacity, dim), 91, 1.0)
    cache_v = randn((requests, kv_heads, capacity, dim), 92, 1.0)
    device_positions = keep(torch.tensor(positions, dtype=torch.int32, device="cuda"))
    longest = max(positions) + depth
    stride = 16 + (longest + 127) // 128 * 128
    scores = empty((requests * heads * depth * stride,))
    out_a = empty((requests * depth, heads * dim))
    check(ours.carat_b200_verify_attention(ptr(queries), ptr(cache_k), ptr(cache_v), None, None,
                                           ptr(device_positions), ptr(out_a), ptr(scores), stride,
                                           requests, depth, heads, kv_heads, dim, capacity, 0,
                                           max(positions), None))
    key_table = pointer_table([cache_k[r] for r in range(requests)])
    value_table = pointer_table([cache_v[r] for r in range(requests)])
    out_b = empty((requests, heads, depth, dim))
    bucket = min(capacity, (longest + 63) // 64 * 64)      # cuda/layer_runner.cu:1004-1010
    ref.check(theirs.ref_attention_run_uniform_batch(
        4096, 32, 24, ptr(queries), ptr(key_table), ptr(value_table), ptr(out_b),
        ptr(device_positions), requests, heads, kv_heads, depth, bucket, capacity, dim))
    torch.cuda.synchronize()
    token_major = out_b.permute(0, 2, 1, 3).reshape(requests * depth, heads * dim)
    assert relative_error(out_a, token_major) < 2e-2
