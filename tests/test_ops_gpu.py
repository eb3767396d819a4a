"""Each device operator against the CPU oracle, called through the C ABI."""
import ctypes

import pytest
import torch

import carat_b200
from carat_b200.capi import check
from helpers import relative_error
from oracle import carat_semantics as cs

pytestmark = pytest.mark.gpu


_alive = []


@pytest.fixture(autouse=True)
def _release_device_tensors():
    yield
    _alive.clear()


def dev(tensor, dtype=torch.bfloat16):
    """Uploads and keeps the device tensor alive until the test ends (the C ABI only sees raw
    pointers, so a temporary would be recycled by the allocator before the kernel runs)."""
    moved = tensor.to(device="cuda", dtype=dtype).contiguous()
    _alive.append(moved)
    return moved


def dev_int(values):
    return dev(torch.tensor(values, dtype=torch.int32), torch.int32)


def ptr(tensor):
    return ctypes.c_void_p(tensor.data_ptr()) if tensor is not None else None


def fp8_values(raw):
    return raw.view(torch.float8_e4m3fn).float().cpu()


def quant_buffers(rows, width):
    return (torch.empty(rows, width, dtype=torch.uint8, device="cuda"),
            torch.zeros(1, dtype=torch.float32, device="cuda"),
            torch.zeros(1, dtype=torch.int32, device="cuda"))


def assert_quantised(raw, scale, expected_bf16):
    """The e4m3 bytes and scale must be exactly what the oracle derives from the same bf16 rows."""
    want, want_scale = cs.quantize_e4m3(expected_bf16)
    assert torch.equal(scale.cpu(), want_scale.reshape(1))
    assert torch.equal(fp8_values(raw), want)


@pytest.mark.parametrize("rows,width", [(1, 256), (5, 5376), (120, 5376), (24, 21504), (128, 1024)])
def test_plain_quantise_is_bit_exact(cuda_device, rows, width):
    lib = carat_b200.library()
    generator = torch.Generator().manual_seed(rows * 7 + width)
    x = cs.bf16(torch.randn(rows, width, generator=generator) * 3.0)
    out, scale, scratch = quant_buffers(rows, width)
    check(lib.carat_b200_quantize_bf16_to_fp8(ptr(dev(x)), ptr(out), ptr(scale), ptr(scratch), rows,
                                              width, None))
    torch.cuda.synchronize()
    assert_quantised(out, scale, x)


def test_zero_tensor_gets_unit_scale(cuda_device):
    lib = carat_b200.library()
    x = torch.zeros(3, 64)
    out, scale, scratch = quant_buffers(3, 64)
    check(lib.carat_b200_quantize_bf16_to_fp8(ptr(dev(x)), ptr(out), ptr(scale), ptr(scratch), 3, 64,
                                              None))
    torch.cuda.synchronize()
    assert float(scale.cpu()) == 1.0
    assert int(out.cpu().sum()) == 0


@pytest.mark.parametrize("rows,width", [(5, 256), (120, 5376), (24, 1024)])
def test_rms_norm_quantise(cuda_device, rows, width):
    lib = carat_b200.library()
    generator = torch.Generator().manual_seed(width + rows)
    x = cs.bf16(torch.randn(rows, width, generator=generator))
    w = cs.bf16(1.0 + 0.1 * torch.randn(width, generator=generator))
    want = cs.rms_norm(x, w, 1e-6)
    out, scale, scratch = quant_buffers(rows, width)
    normalized = torch.empty(rows, width, dtype=torch.bfloat16, device="cuda")
    check(lib.carat_b200_rms_norm_quantize(ptr(dev(x)), ptr(dev(w)), ptr(normalized), ptr(out),
                                           ptr(scale), ptr(scratch), rows, width, 1e-6, None))
    torch.cuda.synchronize()
    got = normalized.float().cpu()
    # fp32 summation order differs; a bf16 rounding may flip on rare elements.
    assert (got != want).float().mean() < 2e-3
    assert relative_error(got, want) < 1e-2
    assert_quantised(out, scale, got)   # quantisation of the device's own rows is exact


def test_post_attention_norms_and_layer_output(cuda_device):
    lib = carat_b200.library()
    rows, width = 40, 5376
    generator = torch.Generator().manual_seed(3)
    x = cs.bf16(torch.randn(rows, width, generator=generator) * 0.3)
    residual = cs.bf16(torch.randn(rows, width, generator=generator))
    w1 = cs.bf16(1.0 + 0.1 * torch.randn(width, generator=generator))
    w2 = cs.bf16(1.0 + 0.1 * torch.randn(width, generator=generator))
    first_want, second_want = cs.rms_norm_add_and_norm(x, w1, residual, w2, 1e-6)
    out, scale, scratch = quant_buffers(rows, width)
    first = torch.empty(rows, width, dtype=torch.bfloat16, device="cuda")
    check(lib.carat_b200_rms_norm_add_and_norm_quantize(
        ptr(dev(x)), ptr(dev(w1)), ptr(dev(residual)), ptr(dev(w2)), ptr(first), ptr(out),
        ptr(scale), ptr(scratch), rows, width, 1e-6, None))
    torch.cuda.synchronize()
    assert (first.float().cpu() != first_want).float().mean() < 2e-3
    assert relative_error(first, first_want) < 1e-2
    second_from_device = cs.rms_norm(first.float().cpu(), w2, 1e-6)
    got = fp8_values(out) * scale.cpu()
    assert relative_error(got, second_from_device) < 0.07   # e4m3 step
    assert relative_error(got, second_want) < 0.07

    scalar = cs.bf16(torch.tensor([0.7]))
    want_output = cs.rms_norm_add_scale(x, w1, residual, scalar, 1e-6)
    want_next = cs.rms_norm(want_output, w2, 1e-6)
    output = torch.empty(rows, width, dtype=torch.bfloat16, device="cuda")
    nxt = torch.empty(rows, width, dtype=torch.bfloat16, device="cuda")
    check(lib.carat_b200_rms_norm_add_scale_then_norm_quantize(
        ptr(dev(x)), ptr(dev(w1)), ptr(dev(residual)), ptr(dev(scalar)), ptr(output), ptr(dev(w2)),
        ptr(nxt), ptr(out), ptr(scale), ptr(scratch), rows, width, 1e-6, None))
    torch.cuda.synchronize()
    assert (output.float().cpu() != want_output).float().mean() < 2e-3
    assert relative_error(output, want_output) < 1e-2
    assert relative_error(nxt, want_next) < 1e-2
    assert_quantised(out, scale, nxt.float().cpu())


def test_gelu_gate_quantise(cuda_device):
    lib = carat_b200.library()
    rows, width = 24, 21504
    generator = torch.Generator().manual_seed(5)
    packed = cs.bf16(torch.randn(rows, 2 * width, generator=generator) * 2.0)
    want = cs.gelu_tanh_gate(packed, width)
    out, scale, scratch = quant_buffers(rows, width)
    check(lib.carat_b200_gelu_gate_quantize(ptr(dev(packed)), ptr(out), ptr(scale), ptr(scratch),
                                            rows, width, None))
    torch.cuda.synchronize()
    got = fp8_values(out) * scale.cpu()
    want_q, want_scale = cs.quantize_e4m3(want)
    # tanhf on the device and torch.tanh on the host may differ in the last bit before rounding.
    assert abs(float(scale.cpu()) - float(want_scale)) <= 0.01 * float(want_scale)
    assert relative_error(got, want_q * want_scale) < 0.07
    assert (fp8_values(out) != want_q).float().mean() < 5e-3


@pytest.mark.parametrize("head_dim,theta,proportional", [(64, 1e4, 0), (256, 1e4, 0), (512, 1e6, 1),
                                                         (64, 1e6, 1)])
def test_rope_tables(cuda_device, head_dim, theta, proportional):
    lib = carat_b200.library()
    positions = 512
    cos = torch.empty(positions, head_dim, dtype=torch.bfloat16, device="cuda")
    sin = torch.empty_like(cos)
    check(lib.carat_b200_rope_tables(ptr(cos), ptr(sin), positions, head_dim, theta, proportional,
                                     None))
    torch.cuda.synchronize()
    want_cos, want_sin = cs.rope_tables(positions, head_dim, theta, bool(proportional))
    # powf / sincosf differ from the host libm in the last bits; at most one bf16 step.
    assert (cos.float().cpu() - want_cos).abs().max() <= 2 ** -7
    assert (sin.float().cpu() - want_sin).abs().max() <= 2 ** -7
    assert (cos.float().cpu() != want_cos).float().mean() < 0.02


@pytest.mark.parametrize("head_dim,heads,kv_heads,k_eq_v", [(64, 4, 2, 0), (64, 4, 2, 1),
                                                           (256, 32, 16, 0), (512, 32, 4, 1)])
def test_qkv_postprocess(cuda_device, head_dim, heads, kv_heads, k_eq_v):
    lib = carat_b200.library()
    requests, depth, table = 3, 5, 512
    generator = torch.Generator().manual_seed(head_dim + heads)
    packed_width = heads * head_dim + kv_heads * head_dim * (1 if k_eq_v else 2)
    packed = cs.bf16(torch.randn(requests * depth, packed_width, generator=generator))
    q_norm = cs.bf16(0.35 + 0.05 * torch.randn(head_dim, generator=generator))
    k_norm = cs.bf16(0.35 + 0.05 * torch.randn(head_dim, generator=generator))
    cos, sin = cs.rope_tables(table, head_dim, 1e4 if not k_eq_v else 1e6, bool(k_eq_v))
    positions = [7, 130, 400]
    rows = torch.tensor([positions[r // depth] + r % depth for r in range(requests * depth)])
    q_raw = packed[:, :heads * head_dim].reshape(-1, heads, head_dim)
    k_raw = packed[:, heads * head_dim:(heads + kv_heads) * head_dim].reshape(-1, kv_heads, head_dim)
    v_raw = k_raw if k_eq_v else packed[:, (heads + kv_heads) * head_dim:].reshape(-1, kv_heads,
                                                                                 head_dim)
    want_q = cs.norm_rope(q_raw, q_norm, cos[rows], sin[rows], 1e-6)
    want_k = cs.norm_rope(k_raw, k_norm, cos[rows], sin[rows], 1e-6)
    want_v = cs.rms_norm(v_raw, None, 1e-6)
    queries = torch.empty(requests, heads, depth, head_dim, dtype=torch.bfloat16, device="cuda")
    keys = torch.empty(requests, kv_heads, depth, head_dim, dtype=torch.bfloat16, device="cuda")
    values = torch.empty_like(keys)
    check(lib.carat_b200_qkv_postprocess(
        ptr(dev(packed)), ptr(dev(q_norm)), ptr(dev(k_norm)), ptr(dev(cos)), ptr(dev(sin)),
        ptr(queries), ptr(keys), ptr(values),
        ptr(dev_int(positions)), requests, depth, heads,
        kv_heads, head_dim, k_eq_v, table, 1e-6, None))
    torch.cuda.synchronize()
    want_q = want_q.reshape(requests, depth, heads, head_dim).permute(0, 2, 1, 3)
    want_k = want_k.reshape(requests, depth, kv_heads, head_dim).permute(0, 2, 1, 3)
    want_v = want_v.reshape(requests, depth, kv_heads, head_dim).permute(0, 2, 1, 3)
    for got, want in ((queries, want_q), (keys, want_k), (values, want_v)):
        assert relative_error(got, want) < 1e-2
        assert (got.float().cpu() != want).float().mean() < 5e-3


def reference_ring_case(query_tokens):
    """The closed-form case of the reference's test_uniform_ring_attention
    (tests/cuda_ops_tests.cu:1630-1779): a full 16-row ring that already holds the proposals, the
    pre-write rows in a backup, expected values from plain float math."""
    requests, heads, kv_heads, capacity, dim = 2, 2, 1, 16, 16
    positions = [11, 13]

    def series(count, mul, mod, sub, div):
        index = torch.arange(count, dtype=torch.int64)
        return cs.bf16(((index * mul) % mod - sub).float() / div)

    query = series(requests * heads * query_tokens * dim, 7, 19, 9, 32.0).reshape(
        requests, heads, query_tokens, dim)
    keys = series(requests * kv_heads * capacity * dim, 5, 23, 11, 48.0).reshape(
        requests, kv_heads, capacity, dim)
    values = series(requests * kv_heads * capacity * dim, 11, 29, 14, 24.0).reshape(
        requests, kv_heads, capacity, dim)
    backup_keys = series(requests * kv_heads * query_tokens * dim, 13, 17, 8, 40.0).reshape(
        requests, kv_heads, query_tokens, dim)
    backup_values = series(requests * kv_heads * query_tokens * dim, 3, 31, 15, 20.0).reshape(
        requests, kv_heads, query_tokens, dim)
    expected = torch.zeros(requests, heads, query_tokens, dim)
    for r in range(requests):
        for h in range(heads):
            for t in range(query_tokens):
                k = keys[r, 0].clone()
                v = values[r, 0].clone()
                for u in range(t + 1, query_tokens):
                    k[(positions[r] + u) % capacity] = backup_keys[r, 0, u]
                    v[(positions[r] + u) % capacity] = backup_values[r, 0, u]
                scores = k @ query[r, h, t]
                weights = torch.softmax(scores, dim=0)
                expected[r, h, t] = weights @ v
    # The same state in this library's form: the ring before the proposals were written, the
    # proposals on the side, and a logical position one full turn later.
    old_keys = keys.clone()
    old_values = values.clone()
    new_keys = torch.zeros(requests, kv_heads, query_tokens, dim)
    new_values = torch.zeros_like(new_keys)
    for r in range(requests):
        for u in range(query_tokens):
            row = (positions[r] + u) % capacity
            new_keys[r, 0, u] = keys[r, 0, row]
            new_values[r, 0, u] = values[r, 0, row]
            old_keys[r, 0, row] = backup_keys[r, 0, u]
            old_values[r, 0, row] = backup_values[r, 0, u]
    logical = [p + capacity for p in positions]
    return query, old_keys, old_values, new_keys, new_values, logical, expected, capacity


@pytest.mark.parametrize("query_tokens", [4, 8])
def test_ring_attention_reference_case(cuda_device, query_tokens):
    lib = carat_b200.library()
    query, old_k, old_v, new_k, new_v, logical, expected, capacity = reference_ring_case(query_tokens)
    # The kernels support head_dim 64/256/512; embed the 16-wide case in 64 columns of zeros.
    def pad(tensor):
        return torch.nn.functional.pad(tensor, (0, 48))
    requests, heads = 2, 2
    out = torch.empty(requests * query_tokens, heads * 64, dtype=torch.bfloat16, device="cuda")
    stride = 16 + 128
    scores = torch.empty(requests * heads * query_tokens * stride, dtype=torch.bfloat16, device="cuda")
    check(lib.carat_b200_verify_attention(
        ptr(dev(pad(query))), ptr(dev(pad(old_k))), ptr(dev(pad(old_v))), ptr(dev(pad(new_k))),
        ptr(dev(pad(new_v))), ptr(dev_int(logical)), ptr(out),
        ptr(scores), stride, requests, query_tokens, heads, 1, 64, capacity, capacity,
        max(logical), None))
    torch.cuda.synchronize()
    got = out.float().cpu().reshape(requests, query_tokens, heads, 64)[..., :16].permute(0, 2, 1, 3)
    assert (got - expected).abs().max() < 0.015   # the reference test's tolerance


@pytest.mark.parametrize("head_dim,heads,kv_heads,window,capacity,positions", [
    (64, 4, 2, 128, 128, [1, 60, 127, 128, 300]),
    (64, 4, 2, 0, 512, [1, 60, 200, 333, 500]),
    (256, 32, 16, 1024, 1024, [5, 1020, 1024, 3000]),
    (512, 32, 4, 0, 2048, [3, 700, 2040]),
    (512, 8, 1, 0, 4096, [1, 2500, 4000]),
    (256, 4, 2, 256, 256, [1, 128, 255, 256, 1000]),
])
def test_verify_attention_matches_oracle(cuda_device, head_dim, heads, kv_heads, window, capacity,
                                         positions):
    lib = carat_b200.library()
    depth = 5
    requests = len(positions)
    generator = torch.Generator().manual_seed(head_dim + window)
    scale = head_dim ** -0.25
    queries = cs.bf16(torch.randn(requests, depth, heads, head_dim, generator=generator) * scale)
    new_k = cs.bf16(torch.randn(requests, depth, kv_heads, head_dim, generator=generator) * scale)
    new_v = cs.bf16(torch.randn(requests, depth, kv_heads, head_dim, generator=generator))
    old_k = cs.bf16(torch.randn(requests, kv_heads, capacity, head_dim, generator=generator) * scale)
    old_v = cs.bf16(torch.randn(requests, kv_heads, capacity, head_dim, generator=generator))
    want = cs.verify_attention(queries, list(old_k), list(old_v), new_k, new_v, positions, window)
    d_queries = dev(queries.permute(0, 2, 1, 3))
    d_positions = dev_int(positions)
    outputs = []
    for entry in (lib.carat_b200_verify_attention, lib.carat_b200_verify_attention_check):
        if window > 0:
            rows = min(max(positions), capacity)
            d_old_k, d_old_v = dev(old_k), dev(old_v)
            d_new_k, d_new_v = dev(new_k.permute(0, 2, 1, 3)), dev(new_v.permute(0, 2, 1, 3))
        else:
            # Linear cache: the proposals are already in the cache at rows position + t.
            rows = max(positions) + depth
            filled_k, filled_v = old_k.clone(), old_v.clone()
            for r, position in enumerate(positions):
                filled_k[r, :, position:position + depth] = new_k[r].permute(1, 0, 2)
                filled_v[r, :, position:position + depth] = new_v[r].permute(1, 0, 2)
            d_old_k, d_old_v, d_new_k, d_new_v = dev(filled_k), dev(filled_v), None, None
        stride = 16 + (rows + 127) // 128 * 128
        out = torch.empty(requests * depth, heads * head_dim, dtype=torch.bfloat16, device="cuda")
        scores = torch.empty(requests * heads * depth * stride, dtype=torch.bfloat16, device="cuda")
        check(entry(ptr(d_queries), ptr(d_old_k), ptr(d_old_v), ptr(d_new_k), ptr(d_new_v),
                    ptr(d_positions), ptr(out), ptr(scores), stride, requests, depth, heads,
                    kv_heads, head_dim, capacity, window, max(positions), None))
        torch.cuda.synchronize()
        code = ctypes.c_int(0)
        check(lib.carat_b200_device_error(ctypes.byref(code)))
        assert code.value == 0
        outputs.append(out.float().cpu().reshape(requests, depth, heads, head_dim))
    for got in outputs:
        assert relative_error(got, want) < 2e-2
        assert (got != want).float().mean() < 0.02
    # The tensor-core kernels and the CUDA-core cross-check agree to rare last-bit differences.
    assert (outputs[0] != outputs[1]).float().mean() < 0.02


def test_backup_restore_is_bit_exact(cuda_device):
    lib = carat_b200.library()
    requests, heads, tokens, dim, capacity = 3, 2, 5, 64, 16
    generator = torch.Generator().manual_seed(11)
    keys = [dev(torch.randn(heads, capacity, dim, generator=generator)) for _ in range(requests)]
    values = [dev(torch.randn(heads, capacity, dim, generator=generator)) for _ in range(requests)]
    positions = [3, 14, 30]
    accepted = [0, 2, 5]
    host_k = [k.float().cpu().clone() for k in keys]
    host_v = [v.float().cpu().clone() for v in values]
    want_bk, want_bv = cs.backup_kv_ring_spans(host_k, host_v, positions, tokens)
    key_pointers = torch.tensor([k.data_ptr() for k in keys], dtype=torch.int64, device="cuda")
    value_pointers = torch.tensor([v.data_ptr() for v in values], dtype=torch.int64, device="cuda")
    backup_k = torch.empty(requests, heads, tokens, dim, dtype=torch.bfloat16, device="cuda")
    backup_v = torch.empty_like(backup_k)
    device_positions = torch.tensor(positions, dtype=torch.int32, device="cuda")
    check(lib.carat_b200_backup_kv_ring_spans(ptr(key_pointers), ptr(value_pointers), ptr(backup_k),
                                              ptr(backup_v), ptr(device_positions), requests, heads,
                                              tokens, dim, capacity, None))
    torch.cuda.synchronize()
    assert torch.equal(backup_k.float().cpu(), want_bk)
    assert torch.equal(backup_v.float().cpu(), want_bv)
    # Overwrite the spans, then restore the rejected suffixes.
    for r in range(requests):
        for t in range(tokens):
            row = (positions[r] + t) % capacity
            keys[r][:, row] = 7.0
            values[r][:, row] = -7.0
            host_k[r][:, row] = 7.0
            host_v[r][:, row] = -7.0
    cs.restore_kv_ring_suffixes(want_bk, want_bv, host_k, host_v, positions, accepted, tokens)
    check(lib.carat_b200_restore_kv_ring_suffixes(
        ptr(backup_k), ptr(backup_v), ptr(key_pointers), ptr(value_pointers), ptr(device_positions),
        ptr(dev_int(accepted)), requests, heads, tokens, dim,
        capacity, None))
    torch.cuda.synchronize()
    for r in range(requests):
        assert torch.equal(keys[r].float().cpu(), host_k[r])
        assert torch.equal(values[r].float().cpu(), host_v[r])


def test_argmax_reference_known_answers(cuda_device):
    """tests/cuda_ops_tests.cu:1137-1164: 3 rows of 513 values, equal maxima pick the lower index."""
    lib = carat_b200.library()
    rows, elements = 3, 513
    values = torch.full((rows, elements), -2.0)
    values[0, 17] = 9.0
    values[1, 0] = 4.0
    values[1, 401] = 4.0
    values[2, 512] = 7.0
    output = torch.zeros(rows, dtype=torch.int32, device="cuda")
    check(lib.carat_b200_argmax_bf16_rows(ptr(dev(values)), rows, elements, ptr(output), None))
    torch.cuda.synchronize()
    assert output.cpu().tolist() == [17, 0, 512]
    assert cs.argmax_lowest_index(values).tolist() == [17, 0, 512]


def test_greedy_prefix_accept_matches_oracle(cuda_device):
    lib = carat_b200.library()
    generator = torch.Generator().manual_seed(2)
    requests, depth = 24, 5
    predictions = torch.randint(0, 6, (requests, depth), generator=generator, dtype=torch.int32)
    proposals = predictions.roll(1, dims=1).clone()
    target_first = torch.randint(0, 6, (requests,), generator=generator, dtype=torch.int32)
    proposals[:, 0] = target_first
    noise = torch.rand(requests, depth, generator=generator) < 0.25
    proposals[noise] = 9
    caps = torch.randint(-1, 7, (requests,), generator=generator, dtype=torch.int32)
    want = cs.greedy_prefix_accept(proposals.tolist(), target_first.tolist(),
                                   predictions.reshape(-1).tolist(), caps.tolist(), depth)
    accepted = torch.zeros(requests, dtype=torch.int32, device="cuda")
    nxt = torch.zeros(requests, dtype=torch.int32, device="cuda")
    check(lib.carat_b200_greedy_prefix_accept(
        ptr(dev(proposals, torch.int32)), ptr(dev(target_first, torch.int32)),
        ptr(dev(predictions, torch.int32)), ptr(dev(caps, torch.int32)), requests, depth,
        ptr(accepted), ptr(nxt), None))
    torch.cuda.synchronize()
    assert accepted.cpu().tolist() == want[0]
    assert nxt.cpu().tolist() == want[1]


def test_a_wait_that_runs_out_reports_a_code_and_leaves_the_device_usable(cuda_device):
    """The bounded-wait path of the pipelined kernels, exercised without breaking any of them: a
    test-only kernel waits about a millisecond on a barrier nothing arrives on."""
    lib = carat_b200.library()
    code = ctypes.c_int(-1)
    check(lib.carat_b200_device_error(ctypes.byref(code)))          # start from a clean word
    report = torch.full((3,), -1, dtype=torch.int32, device="cuda")
    check(lib.carat_b200_selftest_bounded_wait(ptr(report), None))
    torch.cuda.synchronize()
    gave_up, second_returned_at_once, cycles = report.cpu().tolist()
    assert gave_up == 1 and second_returned_at_once == 1, (gave_up, second_returned_at_once, cycles)
    check(lib.carat_b200_device_error(ctypes.byref(code)))
    assert code.value == 90
    check(lib.carat_b200_device_error(ctypes.byref(code)))
    assert code.value == 0                                           # cleared by the read
    # The context is intact: an ordinary operator still runs and is still exact.
    x = cs.bf16(torch.randn(5, 256, generator=torch.Generator().manual_seed(1)))
    out, scale, scratch = quant_buffers(5, 256)
    check(lib.carat_b200_quantize_bf16_to_fp8(ptr(dev(x)), ptr(out), ptr(scale), ptr(scratch), 5,
                                              256, None))
    torch.cuda.synchronize()
    assert_quantised(out, scale, x)
