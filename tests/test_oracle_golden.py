"""Pins the CPU oracle: the reference's own known-answer tests, the reference's compiled
speculation logic (when oracle/_ref was built), and the Hugging Face fixture."""
import ctypes
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import carat_semantics as cs

ORACLE_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle")
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def ints(values):
    values = list(values)
    return (ctypes.c_int * max(len(values), 1))(*values)


@pytest.fixture(scope="module")
def c_oracle():
    subprocess.run(["make", "-C", ORACLE_DIR, "all"], check=True, capture_output=True)
    return ctypes.CDLL(os.path.join(ORACLE_DIR, "_build", "liboracle_accept.so"))


@pytest.fixture(scope="module")
def reference_library():
    path = os.path.join(ORACLE_DIR, "_ref", "libref_speculation.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref was not built (the reference tree is absent on this machine)")
    return ctypes.CDLL(path)


# The reference's speculation_tests.cpp:15-60, restated as data: (depth, remaining, stops) -> cap.
PROPOSALS = [10, 11, 12, 13]
CAP_CASES = [((4, 10, []), 4), ((4, 2, []), 2), ((4, 0, []), 0), ((4, 10, [12]), 3),
             ((4, 10, [13, 11]), 2), ((4, 10, [10]), 4), ((4, 2, [12]), 2)]
# (forced, drafts, next, stops) -> (resident, emitted, next, stopped)
COMMIT_CASES = [((10, [11, 12], 20, [99]), ([10, 11, 12], [11, 12, 20], 20, False)),
                ((10, [], 20, []), ([10], [20], 20, False)),
                ((10, [11, 12], 20, [12]), ([10, 11, 12], [11, 12], 20, True))]


def test_python_oracle_reproduces_reference_speculation_tests():
    for (depth, remaining, stops), want in CAP_CASES:
        assert cs.acceptance_cap(depth, remaining, PROPOSALS, set(stops)) == want
    for (forced, drafts, nxt, stops), want in COMMIT_CASES:
        assert cs.commit_speculation(forced, drafts, nxt, set(stops)) == want


def call_cap(library, name, depth, remaining, proposals, stops):
    return getattr(library, name)(depth, remaining, ints(proposals), len(proposals), ints(stops),
                                  len(stops))


def call_commit(library, name, forced, drafts, nxt, stops, with_next):
    resident = (ctypes.c_int * (len(drafts) + 2))()
    emitted = (ctypes.c_int * (len(drafts) + 2))()
    resident_count = ctypes.c_int()
    emitted_count = ctypes.c_int()
    arguments = [forced, ints(drafts), len(drafts), nxt, ints(stops), len(stops), resident,
                 ctypes.byref(resident_count), emitted, ctypes.byref(emitted_count)]
    next_out = ctypes.c_int(nxt)
    if with_next:
        arguments.append(ctypes.byref(next_out))
    stopped = getattr(library, name)(*arguments)
    return (list(resident[:resident_count.value]), list(emitted[:emitted_count.value]),
            next_out.value, bool(stopped))


def test_c_oracle_reproduces_reference_speculation_tests(c_oracle):
    for (depth, remaining, stops), want in CAP_CASES:
        assert call_cap(c_oracle, "oracle_acceptance_cap", depth, remaining, PROPOSALS, stops) == want
    for (forced, drafts, nxt, stops), want in COMMIT_CASES:
        assert call_commit(c_oracle, "oracle_commit_speculation", forced, drafts, nxt, stops,
                           False) == want


def test_oracles_agree_with_the_compiled_reference(reference_library, c_oracle):
    generator = torch.Generator().manual_seed(0)
    for _ in range(500):
        depth = int(torch.randint(1, 10, (1,), generator=generator))
        remaining = int(torch.randint(0, 12, (1,), generator=generator))
        proposals = torch.randint(0, 8, (depth,), generator=generator).tolist()
        stops = torch.randint(0, 8, (int(torch.randint(0, 3, (1,), generator=generator)),),
                              generator=generator).tolist()
        want = call_cap(reference_library, "ref_acceptance_cap", depth, remaining, proposals, stops)
        assert cs.acceptance_cap(depth, remaining, proposals, set(stops)) == want
        assert call_cap(c_oracle, "oracle_acceptance_cap", depth, remaining, proposals, stops) == want
        drafts = proposals[1:]
        want = call_commit(reference_library, "ref_commit_speculation", proposals[0], drafts, 77,
                           stops, True)
        assert cs.commit_speculation(proposals[0], drafts, 77, set(stops)) == want
        assert call_commit(c_oracle, "oracle_commit_speculation", proposals[0], drafts, 77, stops,
                           False) == want


def test_argmax_tie_rule_known_answers(c_oracle):
    """tests/cuda_ops_tests.cu:1137-1164."""
    rows, elements = 3, 513
    values = torch.full((rows, elements), -2.0)
    values[0, 17] = 9.0
    values[1, 0] = 4.0
    values[1, 401] = 4.0
    values[2, 512] = 7.0
    assert cs.argmax_lowest_index(values).tolist() == [17, 0, 512]
    raw = values.to(torch.bfloat16).view(torch.int16).numpy().astype(np.uint16)
    output = (ctypes.c_int * rows)()
    c_oracle.oracle_argmax_bf16_rows(raw.ctypes.data_as(ctypes.c_void_p), rows, elements, output)
    assert list(output) == [17, 0, 512]


def test_c_accept_loop_matches_python(c_oracle):
    generator = torch.Generator().manual_seed(1)
    for assume in (0, 1):
        requests, depth = 24, 5
        predictions = torch.randint(0, 5, (requests, depth), generator=generator)
        proposals = predictions.roll(1, dims=1).clone()
        target_first = torch.randint(0, 5, (requests,), generator=generator)
        proposals[:, 0] = target_first
        proposals[torch.rand(requests, depth, generator=generator) < 0.3] = 9
        caps = torch.randint(-1, 7, (requests,), generator=generator)
        want = cs.greedy_prefix_accept(proposals.tolist(), target_first.tolist(),
                                       predictions.reshape(-1).tolist(), caps.tolist(), depth,
                                       bool(assume))
        accepted = (ctypes.c_int * requests)()
        next_tokens = (ctypes.c_int * requests)()
        c_oracle.oracle_greedy_prefix_accept(
            ints(proposals.reshape(-1).tolist()), ints(target_first.tolist()),
            ints(predictions.reshape(-1).tolist()), ints(caps.tolist()), requests, depth, assume,
            accepted, next_tokens)
        assert (list(accepted), list(next_tokens)) == want


def test_ring_attention_closed_form_case():
    """tests/cuda_ops_tests.cu:1630-1779 (q = 4 and 8): the reference's expected values come from
    plain float math over a full ring with backup substitution, tolerance 0.015."""
    from test_ops_gpu import reference_ring_case
    for query_tokens in (4, 8):
        query, old_k, old_v, new_k, new_v, logical, expected, capacity = reference_ring_case(
            query_tokens)
        got = cs.verify_attention(query.permute(0, 2, 1, 3), list(old_k), list(old_v),
                                  new_k.permute(0, 2, 1, 3), new_v.permute(0, 2, 1, 3), logical,
                                  capacity)
        assert (got.permute(0, 2, 1, 3) - expected).abs().max() < 0.015


def test_bf16_layer_math_matches_hugging_face_fixture():
    """tests/golden/hf_tiny_bf16.npz was produced by tests/golden/make_hf_golden.py with the
    Hugging Face Gemma4 text model (what the reference's fixture tools run). The reference accepts
    cosine >= 0.999 for a layer against such a fixture (src/layer_parity.cu:114)."""
    fixture = np.load(os.path.join(GOLDEN, "hf_tiny_bf16.npz"))
    config = cs.tiny_config(512)
    runner = cs.OracleRunner(config, cs.golden_tiny_weights(config), 1, fp8=False)
    tokens = fixture["tokens"].tolist()
    runner.prefill_slot_fp8(0, tokens[:-8], chunk=8)   # fp8=False: BF16 projections throughout
    _, _, trace = runner.verify_greedy_proposals([tokens[-8:]], [tokens[-8]], [0],
                                                 assume_match=True, trace=True)
    want = torch.tensor(fixture["final_hidden_tail"])
    cosine = torch.nn.functional.cosine_similarity(trace.final_hidden, want, dim=-1)
    assert float(cosine.min()) > 0.999
    assert float((trace.final_hidden - want).abs().max()) < 0.1
    top = fixture["logits_tail_top"]
    values = fixture["logits_tail_values"]
    for row, prediction in enumerate(trace.predictions.tolist()):
        if prediction != int(top[row, 0]):
            assert values[row, 0] - values[row, 1] < 0.05   # only near-ties may differ
            assert prediction in top[row].tolist()


def test_backup_restore_c_matches_python(c_oracle):
    generator = torch.Generator().manual_seed(4)
    requests, heads, tokens, dim, capacity = 3, 2, 5, 8, 16
    keys = [cs.bf16(torch.randn(heads, capacity, dim, generator=generator)) for _ in range(requests)]
    values = [cs.bf16(torch.randn(heads, capacity, dim, generator=generator)) for _ in range(requests)]
    positions = [3, 14, 30]
    want_k, want_v = cs.backup_kv_ring_spans(keys, values, positions, tokens)

    def raw(tensor):
        return np.ascontiguousarray(tensor.to(torch.bfloat16).view(torch.int16).numpy().astype(np.uint16))

    key_arrays = [raw(k) for k in keys]
    value_arrays = [raw(v) for v in values]
    pointer_type = ctypes.c_void_p * requests
    key_pointers = pointer_type(*[a.ctypes.data for a in key_arrays])
    value_pointers = pointer_type(*[a.ctypes.data for a in value_arrays])
    backup_k = np.zeros((requests, heads, tokens, dim), dtype=np.uint16)
    backup_v = np.zeros_like(backup_k)
    c_oracle.oracle_backup_kv_ring_spans(key_pointers, value_pointers,
                                         backup_k.ctypes.data_as(ctypes.c_void_p),
                                         backup_v.ctypes.data_as(ctypes.c_void_p), ints(positions),
                                         requests, heads, tokens, dim, capacity)
    assert np.array_equal(backup_k, raw(want_k))
    assert np.array_equal(backup_v, raw(want_v))
    accepted = [0, 2, 5]
    for r in range(requests):
        for t in range(tokens):
            row = (positions[r] + t) % capacity
            keys[r][:, row] = 1.0
            values[r][:, row] = 2.0
            key_arrays[r][:, row] = raw(torch.tensor(1.0))
            value_arrays[r][:, row] = raw(torch.tensor(2.0))
    cs.restore_kv_ring_suffixes(want_k, want_v, keys, values, positions, accepted, tokens)
    c_oracle.oracle_restore_kv_ring_suffixes(backup_k.ctypes.data_as(ctypes.c_void_p),
                                             backup_v.ctypes.data_as(ctypes.c_void_p), key_pointers,
                                             value_pointers, ints(positions), ints(accepted),
                                             requests, heads, tokens, dim, capacity)
    for r in range(requests):
        assert np.array_equal(key_arrays[r], raw(keys[r]))
        assert np.array_equal(value_arrays[r], raw(values[r]))


def test_int4_quantiser_follows_the_reference_test_oracle():
    """tests/cuda_ops_tests.cu:824-843 spells the INT4 representation out element by element
    (group maximum, bf16(max / 7), nearbyint, clamp to [-7, 7], bf16(code * scale)); the vectorised
    restatement must agree with that loop on the test's own weights, whose second group of every
    row is sixteen times larger than the first."""
    import struct

    from helpers import int4_reference_test_case

    def to_bf16(value):
        bits = struct.unpack("<I", struct.pack("<f", value))[0]
        bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
        return struct.unpack("<f", struct.pack("<I", bits))[0]

    def f32(value):
        return struct.unpack("<f", struct.pack("<f", value))[0]

    weight, _ = int4_reference_test_case()
    codes, scales = cs.int4_quantize(weight, 256)
    dequantised = cs.int4_dequantize(codes, scales, 256)
    packed = cs.int4_pack(codes)
    for row in (0, 1, 100, 255):
        for begin in (0, 256):
            values = [float(v) for v in weight[row, begin:begin + 256]]
            maximum = max(abs(v) for v in values)
            scale = to_bf16(f32(maximum / 7.0) if maximum > 0 else 1.0)
            assert float(scales[begin // 256, row]) == scale
            for offset, value in enumerate(values):
                code = max(-7, min(7, round(f32(value / scale))))
                assert int(codes[row, begin + offset]) == code
                assert float(dequantised[row, begin + offset]) == to_bf16(f32(code * scale))
                nibble = (int(packed[row, (begin + offset) // 2]) >> (4 * (offset & 1))) & 0xF
                assert nibble == code & 0xF
