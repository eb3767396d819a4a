"""k = 8 drafts at a full batch: 24 slots x depth 9 = 216 verify rows in one step, more than the
128 rows of the k = 4 benchmark shape and more than the device holds row-kernel CTAs at once. The
FP8 linears then run their 256-row form (UMMA N = 256) and the row kernels their two-launch form.
Tiny plumbing configuration, teacher-forced against the oracle like the other runner tests."""
import copy

import pytest
import torch

import carat_b200
import helpers
from helpers import build_pair, rms_relative_error
from oracle import carat_semantics as cs

pytestmark = pytest.mark.gpu

SLOTS = 24
DEPTH = 9
TOLERANCE = 0.12


def test_full_batch_depth_nine(cuda_device):
    config = cs.tiny_config(512)
    weights = cs.golden_tiny_weights(config)
    oracle, device, _ = build_pair(config, weights, SLOTS)
    generator = torch.Generator().manual_seed(21)
    slots = list(range(SLOTS))
    # Ragged short contexts: every slot is prefilled alone (bit-exact state on both sides when the
    # slot was empty), some past the 128-row ring.
    for slot in slots:
        length = 4 + (slot * 7) % 40 + (150 if slot % 5 == 0 else 0)
        text = torch.randint(3, config.vocab, (length,), generator=generator).tolist()
        for start in range(0, length, 8):
            part = text[start:start + 8]
            device.prefill_slot_fp8(slot, part, 8)
            oracle.verify_greedy_proposals([part], [part[0]], [slot], assume_match=True,
                                           allow_empty_slot=True)
        assert device.slot_position(slot) == oracle.positions[slot] == length
    proposals = torch.randint(3, config.vocab, (SLOTS, DEPTH), generator=generator).tolist()
    firsts = [row[0] for row in proposals]
    caps = [1 + (slot * 5) % DEPTH for slot in slots]
    scout = copy.deepcopy(oracle)
    _, _, trace = scout.verify_greedy_proposals(proposals, firsts, slots, caps, assume_match=True,
                                                trace=True)
    starts = [device.slot_position(slot) for slot in slots]
    # The INT4 MLP variant takes at most 128 rows a step (the reference's Int4Bf16Linear::
    # supports_rows): 216 rows are refused before any launch, with the reference's text, and the
    # state is untouched; wrong shapes are refused when the variant is switched on.
    arena = carat_b200.DeviceWeightArena.from_host(weights)
    with pytest.raises(carat_b200.CaratError, match="invalid BF16 INT4 linear weight shape"):
        device.use_int4_mlp(arena, 64)
    device.use_int4_mlp(arena, 128)
    with pytest.raises(carat_b200.CaratError, match="invalid BF16 INT4 linear activation shape"):
        device.verify_greedy_proposals(proposals, firsts, slots, caps,
                                       carat_b200.VERIFY_ASSUME_MATCH)
    assert [device.slot_position(slot) for slot in slots] == starts
    device.use_int4_mlp(None)
    result = device.verify_greedy_proposals(proposals, firsts, slots, caps,
                                            carat_b200.VERIFY_ASSUME_MATCH)
    assert result.accepted_tokens == caps
    predictions = device.last_predictions(SLOTS * DEPTH)
    want = cs.greedy_prefix_accept([list(p) for p in proposals], firsts, predictions, caps, DEPTH,
                                   True)
    assert (result.accepted_tokens, result.next_tokens) == want
    hidden = device.last_final_hidden(SLOTS * DEPTH)
    assert rms_relative_error(hidden, trace.final_hidden) < TOLERANCE
    flagged = 0
    for row, (got, expected) in enumerate(zip(predictions, trace.predictions.tolist())):
        if got != expected:
            logits = trace.logits[row]
            assert helpers.near_tie(logits, got, helpers.NEAR_TIE_RELATIVE_TINY), (row, got, expected)
            flagged += 1
    assert flagged <= SLOTS * DEPTH // 4     # random-init logits are flat: near-ties are common
    for request, slot in enumerate(slots):
        assert device.slot_position(slot) == starts[request] + caps[request]
    # Real acceptance (no injected match): the device's own predictions decide.
    result = device.verify_greedy_proposals(proposals, firsts, slots)
    predictions = device.last_predictions(SLOTS * DEPTH)
    want = cs.greedy_prefix_accept([list(p) for p in proposals], firsts, predictions, [], DEPTH,
                                   False)
    assert (result.accepted_tokens, result.next_tokens) == want
