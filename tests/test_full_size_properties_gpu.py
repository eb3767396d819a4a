"""The whole step at the benchmark's full size (31B shapes: 60 layers, hidden 5376, vocabulary
262144, 24 slots, contexts of 128..6144 tokens), checked through properties that need no oracle
run of that size:

  * twins: slot 2i+1 is a clone of slot 2i (clone_slot) and gets the same tokens, so every integer
    the step produces for the pair (drafts, predictions, accept lengths, next tokens) and every
    row it commits must be identical, whatever rows the two occupy in the batch;
  * bookkeeping: accept lengths and next tokens are exactly the reference's greedy prefix-accept
    rule (cuda/batch_model_runner.cu:1735-1759, restated in the oracle) applied to the device's
    own predictions and the caps; positions advance by the accept lengths;
  * rollback: sliding-ring rows of rejected proposals keep their bytes, accepted rows change;
  * plain decode of the twins agrees as well.
"""
import pytest
import torch

import bench
from oracle import carat_semantics as cs

pytestmark = pytest.mark.gpu

DEPTH = 5


def test_twin_slots_and_bookkeeping_at_full_size(cuda_device):
    config, runner, _ = bench.build_model(seed=0)
    slots = list(range(bench.SLOTS))
    positions = bench.context_lengths(seed=3)
    for even in range(0, bench.SLOTS, 2):
        positions[even + 1] = positions[even]
    runner.seed_slot_positions(positions)
    bench.fill_kv(runner, config, seed=5)
    generator = torch.Generator(device="cuda").manual_seed(9)
    table = torch.randn(bench.SLOTS, config.hidden_size, device="cuda", generator=generator,
                        dtype=torch.bfloat16)
    runner.write_cache(2, 0, table)
    for even in range(0, bench.SLOTS, 2):
        assert runner.clone_slot(even, even + 1) > 0
    host = torch.Generator().manual_seed(4)

    def twinned(high):
        values = torch.randint(3, high, (bench.SLOTS // 2,), generator=host).tolist()
        return [value for value in values for _ in range(2)]

    last, firsts = twinned(config.vocabulary_size), twinned(config.vocabulary_size)
    caps = twinned(DEPTH + 1)
    caps = [max(1, cap) for cap in caps]

    drafted = runner.draft_four(last, slots, firsts, DEPTH)
    for even in range(0, bench.SLOTS, 2):
        assert drafted[even] == drafted[even + 1], even
        assert drafted[even][0] == firsts[even]

    sliding = [index for index, layer in enumerate(config.layers) if layer.attention == "sliding"]
    watched = [sliding[0], sliding[-1]]
    before = {index: (runner.key_cache(index, config.sliding_window).clone(),
                      runner.value_cache(index, config.sliding_window).clone())
              for index in watched}
    start = [runner.slot_position(slot) for slot in slots]
    assert start == positions

    # Rows 1.. of the proposals never match a random-init target, so feed it look-alike rows:
    # every proposal row is accepted as a match (benchmark flag) up to the caps.
    result = runner.verify_greedy_proposals(drafted, firsts, slots, caps, flags=1)
    predictions = runner.last_predictions(bench.SLOTS * DEPTH)
    want = cs.greedy_prefix_accept([list(row) for row in drafted], list(firsts), predictions,
                                   list(caps), DEPTH, True)
    assert (result.accepted_tokens, result.next_tokens) == want
    assert result.accepted_tokens == caps
    for even in range(0, bench.SLOTS, 2):
        assert predictions[even * DEPTH:(even + 1) * DEPTH] == \
            predictions[(even + 1) * DEPTH:(even + 2) * DEPTH], even
        assert result.next_tokens[even] == result.next_tokens[even + 1]
    for slot in slots:
        assert runner.slot_position(slot) == start[slot] + result.accepted_tokens[slot]

    window = config.sliding_window
    for index in watched:
        keys = runner.key_cache(index, window)
        values = runner.value_cache(index, window)
        for slot in slots:
            for t in range(DEPTH):
                row = (start[slot] + t) % window
                same = (torch.equal(keys[slot, :, row], before[index][0][slot, :, row])
                        and torch.equal(values[slot, :, row], before[index][1][slot, :, row]))
                assert same == (t >= result.accepted_tokens[slot]), (index, slot, t)
        for even in range(0, bench.SLOTS, 2):
            # Resident rows only: a clone copies what is resident, the rest of an unwrapped ring
            # is whatever the two slots held before and is never read.
            resident = min(start[even] + result.accepted_tokens[even], window)
            assert torch.equal(keys[even, :, :resident], keys[even + 1, :, :resident])
            assert torch.equal(values[even, :, :resident], values[even + 1, :, :resident])
    hand_off = runner.target_hidden_slots()
    for even in range(0, bench.SLOTS, 2):
        assert torch.equal(hand_off[even], hand_off[even + 1])

    # Plain decode from the committed state, and one more verify with the real accept rule
    # (random-init drafts: only the forced row can be accepted).
    following = runner.append_ragged(result.next_tokens, slots)
    for even in range(0, bench.SLOTS, 2):
        assert following[even] == following[even + 1]
    last = list(result.next_tokens)
    drafted = runner.draft_four(last, slots, following, DEPTH)
    real = runner.verify_greedy_proposals(drafted, following, slots)
    predictions = runner.last_predictions(bench.SLOTS * DEPTH)
    want = cs.greedy_prefix_accept([list(row) for row in drafted], list(following), predictions,
                                   [], DEPTH, False)
    assert (real.accepted_tokens, real.next_tokens) == want
    assert all(count >= 1 for count in real.accepted_tokens)
    for even in range(0, bench.SLOTS, 2):
        assert drafted[even] == drafted[even + 1]
        assert real.accepted_tokens[even] == real.accepted_tokens[even + 1]
        assert real.next_tokens[even] == real.next_tokens[even + 1]
    runner.close()
