"""The replica scheduler and the dispatcher over real runners on the GPU (tiny model).

What a stand-in runner cannot show: that the calls the scheduler makes are calls the C library
accepts in that order (reset, clone, prefill from a resident prefix, draft, verify with caps,
plain-decode fall-back), and that the host's idea of every slot (cached tokens) stays equal to the
device's position after every step. Token streams of a speculative cohort are not compared with
a plain decode of the same prompt: the rows of a call share one activation scale, so the two are
different computations and part at near-ties.
"""
import pytest
import torch

import helpers
from carat_b200.dispatcher import Dispatcher, LocalChannel, ReplicaScheduler, ReplicaWorker, Request
from oracle import carat_semantics as cs

pytestmark = pytest.mark.gpu

SLOTS = 4


def build_runner(seed):
    config = cs.tiny_config(512)
    assistant = cs.tiny_assistant()
    weights = cs.random_weights(config, seed=seed)
    assistant_weights = cs.random_assistant_weights(config, assistant, seed=seed + 1)
    _, device, _ = helpers.build_pair(config, weights, SLOTS, assistant, assistant_weights)
    return config, device


def check_positions(worker):
    for index, slot in enumerate(worker.scheduler.slots):
        if slot.request is not None or slot.cached_tokens:
            assert worker.scheduler.engine.slot_position(index) == len(slot.cached_tokens), index


def test_two_replicas_serve_conversations_with_prefix_reuse(cuda_device):
    config, first = build_runner(seed=5)
    _, second = build_runner(seed=5)
    channel = LocalChannel()
    front = Dispatcher(channel, replica_count=2, slots_per_replica=SLOTS)
    workers = [ReplicaWorker(channel, replica, ReplicaScheduler(runner, SLOTS, depth=5))
               for replica, runner in enumerate((first, second))]
    generator = torch.Generator().manual_seed(2)

    def tokens(count):
        return torch.randint(3, config.vocab, (count,), generator=generator).tolist()

    def drive():
        for _ in range(500):
            front.poll()
            for worker in workers:
                worker.step()
                check_positions(worker)
            if front.finished():
                front.poll()
                return
        raise AssertionError("requests did not finish")

    opening = [Request(index, tokens(20 + 3 * index), 12 + index) for index in range(6)]
    for request in opening:
        front.submit(request)
    drive()
    for request in opening:
        assert len(front.completed[request.request_id]) == request.max_tokens
    # Second turns: history + answer + a few new tokens; each must go back to the replica that
    # holds its cache and reuse it (in place or, if that slot is busy, by a clone).
    following = []
    for request in opening:
        history = request.input_ids + front.completed[request.request_id]
        following.append(Request(100 + request.request_id, history + tokens(3), 9))
        following.append(Request(200 + request.request_id, history + tokens(2), 7))
    for request in following:
        front.submit(request)
    drive()
    reused = 0
    for request in following:
        assert len(front.completed[request.request_id]) == request.max_tokens
        placement = front.placements[request.request_id][0]
        origin = front.placements[request.request_id % 100][0]
        if placement.prefix_tokens:
            reused += 1
            assert placement.replica == origin.replica
    total = front.aggregate_metrics()
    assert reused >= 6 and total["prefix_tokens_reused"] > 0
    assert total["speculative_cycles"] > 0
    assert total["accepted_tokens"] >= total["speculative_cycles"]
    # The two replicas are the same model: an opening prompt gets the same first token on either.
    probe = opening[0].input_ids
    assert first.prefill_slot(0, probe) == second.prefill_slot(0, probe) == \
        front.completed[opening[0].request_id][0]
    first.close()
    second.close()


def test_plain_decode_path_without_an_assistant(cuda_device):
    config = cs.tiny_config(512)
    weights = cs.random_weights(config, seed=8)
    _, runner, _ = helpers.build_pair(config, weights, SLOTS)
    channel = LocalChannel()
    front = Dispatcher(channel, 1, SLOTS)
    worker = ReplicaWorker(channel, 0, ReplicaScheduler(runner, SLOTS))
    generator = torch.Generator().manual_seed(4)
    requests = [Request(index, torch.randint(3, config.vocab, (15 + index,),
                                             generator=generator).tolist(), 6)
                for index in range(SLOTS + 2)]
    for request in requests:
        front.submit(request)
    for _ in range(200):
        front.poll()
        worker.step()
        check_positions(worker)
        if front.finished():
            break
    front.poll()
    # One request alone in a slot: prefill then append_ragged of a cohort whose other rows do
    # not change its own (BF16 prefill has no shared scale; the first token is comparable).
    for request in requests:
        assert len(front.completed[request.request_id]) == 6
    runner.reset_slot(0)
    assert runner.prefill_slot(0, requests[0].input_ids) == front.completed[0][0]
    assert front.aggregate_metrics()["speculative_cycles"] == 0
    runner.close()
