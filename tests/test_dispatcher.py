"""Request placement and the multi-replica dispatcher, on CPU.

Placement inside one replica is the reference's select_placement: checked against the cases of the
reference's tests/slot_policy_tests.cpp:75-176 (restated as data) and, where the reference's own
slot_policy.cpp was compiled into oracle/_ref, against that code on random slot tables. Routing
across replicas and the dispatcher have no counterpart in the single-GPU reference; they are
tested for their stated rule and for the one property that matters: whatever the routing, the
cache reuse and the loss of a replica, every request's token stream is the greedy stream of the
model. The model here is a deterministic stand-in with the runner's methods, which also checks the
KV bookkeeping (positions, clones, prefixes) the scheduler asks of a runner.
"""
import ctypes
import os
import pickle
import random
import socket
import subprocess
import sys
import textwrap

import pytest

from carat_b200 import capi, dispatcher
from carat_b200.dispatcher import (Dispatcher, LocalChannel, ReplicaScheduler, ReplicaWorker,
                                   Request, Router)
from oracle import carat_semantics as cs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def place(input_ids, slots, reserve=0):
    """slots: (cached tokens, occupied, age[, prefilling]) -> (decision, destination, source,
    prefix) through the C entry point."""
    keep = []
    views = (capi.SlotView * len(slots))()
    for index, state in enumerate(slots):
        tokens, occupied, age = state[:3]
        prefilling = state[3] if len(state) > 3 else False
        array = (ctypes.c_int * max(len(tokens), 1))(*tokens)
        keep.append(array)
        views[index] = capi.SlotView(ctypes.cast(array, ctypes.POINTER(ctypes.c_int)), len(tokens), int(occupied), age, int(prefilling))
    placement = capi.Placement()
    ids = (ctypes.c_int * len(input_ids))(*input_ids)
    capi.check(capi.library().carat_b200_select_placement(ids, len(input_ids), views, len(slots),
                                                       reserve, ctypes.byref(placement)))
    return (placement.decision, placement.destination, placement.source,
            placement.prefix_tokens)


# (input, slots, reserve) -> (destination, source or -1, prefix): slot_policy_tests.cpp:75-146.
PLACED_CASES = [
    (([1, 2], [([], False, 0), ([9], False, 0)], 0), (0, -1, 0)),
    (([1, 2, 3], [([1], False, 0), ([1, 2], False, 0), ([1, 2, 3, 4], False, 0)], 0), (1, 1, 2)),
    (([1, 2, 3], [([1, 2], True, 0), ([1, 2], False, 0)], 0), (1, 1, 2)),
    (([1, 2, 3], [([1, 2], False, 0), ([1, 2], True, 0)], 0), (0, 0, 2)),
    (([1, 2, 3], [([7], False, 1), ([1, 2], True, 0), ([], False, 0)], 0), (2, 1, 2)),
    (([1], [([5], True, 0), ([6], False, 9), ([7], False, 3), ([8], False, 3)], 0), (2, -1, 0)),
    (([1, 2, 3], [([1, 2], False, 0), ([1, 2, 3], True, 0, True), ([], False, 0)], 0), (0, 0, 2)),
    (([1, 2, 3], [([1, 2], True, 0, True), ([], False, 0)], 0), (1, 0, 2)),
    (([1, 2, 3], [([1, 2, 3], True, 0, False), ([], False, 0)], 0), (1, 0, 3)),
    (([9], [([5, 5, 5], True, 0), ([6, 6], False, 1)], 0), (1, -1, 0)),
    (([9], [([6, 6], False, 1)], 1), (0, -1, 0)),
    (([9], [([5], True, 0), ([6, 6], False, 1), ([7, 7], False, 2)], 1), (1, -1, 0)),
    (([5, 5, 1], [([5, 5], True, 0), ([6, 6], False, 1)], 1), (1, 0, 2)),
]
# slot_policy_tests.cpp:148-175.
REFUSED_CASES = [
    (([1], [([], True, 0), ([1], True, 0)], 1), dispatcher.NO_FREE_SLOT),
    (([9], [([5, 5, 5], True, 0), ([6, 6], False, 1)], 1), dispatcher.RESERVE_BLOCKED),
    (([9], [([5], True, 0), ([6, 6], False, 1), ([7, 7], False, 2)], 2),
     dispatcher.RESERVE_BLOCKED),
    (([5, 1], [([5], True, 0), ([6, 6], False, 1)], 1), dispatcher.RESERVE_BLOCKED),
]


def test_placement_reproduces_the_references_cases():
    for arguments, want in PLACED_CASES:
        decision, destination, source, prefix = place(*arguments)
        assert decision == dispatcher.PLACED, arguments
        assert (destination, source, prefix) == want, arguments
    for arguments, want in REFUSED_CASES:
        assert place(*arguments)[0] == want, arguments


def random_table(generator, slot_count):
    def tokens():
        return [generator.randint(1, 2) for _ in range(generator.randint(0, 4))]
    return [(tokens(), generator.random() < 0.5, generator.randint(0, 5),
             generator.random() < 0.3) for _ in range(slot_count)]


def test_placement_equals_the_compiled_reference_on_random_tables():
    path = os.path.join(ROOT, "oracle", "_ref", "libref_speculation.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref was not built (the reference tree is absent on this machine)")
    reference = ctypes.CDLL(path)
    if not hasattr(reference, "ref_select_placement"):
        pytest.skip("oracle/_ref predates the placement wrapper")
    generator = random.Random(11)
    outcomes = [0, 0, 0]
    for _ in range(4000):
        slots = random_table(generator, generator.randint(1, 6))
        input_ids = [generator.randint(1, 2) for _ in range(generator.randint(1, 5))]
        reserve = generator.randint(0, 2)
        flat = [token for state in slots for token in state[0]]
        offsets = [0]
        for state in slots:
            offsets.append(offsets[-1] + len(state[0]))
        destination, source = ctypes.c_int(-7), ctypes.c_int(-7)
        prefix = ctypes.c_ulonglong(0)
        decision = reference.ref_select_placement(
            (ctypes.c_int * len(input_ids))(*input_ids), len(input_ids),
            (ctypes.c_int * max(len(flat), 1))(*flat), (ctypes.c_int * len(offsets))(*offsets),
            (ctypes.c_int * len(slots))(*[int(state[1]) for state in slots]),
            (ctypes.c_ulonglong * len(slots))(*[state[2] for state in slots]),
            (ctypes.c_int * len(slots))(*[int(state[3]) for state in slots]),
            len(slots), reserve, ctypes.byref(destination), ctypes.byref(source),
            ctypes.byref(prefix))
        ours = place(input_ids, slots, reserve)
        assert ours[0] == decision, (input_ids, slots, reserve)
        outcomes[decision] += 1
        if decision == 0:
            assert ours[1:] == (destination.value, source.value, prefix.value), \
                (input_ids, slots, reserve)
    assert all(count > 50 for count in outcomes), outcomes


def test_host_speculation_logic_equals_the_oracle():
    generator = random.Random(5)
    for _ in range(3000):
        depth = generator.randint(1, 8)
        proposals = [generator.randint(1, 6) for _ in range(depth)]
        stops = frozenset(generator.sample(range(1, 7), generator.randint(0, 2)))
        remaining = generator.randint(0, 10)
        assert dispatcher.acceptance_cap(depth, remaining, proposals, stops) == \
            cs.acceptance_cap(depth, remaining, proposals, set(stops))
        accepted = generator.randint(0, depth)
        drafts = proposals[1:accepted] if accepted > 1 else []
        next_token = generator.randint(1, 6)
        ours = dispatcher.commit_speculation(proposals[0], drafts, next_token, stops)
        assert tuple(ours) == tuple(cs.commit_speculation(proposals[0], drafts, next_token,
                                                          set(stops)))


def test_routing_prefers_prefix_then_load_then_index_and_skips_lost_replicas():
    router = Router(3, 2)
    assert router.route([1, 2, 3]).replica == 0                     # all equal: lowest index
    router.tables[0][0].occupied = True
    assert router.route([1, 2, 3]).replica == 1                     # least loaded
    router.tables[2][1].cached_tokens = [1, 2]
    placement = router.route([1, 2, 3])
    assert (placement.replica, placement.destination, placement.source,
            placement.prefix_tokens) == (2, 1, 1, 2)                # cached prefix wins over load
    router.tables[2][0].occupied = True
    assert router.route([1, 2, 3]).replica == 2                     # ... even when it is busier
    router.mark_left(2)
    assert router.route([1, 2, 3]).replica == 1
    for replica in (0, 1):
        for record in router.tables[replica]:
            record.occupied = True
    assert router.route([1, 2, 3]) == dispatcher.NO_FREE_SLOT
    blocked = Router(1, 2, idle_cache_reserve_slots=1)
    blocked.tables[0][0].occupied = True
    blocked.tables[0][1].cached_tokens = [6, 6]
    assert blocked.route([9]) == dispatcher.RESERVE_BLOCKED


# ---------------------------------------------------------------------------------------------
# A deterministic stand-in for the runner.

def model_next(tokens):
    state = 17
    for token in tokens[-6:]:
        state = (state * 31 + token * 7 + 3) % 1009
    return state % 50 + 2


def greedy_stream(prompt, max_tokens, stop_ids=()):
    tokens, out = list(prompt), []
    while len(out) < max_tokens:
        out.append(model_next(tokens))
        tokens.append(out[-1])
        if out[-1] in stop_ids:
            break
    return out


class Verification:
    def __init__(self, accepted, following):
        self.accepted_tokens, self.next_tokens = accepted, following


class StandInRunner:
    """Keeps, per slot, the tokens whose KV is resident, and refuses any call a real runner
    would refuse or silently get wrong (a prefix that is not resident, a draft from the wrong
    last token)."""

    def __init__(self, slots, assistant=True, draft_hits=3):
        self.resident = [[] for _ in range(slots)]
        self.assistant, self.draft_hits = assistant, draft_hits
        self.calls = {"verify": 0, "append": 0, "clone": 0, "prefill_tokens": 0}

    def has_assistant(self):
        return self.assistant

    def slot_position(self, slot):
        return len(self.resident[slot])

    def reset_slot(self, slot):
        self.resident[slot] = []

    def clone_slot(self, source, destination):
        self.resident[destination] = list(self.resident[source])
        self.calls["clone"] += 1
        return 0

    def prefill_slots_chunks(self, slots, token_ids, chunk_tokens):
        out = []
        for slot, tokens in zip(slots, token_ids):
            resident = len(self.resident[slot])
            assert self.resident[slot] == list(tokens[:resident]), "prefix not resident"
            assert resident < len(tokens)
            advance = min(chunk_tokens, len(tokens) - resident)
            self.calls["prefill_tokens"] += advance
            self.resident[slot] = list(tokens[:resident + advance])
            done = resident + advance == len(tokens)
            out.append(model_next(self.resident[slot]) if done else None)
        return out

    def append_ragged(self, token_ids, slots):
        self.calls["append"] += 1
        out = []
        for token, slot in zip(token_ids, slots):
            self.resident[slot].append(token)
            out.append(model_next(self.resident[slot]))
        return out

    def draft_four(self, last_tokens, slots, forced_first_tokens=(), depth=4):
        proposals = []
        for row, slot in enumerate(slots):
            assert self.resident[slot][-1] == last_tokens[row]
            tokens = list(self.resident[slot])
            row_out = [forced_first_tokens[row]]
            tokens.append(row_out[0])
            for index in range(1, depth):
                guess = model_next(tokens)
                if index > (len(tokens) + slot) % (self.draft_hits + 1):
                    guess = guess % 50 + 2 if guess != 2 else 3     # a wrong guess now and then
                row_out.append(guess)
                tokens.append(guess)
            proposals.append(row_out)
        return proposals

    def verify_greedy_proposals(self, proposals, target_first_tokens, slots,
                                maximum_accepted_tokens=(), flags=0):
        self.calls["verify"] += 1
        assert len(set(slots)) == len(slots)
        positions = [len(self.resident[slot]) for slot in slots]
        assert positions == sorted(positions), "cohort is not ordered by position"
        accepted_out, next_out = [], []
        for row, slot in enumerate(slots):
            assert proposals[row][0] == target_first_tokens[row]
            tokens = list(self.resident[slot])
            accepted, following = 0, 0
            for index, token in enumerate(proposals[row]):
                if index >= maximum_accepted_tokens[row]:
                    break
                if index > 0 and token != following:
                    break
                tokens.append(token)
                following = model_next(tokens)
                accepted += 1
            self.resident[slot] = tokens
            accepted_out.append(accepted)
            next_out.append(following)
        return Verification(accepted_out, next_out)


def drive(front, workers, rounds=4000):
    for _ in range(rounds):
        front.poll()
        for worker in workers:
            worker.step()
        if front.finished():
            front.poll()
            return
    raise AssertionError("requests did not finish")


def make_requests(generator, count, shared_prefixes):
    requests = []
    for request_id in range(count):
        prefix = generator.choice(shared_prefixes)
        suffix = [generator.randint(2, 40) for _ in range(generator.randint(1, 6))]
        stops = frozenset({generator.randint(2, 51)}) if generator.random() < 0.5 else frozenset()
        requests.append(Request(request_id, prefix + suffix, generator.randint(1, 40), stops))
    return requests


@pytest.mark.parametrize("assistant", [True, False])
def test_streams_are_the_greedy_streams_whatever_the_routing(assistant):
    generator = random.Random(3)
    channel = LocalChannel()
    front = Dispatcher(channel, replica_count=3, slots_per_replica=4)
    runners = [StandInRunner(4, assistant) for _ in range(3)]
    workers = [ReplicaWorker(channel, replica, ReplicaScheduler(runners[replica], 4, depth=5))
               for replica in range(3)]
    # Conversations: every later round continues some finished ones (previous prompt + the
    # answer + a new turn), which is what leaves a reusable cache behind in the reference too.
    requests = make_requests(generator, 10, [[]])
    for request in requests:
        front.submit(request)
    drive(front, workers)
    follow_ups = 0
    stayed = 0
    for _ in range(5):
        batch = []
        for previous in generator.sample(requests, 6):
            history = previous.input_ids + front.completed[previous.request_id]
            turn = [generator.randint(2, 40) for _ in range(generator.randint(1, 4))]
            batch.append(Request(len(requests) + len(batch), history + turn,
                                 generator.randint(1, 30)))
            batch[-1].previous = previous.request_id
        for _ in range(2):
            batch.append(Request(len(requests) + len(batch),
                                 [generator.randint(2, 40) for _ in range(7)],
                                 generator.randint(1, 30)))
        for request in batch:
            front.submit(request)
        drive(front, workers)
        for request in batch:
            placement = front.placements[request.request_id][0]
            if hasattr(request, "previous") and placement.prefix_tokens > 0:
                follow_ups += 1
                stayed += placement.replica == front.placements[request.previous][-1].replica
        requests += batch
    for request in requests:
        assert front.completed[request.request_id] == greedy_stream(
            request.input_ids, request.max_tokens, request.stop_ids), request
    total = front.aggregate_metrics()
    assert total["prefix_tokens_reused"] > 0 and follow_ups >= 10
    assert stayed == follow_ups          # a cached prefix is only ever reused where it lives
    assert sum(runner.calls["prefill_tokens"] for runner in runners) == total["prefill_tokens"]
    if assistant:
        assert total["speculative_cycles"] > 0 and total["accepted_tokens"] > 0
        assert total["first_token_rejections"] == 0     # the forced first row is always accepted
    else:
        assert total["speculative_cycles"] == 0


def test_a_lost_replica_has_its_requests_continued_elsewhere():
    generator = random.Random(9)
    channel = LocalChannel()
    front = Dispatcher(channel, replica_count=2, slots_per_replica=3, report_timeout=0.05)
    workers = [ReplicaWorker(channel, replica, ReplicaScheduler(StandInRunner(3), 3, depth=4))
               for replica in range(2)]
    requests = [Request(index, [generator.randint(2, 40) for _ in range(5)], 30)
                for index in range(6)]
    for request in requests:
        front.submit(request)
    for _ in range(3):                      # both replicas work for three rounds ...
        front.poll()
        for worker in workers:
            worker.step()
    assert any(owner == 1 for owner, _ in front.assigned.values())
    import time
    deadline = time.monotonic() + 10.0
    while not front.finished():             # ... then replica 1 is gone, between two steps
        front.poll()
        workers[0].step()
        assert time.monotonic() < deadline
    assert front.lost == [1]
    for request in requests:
        assert front.completed[request.request_id] == greedy_stream(request.input_ids, 30)
    assert all(placement.replica == 0 for placements in front.placements.values()
               for placement in placements[1:])


PROCESS = textwrap.dedent("""
    import os, pickle, sys, time
    from datetime import timedelta
    sys.path.insert(0, os.environ["CARAT_ROOT"]); sys.path.insert(0, os.environ["CARAT_TESTS"])
    from torch.distributed import TCPStore
    from carat_b200.dispatcher import (Dispatcher, ReplicaScheduler, ReplicaWorker, Request,
                                       StoreChannel)
    import test_dispatcher as shared
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    store = TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]), world, rank == 0,
                     timeout=timedelta(seconds=60))
    channel = StoreChannel(store)
    if rank == 0:
        front = Dispatcher(channel, world - 1, 3, report_timeout=4.0)
        with open(os.environ["CARAT_REQUESTS"], "rb") as source:
            requests = pickle.load(source)
        for request in requests:
            front.submit(request)
        deadline = time.monotonic() + 90
        while not front.finished() and time.monotonic() < deadline:
            front.poll()
            time.sleep(0.002)
        front.stop_replicas()
        survivors = [replica for replica in range(world - 1) if front.router.alive[replica]]
        store.wait([f"carat/bye/{replica}" for replica in survivors], timedelta(seconds=30))
        with open(os.environ["CARAT_RESULT"], "wb") as out:
            pickle.dump({"completed": front.completed, "lost": front.lost,
                         "placements": {key: [(p.replica, p.prefix_tokens) for p in value]
                                        for key, value in front.placements.items()},
                         "metrics": front.aggregate_metrics()}, out)
    else:
        replica = rank - 1
        worker = ReplicaWorker(channel, replica,
                               ReplicaScheduler(shared.StandInRunner(3), 3, depth=5))
        leaves = int(os.environ["CARAT_LEAVER"]) == replica
        worker.run(leave_after_ticks=6 if leaves else None)
        if leaves:
            os._exit(0)          # no goodbye: the router has to notice by itself
        store.set(f"carat/bye/{replica}", b"1")
""")


def free_port():
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        return probe.getsockname()[1]


@pytest.mark.parametrize("leaver", [-1, 1])
def test_router_and_replicas_as_processes_over_a_store(tmp_path, leaver):
    """World size 4: a router and three replica processes; in the second case replica 1 exits
    between two steps without telling anybody."""
    generator = random.Random(21)
    prefixes = [[generator.randint(2, 40) for _ in range(10)] for _ in range(2)]
    requests = make_requests(generator, 24, prefixes)
    for request in requests:
        request.max_tokens += 40            # long enough to be in flight when the replica leaves
    script = tmp_path / "process.py"
    script.write_text(PROCESS)
    (tmp_path / "requests.pkl").write_bytes(pickle.dumps(requests))
    environment = dict(os.environ, CARAT_ROOT=ROOT, CARAT_TESTS=os.path.join(ROOT, "tests"),
                       MASTER_PORT=str(free_port()), WORLD_SIZE="4", CARAT_LEAVER=str(leaver),
                       CARAT_REQUESTS=str(tmp_path / "requests.pkl"),
                       CARAT_RESULT=str(tmp_path / "result.pkl"))
    processes = [subprocess.Popen([sys.executable, str(script)], env=dict(environment,
                                                                          RANK=str(rank)),
                                  cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                                  text=True) for rank in range(4)]
    try:
        for process in processes:
            _, errors = process.communicate(timeout=240)
            assert process.returncode == 0, errors[-3000:]
    finally:
        for process in processes:
            if process.poll() is None:
                process.kill()
    result = pickle.loads((tmp_path / "result.pkl").read_bytes())
    assert result["lost"] == ([] if leaver < 0 else [leaver])
    for request in requests:
        assert result["completed"][request.request_id] == greedy_stream(
            request.input_ids, request.max_tokens, request.stop_ids), request
    used = {replica for placements in result["placements"].values() for replica, _ in placements}
    assert used == {0, 1, 2}
    if leaver >= 0:
        moved = [placements for placements in result["placements"].values() if len(placements) > 1]
        assert moved and all(placements[0][0] == leaver and placements[-1][0] != leaver
                             for placements in moved)


def test_a_stale_prefix_decision_falls_back_to_a_fresh_prefill():
    """The router decides on its mirror of a replica's table; a source slot that was decoding has
    moved on by the time the replica admits the request. Its cache then no longer is the prefix
    the router saw, and the request must prefill from an empty slot instead of cloning it."""
    runner = StandInRunner(3)
    scheduler = ReplicaScheduler(runner, 3, depth=4)
    first = Request(1, [5, 6, 7, 8], 40)
    scheduler.admit(first, 0, None, 0)
    scheduler.tick()                                   # prefill + first decode step
    seen = list(scheduler.slots[0].cached_tokens)      # what a router would have mirrored
    for _ in range(3):
        scheduler.tick()                               # ... and the slot decodes on
    assert len(scheduler.slots[0].cached_tokens) > len(seen)
    follower = Request(2, seen + [9, 9], 6)
    scheduler.admit(follower, 1, 0, len(seen))         # the router's (stale) decision: clone slot 0
    assert scheduler.metrics["stale_prefix_fallbacks"] == 1
    assert scheduler.metrics["kv_clones"] == 0
    outputs = {1: [], 2: []}
    for _ in range(60):
        emitted, _ = scheduler.tick()
        for request_id, tokens in emitted.items():
            outputs[request_id] += tokens
        if scheduler.idle():
            break
    assert outputs[2] == greedy_stream(follower.input_ids, 6)
    assert runner.calls["clone"] == 0
