"""Requests over several independent full-model replicas of one box (one runner per GPU).

The reference serves one GPU: its ContinuousScheduler (src/native_runtime_main.cpp:82-883) owns
one Gemma4BatchModelRunner and places requests into that runner's slots with
carat::select_placement (src/runtime/slot_policy.cpp:22-84). A 31B FP8 model with its KV fits one
B200, so a box of eight is eight such replicas that share nothing: no tensor ever crosses NVLink,
a slot never migrates, and the only box-level decision is which replica a request goes to. This
module is that decision and the plumbing round it:

  Router            mirrors every replica's slot table on the host and asks the C library
                    (carat_b200_route_request) for replica + slot: longest reusable cached prefix
                    first, then the least loaded replica, then the lowest index.
  ReplicaScheduler  the per-replica step loop, the part of the reference's scheduler that sits on
                    the hot path: admit (reset / clone / reuse in place), prefill, then
                    draft -> acceptance caps -> verify -> plain-decode fall-back for first-token
                    rejections -> commit (speculative_decode, native_runtime_main.cpp:583-678).
  Dispatcher        the router plus a request queue, driven by the replicas' reports; a replica
                    that stops reporting is marked lost and its unfinished requests continue on
                    another replica from the tokens already emitted.
  ReplicaWorker     a replica's process loop: commands in, one scheduler tick, one report out.

Messages travel through a key-value store (torch.distributed.TCPStore between processes, a dict
inside one process); the data path has no collective.
"""
from __future__ import annotations

import ctypes
import pickle
import time
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

from . import capi


# ---------------------------------------------------------------------------------------------
# Host logic of one speculative step (src/runtime/speculation.cpp:7-36).

def acceptance_cap(depth: int, remaining: int, proposals: Sequence[int], stop_ids) -> int:
    """How many rows of a slot's verify block may be accepted: never more than the tokens the
    request may still emit, and nothing after the first proposed stop token (index >= 1; the
    forced token at index 0 was checked when it was emitted)."""
    cap = min(depth, remaining)
    for index in range(1, min(cap, len(proposals))):
        if proposals[index] in stop_ids:
            return index + 1
    return cap


def commit_speculation(forced_token: int, accepted_drafts: Sequence[int], next_token: int,
                       stop_ids) -> Tuple[List[int], List[int], int, bool]:
    """(resident, emitted, next, stopped): the tokens the slot's cache now holds, the tokens the
    caller sees, the token to append next, and whether an accepted draft was a stop token. A
    stop token in `next` is the caller's to notice, as in the reference's finish_if_done."""
    resident, emitted = [forced_token], []
    for token in accepted_drafts:
        resident.append(token)
        emitted.append(token)
        if token in stop_ids:
            return resident, emitted, next_token, True
    emitted.append(next_token)
    return resident, emitted, next_token, False


# ---------------------------------------------------------------------------------------------
# Requests and slot tables.

@dataclass
class Request:
    request_id: int
    input_ids: List[int]
    max_tokens: int
    stop_ids: frozenset = frozenset()


@dataclass
class SlotRecord:
    """What the router knows of one slot (carat::SlotView, src/runtime/slot_policy.h:13-19)."""
    cached_tokens: List[int] = field(default_factory=list)
    occupied: bool = False
    age: int = 0
    prefilling: bool = False


@dataclass
class Placement:
    replica: int
    destination: int
    source: Optional[int]
    prefix_tokens: int


PLACED, NO_FREE_SLOT, RESERVE_BLOCKED = 0, 1, 2


class Router:
    """Slot tables of every replica and the routing rule over them."""

    def __init__(self, replica_count: int, slots_per_replica: int,
                 idle_cache_reserve_slots: int = 0):
        self.tables = [[SlotRecord() for _ in range(slots_per_replica)]
                       for _ in range(replica_count)]
        self.alive = [True] * replica_count
        self.queued = [0] * replica_count
        self.reserve = idle_cache_reserve_slots
        self._library = capi.library()

    def route(self, input_ids: Sequence[int]):
        """A Placement, or the reason there is none (NO_FREE_SLOT / RESERVE_BLOCKED)."""
        keep = []
        views = (capi.ReplicaView * len(self.tables))()
        for replica, table in enumerate(self.tables):
            slots = (capi.SlotView * len(table))()
            for index, record in enumerate(table):
                tokens = (ctypes.c_int * max(len(record.cached_tokens), 1))(*record.cached_tokens)
                keep.append(tokens)
                slots[index] = capi.SlotView(ctypes.cast(tokens, ctypes.POINTER(ctypes.c_int)), len(record.cached_tokens),
                                             int(record.occupied), record.age,
                                             int(record.prefilling))
            keep.append(slots)
            views[replica] = capi.ReplicaView(ctypes.cast(slots, ctypes.POINTER(capi.SlotView)), len(table), self.queued[replica],
                                              int(self.alive[replica]))
        ids = (ctypes.c_int * len(input_ids))(*input_ids)
        placement = capi.Placement()
        capi.check(self._library.carat_b200_route_request(
            ids, len(input_ids), views, len(self.tables), self.reserve, ctypes.byref(placement)))
        if placement.decision != PLACED:
            return placement.decision
        return Placement(placement.replica, placement.destination,
                         placement.source if placement.source >= 0 else None,
                         int(placement.prefix_tokens))

    def reserve_slot(self, placement: Placement, input_ids: Sequence[int]) -> None:
        """Book the destination before the replica's own report confirms it, so that the next
        request routed in the same round sees the slot taken."""
        table = self.tables[placement.replica]
        age = max(record.age for record in table) + 1
        table[placement.destination] = SlotRecord(list(input_ids[:placement.prefix_tokens]), True,
                                                  age, placement.prefix_tokens < len(input_ids))

    def apply_report(self, replica: int, changes: Iterable[tuple]) -> None:
        """changes: (slot, keep, extra, occupied, age, prefilling); the slot's cached tokens become
        the first `keep` it had plus `extra`."""
        for slot, keep, extra, occupied, age, prefilling in changes:
            record = self.tables[replica][slot]
            record.cached_tokens = record.cached_tokens[:keep] + list(extra)
            record.occupied, record.age, record.prefilling = occupied, age, prefilling

    def mark_left(self, replica: int) -> None:
        self.alive[replica] = False


# ---------------------------------------------------------------------------------------------
# One replica's step loop.

@dataclass
class _Slot:
    request: Optional[Request] = None
    cached_tokens: List[int] = field(default_factory=list)
    output_ids: List[int] = field(default_factory=list)
    token_to_append: int = 0
    decode_ready: bool = False
    age: int = 0
    reported: int = 0           # how many cached tokens the router has been told about
    inherited_token: Optional[int] = None   # whole prompt was cached: the source's prediction
    prompt_array: object = None             # the prompt as a C int array while it is prefilling
    dirty: bool = True


class ReplicaScheduler:
    """Drives one runner. `engine` is a Gemma4BatchModelRunner or anything with its methods
    (reset_slot, clone_slot, prefill_slots_chunks, draft_four, verify_greedy_proposals,
    append_ragged, has_assistant, slot_position). `chunk_tokens` is the prefill quantum: how many
    prompt tokens a slot advances per tick, so that decoding slots are not starved by a long
    prompt (the reference's idle_prefill_quantum_tokens)."""

    def __init__(self, engine, slots: int, depth: int = 5, speculative_minimum_batch: int = 1,
                 chunk_tokens: int = 64):
        self.engine = engine
        self.slots = [_Slot() for _ in range(slots)]
        self.depth = depth
        self.minimum_batch = speculative_minimum_batch
        self.chunk_tokens = chunk_tokens
        self.clock = 0
        self.metrics = {"speculative_cycles": 0, "proposed_tokens": 0, "accepted_tokens": 0,
                        "first_token_rejections": 0, "prefix_tokens_reused": 0, "kv_clones": 0,
                        "prefill_tokens": 0, "decode_steps": 0,
                        "stale_prefix_fallbacks": 0}

    # admit_one (native_runtime_main.cpp:342-413) for a placement the router already chose.
    def admit(self, request: Request, destination: int, source: Optional[int],
              prefix_tokens: int) -> None:
        slot = self.slots[destination]
        if slot.request is not None:
            raise RuntimeError("destination slot is occupied")
        self.clock += 1
        slot.request, slot.output_ids, slot.decode_ready = request, [], False
        slot.inherited_token = None
        slot.prompt_array = None
        slot.age, slot.dirty = self.clock, True
        # The router decided on its mirror of the table; a source that was decoding has moved on
        # since (its cache only grows while occupied), and a ring cannot be wound back, so a
        # stale prefix is not reused: the request prefills from an empty slot instead.
        if source is not None and len(self.slots[source].cached_tokens) != prefix_tokens:
            self.metrics["stale_prefix_fallbacks"] += 1
            source = None
        if source is None:
            self.engine.reset_slot(destination)
            slot.cached_tokens, slot.reported = [], 0
            return
        if source != destination:
            self.engine.clone_slot(source, destination)
            slot.cached_tokens, slot.reported = list(self.slots[source].cached_tokens), 0
            self.metrics["kv_clones"] += 1
        self.metrics["prefix_tokens_reused"] += prefix_tokens
        if prefix_tokens == len(request.input_ids):
            slot.inherited_token = self.slots[source].token_to_append

    def _start_decode(self, index: int, first_token: int) -> List[int]:
        slot = self.slots[index]
        slot.prompt_array = None
        slot.token_to_append, slot.decode_ready = first_token, True
        slot.output_ids.append(first_token)
        slot.dirty = True
        return [first_token]

    def _finish_if_done(self, index: int, stopped: bool, finished: list) -> None:
        slot = self.slots[index]
        if (stopped or slot.token_to_append in slot.request.stop_ids
                or len(slot.output_ids) >= slot.request.max_tokens):
            finished.append(slot.request.request_id)
            self.clock += 1
            slot.request, slot.decode_ready, slot.age, slot.dirty = None, False, self.clock, True

    def tick(self):
        """One pass: one prefill quantum for every slot whose prompt is not resident yet (all of
        them in one batched call, like the reference's idle_prefill_batch,
        src/native_runtime_main.cpp:421-478), then one decode step over the decode-ready slots.
        Returns ({request id: tokens emitted this tick}, [request ids finished])."""
        emitted: Dict[int, List[int]] = {}
        finished: List[int] = []
        prefilling = []
        for index, slot in enumerate(self.slots):
            if slot.request is None or slot.decode_ready:
                continue
            if slot.inherited_token is not None:
                first, slot.inherited_token = slot.inherited_token, None
                emitted.setdefault(slot.request.request_id, []).extend(
                    self._start_decode(index, first))
                self._finish_if_done(index, False, finished)
            else:
                prefilling.append(index)
        if prefilling:
            # The prompt goes to the engine once per quantum; convert it to a C array once.
            for index in prefilling:
                slot = self.slots[index]
                if slot.prompt_array is None:
                    slot.prompt_array = capi.int_array(slot.request.input_ids)
            prompts = [self.slots[index].prompt_array for index in prefilling]
            firsts = self.engine.prefill_slots_chunks(prefilling, prompts, self.chunk_tokens)
            for index, first in zip(prefilling, firsts):
                slot = self.slots[index]
                resident = self.engine.slot_position(index)
                self.metrics["prefill_tokens"] += resident - len(slot.cached_tokens)
                slot.cached_tokens = list(slot.request.input_ids[:resident])
                slot.dirty = True
                if first is not None:
                    emitted.setdefault(slot.request.request_id, []).extend(
                        self._start_decode(index, first))
                    self._finish_if_done(index, False, finished)
        batch = [index for index, slot in enumerate(self.slots)
                 if slot.request is not None and slot.decode_ready]
        if batch:
            self.metrics["decode_steps"] += 1
            if self.engine.has_assistant() and len(batch) >= self.minimum_batch:
                self._speculative_decode(batch, emitted, finished)
            else:
                self._decode_step(batch, emitted, finished)
        return emitted, finished

    # decode_step: one token per slot through append_ragged.
    def _decode_step(self, batch, emitted, finished) -> None:
        tokens = [self.slots[index].token_to_append for index in batch]
        following = self.engine.append_ragged(tokens, batch)
        for index, token, next_token in zip(batch, tokens, following):
            slot = self.slots[index]
            slot.cached_tokens.append(token)
            slot.token_to_append = next_token
            slot.output_ids.append(next_token)
            slot.dirty = True
            emitted.setdefault(slot.request.request_id, []).append(next_token)
            self._finish_if_done(index, False, finished)

    # speculative_decode (native_runtime_main.cpp:583-678).
    def _speculative_decode(self, batch, emitted, finished) -> None:
        batch = sorted(batch, key=lambda index: (self.engine.slot_position(index), index))
        last_tokens = [self.slots[index].cached_tokens[-1] for index in batch]
        target_first = [self.slots[index].token_to_append for index in batch]
        proposals = self.engine.draft_four(last_tokens, batch, target_first, self.depth)
        caps = []
        for row, index in enumerate(batch):
            slot = self.slots[index]
            remaining = slot.request.max_tokens - len(slot.output_ids)
            caps.append(acceptance_cap(self.depth, remaining, proposals[row],
                                       slot.request.stop_ids))
        verification = self.engine.verify_greedy_proposals(proposals, target_first, batch, caps)
        self.metrics["speculative_cycles"] += 1
        self.metrics["proposed_tokens"] += self.depth * len(batch)
        self.metrics["accepted_tokens"] += sum(verification.accepted_tokens)
        rejected = [row for row, accepted in enumerate(verification.accepted_tokens)
                    if accepted == 0]
        self.metrics["first_token_rejections"] += len(rejected)
        fallback = {}
        if rejected:
            following = self.engine.append_ragged([target_first[row] for row in rejected],
                                                  [batch[row] for row in rejected])
            fallback = dict(zip(rejected, following))
        for row, index in enumerate(batch):
            slot = self.slots[index]
            accepted = verification.accepted_tokens[row]
            drafts = proposals[row][1:accepted] if accepted > 1 else []
            next_token = fallback[row] if accepted == 0 else verification.next_tokens[row]
            resident, shown, following, stopped = commit_speculation(
                slot.token_to_append, drafts, next_token, slot.request.stop_ids)
            slot.cached_tokens.extend(resident)
            slot.output_ids.extend(shown)
            slot.token_to_append = following
            slot.dirty = True
            emitted.setdefault(slot.request.request_id, []).extend(shown)
            self._finish_if_done(index, stopped, finished)

    def changes(self) -> List[tuple]:
        """Slot-table changes since the last call, in Router.apply_report's form."""
        out = []
        for index, slot in enumerate(self.slots):
            if not slot.dirty:
                continue
            keep = min(slot.reported, len(slot.cached_tokens))
            out.append((index, keep, slot.cached_tokens[keep:], slot.request is not None,
                        slot.age, slot.request is not None and not slot.decode_ready))
            slot.reported, slot.dirty = len(slot.cached_tokens), False
        return out

    def idle(self) -> bool:
        return all(slot.request is None for slot in self.slots)


# ---------------------------------------------------------------------------------------------
# Messages.

class LocalChannel:
    """Ordered topics inside one process."""

    def __init__(self):
        self.topics: Dict[str, list] = {}
        self.cursor: Dict[Tuple[int, str], int] = {}

    def send(self, topic: str, message) -> None:
        self.topics.setdefault(topic, []).append(message)

    def receive(self, reader: int, topic: str) -> list:
        messages = self.topics.get(topic, [])
        start = self.cursor.get((reader, topic), 0)
        self.cursor[(reader, topic)] = len(messages)
        return messages[start:]


class StoreChannel:
    """Ordered topics over a torch.distributed store shared by the router's and the replicas'
    processes. A topic has one writer; it numbers its messages with the store's atomic counter and
    readers fetch the numbers they have not seen."""

    def __init__(self, store):
        self.store = store
        self.cursor: Dict[str, int] = {}

    def send(self, topic: str, message) -> None:
        number = self.store.add(f"{topic}/sent", 1)
        self.store.set(f"{topic}/{number}", pickle.dumps(message))
        self.store.add(f"{topic}/ready", 1)

    def receive(self, reader: int, topic: str) -> list:
        ready = self.store.add(f"{topic}/ready", 0)
        start = self.cursor.get(topic, 0)
        # "ready" counts completed writes; with one writer per topic they complete in order.
        messages = [pickle.loads(self.store.get(f"{topic}/{number}"))
                    for number in range(start + 1, ready + 1)]
        self.cursor[topic] = ready
        return messages


def commands_topic(replica: int) -> str:
    return f"carat/commands/{replica}"


def reports_topic(replica: int) -> str:
    return f"carat/reports/{replica}"


class ReplicaWorker:
    """A replica's loop: take the router's commands, run one scheduler tick, report."""

    def __init__(self, channel, replica: int, scheduler: ReplicaScheduler):
        self.channel, self.replica, self.scheduler = channel, replica, scheduler
        self.ticks = 0
        self.stopped = False

    def step(self) -> None:
        for command in self.channel.receive(self.replica, commands_topic(self.replica)):
            if command[0] == "admit":
                _, request, destination, source, prefix = command
                self.scheduler.admit(request, destination, source, prefix)
            elif command[0] == "stop":
                self.stopped = True
        emitted, finished = ({}, []) if self.scheduler.idle() else self.scheduler.tick()
        self.ticks += 1
        self.channel.send(reports_topic(self.replica),
                          {"tick": self.ticks, "emitted": emitted, "finished": finished,
                           "changes": self.scheduler.changes(),
                           "metrics": dict(self.scheduler.metrics), "bye": self.stopped})

    def run(self, idle_sleep: float = 0.002, leave_after_ticks: Optional[int] = None) -> None:
        """Until the router says stop. `leave_after_ticks` makes the replica go away between two
        steps without a word, the way a lost host or a killed process does."""
        while not self.stopped:
            if leave_after_ticks is not None and self.ticks >= leave_after_ticks:
                return
            self.step()
            if self.scheduler.idle():
                time.sleep(idle_sleep)


class Dispatcher:
    """The box-level front: queue, route, follow the replicas' reports, survive a lost replica."""

    def __init__(self, channel, replica_count: int, slots_per_replica: int,
                 idle_cache_reserve_slots: int = 0, report_timeout: float = 5.0):
        self.channel = channel
        self.router = Router(replica_count, slots_per_replica, idle_cache_reserve_slots)
        self.pending: List[Request] = []
        self.assigned: Dict[int, Tuple[int, Request]] = {}      # request id -> (replica, request)
        self.origin: Dict[int, Request] = {}
        self.outputs: Dict[int, List[int]] = {}
        self.completed: Dict[int, List[int]] = {}
        self.placements: Dict[int, List[Placement]] = {}
        self.metrics = [dict() for _ in range(replica_count)]
        self.report_timeout = report_timeout
        self.last_report = [time.monotonic()] * replica_count
        self.lost: List[int] = []

    def submit(self, request: Request) -> None:
        if not request.input_ids or request.max_tokens <= 0:
            raise ValueError("a request needs input tokens and a positive token budget")
        self.origin[request.request_id] = request
        self.outputs[request.request_id] = []
        self.pending.append(request)

    def poll(self) -> None:
        """One round: read reports, retire lost replicas, route what can be routed."""
        now = time.monotonic()
        for replica in range(len(self.router.tables)):
            if not self.router.alive[replica]:
                continue
            reports = self.channel.receive(-1, reports_topic(replica))
            for report in reports:
                self._apply(replica, report)
            if reports:
                self.last_report[replica] = now
            elif now - self.last_report[replica] > self.report_timeout:
                self._retire(replica)
        waiting: List[Request] = []
        for request in self.pending:
            placement = self.router.route(request.input_ids)
            if not isinstance(placement, Placement):
                waiting.append(request)
                continue
            self.router.reserve_slot(placement, request.input_ids)
            self.assigned[request.request_id] = (placement.replica, request)
            self.placements.setdefault(request.request_id, []).append(placement)
            self.channel.send(commands_topic(placement.replica),
                              ("admit", request, placement.destination, placement.source,
                               placement.prefix_tokens))
        self.pending = waiting

    def _apply(self, replica: int, report) -> None:
        self.router.apply_report(replica, report["changes"])
        self.metrics[replica] = report["metrics"]
        for request_id, tokens in report["emitted"].items():
            if self.assigned.get(request_id, (None,))[0] == replica:
                self.outputs[request_id].extend(tokens)
        for request_id in report["finished"]:
            if self.assigned.get(request_id, (None,))[0] == replica:
                del self.assigned[request_id]
                self.completed[request_id] = self.outputs[request_id]

    def _retire(self, replica: int) -> None:
        """The replica stopped reporting: nothing of it is trusted any more. Its requests go back
        to the queue as continuations (prompt + what was already emitted); greedy decoding makes
        the continuation the same stream."""
        self.router.mark_left(replica)
        self.lost.append(replica)
        for request_id, (owner, _) in list(self.assigned.items()):
            if owner != replica:
                continue
            del self.assigned[request_id]
            origin = self.origin[request_id]
            done = self.outputs[request_id]
            if len(done) >= origin.max_tokens or (done and done[-1] in origin.stop_ids):
                self.completed[request_id] = done
                continue
            self.pending.insert(0, Request(request_id, origin.input_ids + done,
                                           origin.max_tokens - len(done), origin.stop_ids))

    def finished(self) -> bool:
        return not self.pending and not self.assigned

    def stop_replicas(self) -> None:
        for replica, alive in enumerate(self.router.alive):
            if alive:
                self.channel.send(commands_topic(replica), ("stop",))

    def aggregate_metrics(self) -> Dict[str, int]:
        total: Dict[str, int] = {}
        for metrics in self.metrics:
            for name, value in metrics.items():
                total[name] = total.get(name, 0) + value
        return total
