#!/usr/bin/env python3
"""Benchmark of the speculative-decoding step on Gemma-4-31B shapes (random-init FP8 weights).

One step = draft (k proposals per slot) + one batched (k+1)-row FP8 verify forward over all slots
+ fused LM-head argmax, greedy prefix-accept and KV commit. Per-step accept lengths are injected
from a seeded geometric distribution (mean 2.5) through the acceptance caps, because random-init
weights never agree with a random-init drafter; the work per step does not depend on them.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N > 1 is launched by torchrun: every rank runs an independent full-model replica on its own GPU
(no data-path collective); the printed value is the sum over replicas divided by the slowest
replica's time.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import subprocess
import sys
import tempfile
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "Gemma-4-31B FP8 spec-decode tokens/s/GPU (24 slots); verify-step HBM GB/s"
UNIT = "tokens/s"
SLOTS = 24
DRAFTS = 4                 # k
DEPTH = DRAFTS + 1         # verify rows per slot: the forced token + k drafts
MAX_CONTEXT = 8192
MEAN_ACCEPT = 2.5


def workload_config(args):
    return {
        "workload": "configs[3] on one replica: 24 slots x 8192-token context, FP8 31B-shaped "
                    f"target + 4-layer 1024-wide FP8 drafter, k={DRAFTS} ({DEPTH} verify rows per slot), "
                    "context lengths uniform in [128, 6144] (seeded), KV caches filled with seeded "
                    "random bf16 rows, accept lengths injected from a seeded geometric distribution "
                    "with mean 2.5; a static snapshot of the request mix (no arrivals, prefill or "
                    "slot turnover inside the timed region)",
        "slots": SLOTS, "drafts": DRAFTS, "verify_rows": SLOTS * DEPTH,
        "max_context": MAX_CONTEXT, "parallelism": f"replicas x{args.gpus}",
        "l2": "inputs (30.7 GB of weights + KV per step) exceed the 126 MB L2",
    }


def accept_lengths(steps, seed):
    generator = torch.Generator().manual_seed(seed)
    p = 1.0 / MEAN_ACCEPT
    uniform = torch.rand(steps, SLOTS, generator=generator).clamp_min(1e-9)
    lengths = torch.floor(torch.log(uniform) / math.log(1.0 - p)).to(torch.int64) + 1
    return lengths.clamp(1, DEPTH)


def context_lengths(seed):
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(128, 6145, (SLOTS,), generator=generator).tolist()


def rank_workload(steps, rank, same_seeds=False):
    """Context lengths and per-step accept lengths of one replica. Weak scaling keeps the work per
    GPU fixed, so every replica gets the multiset of the single-GPU run (the same KV bytes, the
    same number of accepted tokens in every step) dealt to its slots in an order of its own;
    `same_seeds` gives every replica the very same assignment."""
    contexts = context_lengths(seed=3)
    lengths = accept_lengths(steps, seed=7)
    if rank == 0 or same_seeds:
        return contexts, lengths
    generator = torch.Generator().manual_seed(1000 + rank)
    order = torch.randperm(SLOTS, generator=generator).tolist()
    contexts = [contexts[index] for index in order]
    shuffled = torch.stack([row[torch.randperm(SLOTS, generator=generator)] for row in lengths])
    return contexts, shuffled


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """SM clock and throttle reasons while the timed region runs. NVML is read from a thread of
    this process every 10 ms (a sample is there within milliseconds, also when eight ranks start
    at once); where the NVML binding is missing, `nvidia-smi -lms 200` runs beside the bench, which
    needs a region of a second or more to see anything. Nothing is ever set, only read."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40),
                   ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, device_index):
        self.device_index = device_index
        self.process = None
        self.path = None
        self.thread = None
        self.stop_flag = None
        self.samples = []          # (sm MHz, reason bit mask)
        self.maximum = None

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(self.device_index).uuid)
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.device_index)

    def _sample_loop(self, pynvml, handle):
        while not self.stop_flag.is_set():
            try:
                clock = pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
                mask = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.samples.append((float(clock), int(mask)))
            except Exception:
                pass
            self.stop_flag.wait(0.01)

    def start(self):
        try:
            import threading
            pynvml, handle = self._nvml_handle()
            self.maximum = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            self.stop_flag = threading.Event()
            self.thread = threading.Thread(target=self._sample_loop, args=(pynvml, handle),
                                           daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            handle = tempfile.NamedTemporaryFile(prefix="clocks", suffix=".csv", delete=False)
            self.path = handle.name
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.device_index)], stdout=handle,
                stderr=subprocess.DEVNULL)
        except OSError:
            self.process = None

    def stop(self):
        result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        clocks, reasons, maximum = [], set(), None
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            maximum = self.maximum
            for clock, mask in self.samples:
                clocks.append(clock)
                for name, bit in self.REASON_BITS:
                    if mask & bit:
                        reasons.add(name)
            result["source"] = "nvml, 10 ms"
        elif self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()
            try:
                for line in open(self.path):
                    fields = [field.strip() for field in line.split(",")]
                    if len(fields) < 9:
                        continue
                    try:
                        clocks.append(float(fields[1]))
                        maximum = float(fields[2])
                    except ValueError:
                        continue
                    for name, value in zip(("hw_slowdown", "hw_thermal_slowdown",
                                            "sw_thermal_slowdown", "sw_power_cap"), fields[5:9]):
                        if value.lower().startswith("active"):
                            reasons.add(name)
                os.unlink(self.path)
            except OSError:
                pass
            result["source"] = "nvidia-smi, 200 ms"
        if clocks:
            clocks.sort()
            busy = clocks[len(clocks) // 2:]   # upper half: samples taken under load
            result["sm_mhz"] = busy[len(busy) // 2]
            result["sm_max_mhz"] = maximum
            result["reasons"] = sorted(reasons)
            result["samples"] = len(clocks)
        return result


# --------------------------------------------------------------------------- model construction
def random_fp8_segment(arena_fp8, name, rows, cols, generator, std, keep_bf16=None):
    import carat_b200
    values = torch.empty(rows, cols, dtype=torch.bfloat16, device="cuda")
    step = max(1, (64 << 20) // cols)
    for start in range(0, rows, step):
        stop = min(rows, start + step)
        values[start:stop] = (torch.randn(stop - start, cols, device="cuda", generator=generator)
                              * std).to(torch.bfloat16)
    fp8_bytes, scale = carat_b200.quantize_tensor_to_fp8(values)
    arena_fp8.add(name, fp8_bytes, scale)
    if keep_bf16 is not None:
        keep_bf16[name] = values


def build_model(seed):
    """Random-init 31B-shaped target and the reference-shaped drafter, quantised to e4m3 on the
    device segment by segment (N(0, 0.02) matrices, unit norm weights and layer scalars)."""
    import carat_b200
    config = carat_b200.Gemma4Config.gemma4_31b()
    assistant_config = carat_b200.Gemma4AssistantConfig()
    generator = torch.Generator(device="cuda").manual_seed(seed)
    bf16 = {}
    fp8 = carat_b200.Fp8WeightArena()
    hidden, inter = config.hidden_size, config.intermediate_size

    def ones(n):
        return torch.ones(n, dtype=torch.bfloat16, device="cuda")

    random_fp8_segment(fp8, "token_embedding", config.vocabulary_size, hidden, generator, 0.02, bf16)
    for index, layer in enumerate(config.layers):
        prefix = f"layer.{index}."
        for name, width in (("input_norm", hidden), ("q_norm", layer.head_dimension),
                            ("k_norm", layer.head_dimension), ("post_attention_norm", hidden),
                            ("pre_mlp_norm", hidden), ("post_mlp_norm", hidden), ("scalar", 1)):
            bf16[prefix + name] = ones(width)
        random_fp8_segment(fp8, prefix + "qkv", layer.packed_width(), hidden, generator, 0.02)
        random_fp8_segment(fp8, prefix + "o", hidden, layer.query_width(), generator, 0.02)
        random_fp8_segment(fp8, prefix + "gate_up", 2 * inter, hidden, generator, 0.02)
        random_fp8_segment(fp8, prefix + "down", hidden, inter, generator, 0.02)
    bf16["final_norm"] = ones(hidden)
    weights = carat_b200.DeviceWeightArena(bf16)

    a_generator = torch.Generator(device="cuda").manual_seed(seed + 1)
    a_bf16 = {}
    a_fp8 = carat_b200.Fp8WeightArena()
    a_hidden, a_inter = assistant_config.hidden_size, assistant_config.intermediate_size
    random_fp8_segment(a_fp8, "token_embedding", config.vocabulary_size, a_hidden, a_generator, 0.02)
    random_fp8_segment(a_fp8, "pre_projection", a_hidden, 2 * hidden, a_generator, 0.02)
    random_fp8_segment(a_fp8, "post_projection", hidden, a_hidden, a_generator, 0.02)
    for index, kind in enumerate(assistant_config.layers):
        prefix = f"layer.{index}."
        head_dim = 512 if kind == "global" else 256
        query = assistant_config.query_heads * head_dim
        for name, width in (("input_norm", a_hidden), ("q_norm", head_dim),
                            ("post_attention_norm", a_hidden), ("pre_mlp_norm", a_hidden),
                            ("post_mlp_norm", a_hidden), ("scalar", 1)):
            a_bf16[prefix + name] = ones(width)
        random_fp8_segment(a_fp8, prefix + "q", query, a_hidden, a_generator, 0.02)
        random_fp8_segment(a_fp8, prefix + "o", a_hidden, query, a_generator, 0.02)
        random_fp8_segment(a_fp8, prefix + "gate_up", 2 * a_inter, a_hidden, a_generator, 0.02)
        random_fp8_segment(a_fp8, prefix + "down", a_hidden, a_inter, a_generator, 0.02)
    a_bf16["final_norm"] = ones(a_hidden)
    a_weights = carat_b200.DeviceWeightArena(a_bf16)
    torch.cuda.synchronize()
    runner = carat_b200.Gemma4BatchModelRunner(config, weights, SLOTS, MAX_CONTEXT, fp8, a_weights,
                                               a_fp8, assistant_config, assistant_fp8_mode="all")
    return config, runner, fp8


def fill_kv(runner, config, seed):
    """Seeded random bf16 rows in every K and V cache (unit variance, like normalised keys and
    values): the step's work does not depend on the values, but power and clocks under real data
    are not those of a zero-filled cache."""
    generator = torch.Generator(device="cuda").manual_seed(seed)
    for index, layer in enumerate(config.layers):
        capacity = config.sliding_window if layer.attention == "sliding" else MAX_CONTEXT
        shape = (SLOTS, layer.kv_heads, capacity, layer.head_dimension)
        for which in (0, 1):
            values = torch.randn(shape, device="cuda", generator=generator, dtype=torch.bfloat16)
            runner.write_cache(which, index, values)
            del values
    torch.cuda.synchronize()


# --------------------------------------------------------------------------- byte accounting
def linear_bytes(rows, k, n, fused_argmax=False):
    """Algorithmic bytes of one FP8 linear call: e4m3 weights + e4m3 activations in + bf16 out
    (+ two fp32 scales); the fused LM head writes 8 bytes per row instead of logits."""
    return k * n + rows * k + (rows * 8 if fused_argmax else 2 * rows * n) + 8


def step_weight_bytes(config):
    total = 0
    for layer in config.layers:
        h, i = config.hidden_size, config.intermediate_size
        total += layer.packed_width() * h + h * layer.query_width() + 2 * i * h + h * i
    return total + config.vocabulary_size * config.hidden_size


def step_kv_bytes(config, positions):
    """Every resident K and V row read once: 2 B x (K + V) x kv width x visible rows."""
    total = 0
    for layer in config.layers:
        per_row = 2 * 2 * layer.kv_width()
        for position in positions:
            rows = position + DEPTH
            if layer.attention == "sliding":
                rows = min(rows, config.sliding_window)
            total += per_row * rows
    return total


# --------------------------------------------------------------------------- our arm
def run_ours(args, rank, world):
    import carat_b200
    library = carat_b200.library()
    config, runner, fp8 = build_model(seed=0)
    seed_shift = 0 if args.same_seeds else rank
    start_positions, lengths = rank_workload(args.steps + args.warmup, rank, args.same_seeds)
    generator = torch.Generator().manual_seed(11 + seed_shift)
    slots = list(range(SLOTS))

    def reseed():
        runner.seed_slot_positions(start_positions)
        fill_kv(runner, config, seed=5 + seed_shift)

    reseed()
    last_tokens = torch.randint(3, config.vocabulary_size, (SLOTS,), generator=generator).tolist()
    next_tokens = torch.randint(3, config.vocabulary_size, (SLOTS,), generator=generator).tolist()

    def one_step(step):
        nonlocal last_tokens, next_tokens
        if any(runner.slot_position(slot) + DEPTH > MAX_CONTEXT for slot in slots):
            reseed()
        proposals = runner.draft_four(last_tokens, slots, next_tokens, DEPTH)
        caps = lengths[step].tolist()
        result = runner.verify_greedy_proposals(proposals, next_tokens, slots, caps,
                                                carat_b200.VERIFY_ASSUME_MATCH)
        verify_ms, draft_ms = runner.last_device_ms()
        verify_launches, draft_launches = runner.last_launches()
        last_tokens = [proposals[r][result.accepted_tokens[r] - 1] for r in range(SLOTS)]
        next_tokens = result.next_tokens
        return result.accepted_tokens, verify_ms, draft_ms, verify_launches + draft_launches

    def timed_run():
        for step in range(args.warmup):
            one_step(step)
        barrier(world)
        torch.cuda.synchronize()
        sampler = ClockSampler(torch.cuda.current_device())
        sampler.start()
        positions = [runner.slot_position(slot) for slot in slots]
        tokens = 0
        device_ms = 0.0
        verify_total_ms = 0.0
        launches = 0
        token_gaps = []      # per slot and step: step time / tokens the slot emitted in it
        wall_start = time.perf_counter()
        for step in range(args.warmup, args.warmup + args.steps):
            accepted, verify_ms, draft_ms, step_launches = one_step(step)
            tokens += sum(accepted)
            device_ms += verify_ms + draft_ms
            verify_total_ms += verify_ms
            launches += step_launches
            token_gaps += [(verify_ms + draft_ms) / count for count in accepted if count > 0]
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - wall_start) * 1e3
        clocks = sampler.stop()
        barrier(world)
        return positions, tokens, device_ms, verify_total_ms, launches, wall_ms, clocks, token_gaps

    (positions_at_start, tokens, device_ms, verify_total_ms, launches, wall_ms, clocks,
     token_gaps) = timed_run()

    totals = reduce_max_and_sum(world, [device_ms, wall_ms], [float(tokens)])
    device_ms_max, wall_ms_max = totals[0]
    tokens_all = totals[1][0]
    weight_bytes = step_weight_bytes(config)
    kv_bytes = step_kv_bytes(config, positions_at_start)
    per_rank = gather_rows(world, [float(rank), device_ms / args.steps,
                                   verify_total_ms / args.steps, float(kv_bytes), float(tokens),
                                   (wall_ms - device_ms) / args.steps])
    if rank != 0:
        return
    peaks = measured_peaks()
    verify_ms_step = verify_total_ms / args.steps
    token_gaps.sort()
    line = {
        "metric": METRIC, "value": tokens_all / (device_ms_max / 1e3), "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": device_ms_max / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate, bf16 activations)",
        "data": "synthetic", "config": workload_config(args), "clocks": clocks,
        "e2e": {"value": tokens_all / (wall_ms_max / 1e3), "unit": UNIT,
                "h2d_bytes_per_step": 4 * (256 + 4 * SLOTS) + 4 * 4 * SLOTS,
                "d2h_bytes_per_step": 4 * (2 * SLOTS + 256 + 1) + 4 * (DEPTH * SLOTS + 1)},
        "gpu_launches": launches,
        "verify_step": {
            "ms": verify_ms_step, "weight_bytes": weight_bytes, "kv_bytes": kv_bytes,
            "hbm_gbs": (weight_bytes + kv_bytes) / verify_ms_step / 1e6,
            "frac_of_measured_peak": (weight_bytes + kv_bytes) / verify_ms_step / 1e6 / peaks["hbm_gbs"],
            "frac_of_nominal_8000": (weight_bytes + kv_bytes) / verify_ms_step / 1e6 / 8000.0},
        "mean_accepted": tokens / args.steps / SLOTS,
        "inter_token_ms_p50": token_gaps[len(token_gaps) // 2] if token_gaps else None,
        # Replicas never wait for one another, so the box's throughput is also the plain sum of
        # what each replica does in its own time; `value` divides by the slowest replica's time.
        "value_independent": sum(row[4] / (row[1] * args.steps / 1e3) for row in per_rank),
        "per_rank": [{"rank": int(row[0]), "ms_per_step": row[1], "verify_ms": row[2],
                      "kv_bytes": int(row[3]), "tokens": int(row[4]),
                      "host_ms_per_step_beyond_device": row[5]} for row in per_rank],
        "same_seeds_on_every_rank": bool(args.same_seeds),
    }
    line["near_ties"] = near_tie_count(runner)
    line["plain_decode"] = plain_decode(runner, config, slots, args)
    line["roofline"] = linear_roofline(library, config, fp8, peaks)
    if world == 1 and not args.skip_int4:
        line["int4_mlp"] = int4_variant(config, runner, timed_run, args, weight_bytes)
    if world == 1 and not args.skip_cpu:
        line["library_baseline"] = library_baseline(config, fp8, peaks)
        line["cpu_baseline"] = cpu_sample(config, lengths, kind_only=False)
    print(json.dumps(line), flush=True)


def near_tie_count(runner):
    """Top-2 margins of the last verify call's logits (recomputed outside the timed region; the
    step itself never stores logits): rows whose argmax a logit change within the path's
    tolerance could flip."""
    rows = SLOTS * DEPTH
    logits = runner.last_logits(rows).float()
    top2 = logits.topk(2, dim=1).values
    margin = top2[:, 0] - top2[:, 1]
    return {"rows": rows, "margin_below_1e-2": int((margin < 1e-2).sum()),
            "margin_within_relative_2e-2": int((margin <= 2e-2 * top2[:, 0].abs()).sum())}


def plain_decode(runner, config, slots, args):
    """append_ragged, one token per slot over all 24 slots: the step the scheduler falls back to
    below its speculation threshold (the same kernels at 24 rows)."""
    generator = torch.Generator().manual_seed(23)
    tokens = torch.randint(3, config.vocabulary_size, (SLOTS,), generator=generator).tolist()
    for _ in range(args.warmup):
        tokens = runner.append_ragged(tokens, slots)
    device_ms = 0.0
    launches = 0
    steps = max(3, args.steps // 2)
    begin = time.perf_counter()
    for _ in range(steps):
        tokens = runner.append_ragged(tokens, slots)
        device_ms += runner.last_device_ms()[0]
        launches = runner.last_launches()[0]
    wall_ms = (time.perf_counter() - begin) * 1e3
    return {"rows": SLOTS, "steps": steps, "ms_per_step": device_ms / steps,
            "tokens_per_s": SLOTS * steps / (device_ms / 1e3),
            "e2e_tokens_per_s": SLOTS * steps / (wall_ms / 1e3), "launches_per_step": launches}


def int4_variant(config, runner, timed_run, args, fp8_weight_bytes):
    """The same timed loop with the target's gate_up / down as INT4 weight-only linears (groups of
    128, bf16 activations): random codes and a constant scale stand in for quantised weights, the
    work per step does not depend on the values."""
    from carat_b200 import capi
    try:
        hidden, inter = config.hidden_size, config.intermediate_size
        group = 128
        generator = torch.Generator(device="cuda").manual_seed(5)
        layers = (capi.Int4MlpLayer * len(config.layers))()
        keep = []
        up_scales = torch.full((hidden // group, 2 * inter), 0.006, dtype=torch.bfloat16,
                               device="cuda")
        down_scales = torch.full((inter // group, hidden), 0.006, dtype=torch.bfloat16,
                                 device="cuda")
        for index in range(len(config.layers)):
            up = torch.randint(0, 256, (2 * inter, hidden // 2), dtype=torch.uint8, device="cuda",
                               generator=generator)
            down = torch.randint(0, 256, (hidden, inter // 2), dtype=torch.uint8, device="cuda",
                                 generator=generator)
            keep += [up, down]
            layers[index].gate_up_codes = up.data_ptr()
            layers[index].gate_up_scales = up_scales.data_ptr()
            layers[index].down_codes = down.data_ptr()
            layers[index].down_scales = down_scales.data_ptr()
        torch.cuda.synchronize()
        capi.check(capi.library().carat_b200_runner_use_int4_mlp(runner._handle, layers,
                                                                 len(layers), group))
        _, tokens, device_ms, verify_total_ms, launches, wall_ms, _, _ = timed_run()
        capi.check(capi.library().carat_b200_runner_use_int4_mlp(runner._handle, None, 0, 0))
        mlp_e4m3 = len(config.layers) * 3 * inter * hidden
        mlp_int4 = len(config.layers) * (3 * inter * hidden // 2 + 3 * inter * hidden // group * 2)
        return {"value": tokens / (device_ms / 1e3), "unit": UNIT,
                "e2e": tokens / (wall_ms / 1e3), "ms_per_step": device_ms / args.steps,
                "verify_ms": verify_total_ms / args.steps, "gpu_launches": launches,
                "group_width": group,
                "weight_bytes": fp8_weight_bytes - mlp_e4m3 + mlp_int4}
    except Exception as error:  # the e4m3 numbers of the line stand on their own
        capi.library().carat_b200_runner_use_int4_mlp(runner._handle, None, 0, 0)
        return {"error": str(error)}


# dram__bytes_read.sum + dram__bytes_write.sum of the captured gate_up launch
# (profiles/fp8_linear_gate_up_120x5376x43008.md, capture of 2026-11-25) and that launch's
# algorithmic bytes: weights + activations + bf16 output + two scales.
NCU_GATE_UP_DRAM_BYTES = 231.931904e6 + 6.040832e6
NCU_GATE_UP_ALGORITHMIC_BYTES = 231211008 + 645120 + 10321920 + 8


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        data = json.load(open(path))
        return {"hbm_gbs": float(data["hbm_gbs"]), "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": 6650.0, "source": "fallback (no MEASURED_PEAKS.json)"}


def linear_roofline(library, config, fp8, peaks):
    """The dominant kernel is the FP8 weight-streaming linear. Times every target linear of one
    verify step (60 layers x 4 + the fused LM head, 241 launches over 30.7 GB of distinct weights,
    so every launch starts with a cold L2) back to back with CUDA events on the launching stream
    and reports algorithmic bytes / time."""
    from carat_b200.capi import check
    rows = SLOTS * DEPTH
    hidden, inter = config.hidden_size, config.intermediate_size
    widest = max(inter, max(layer.query_width() for layer in config.layers))
    x = torch.randint(0, 120, (rows, widest), dtype=torch.uint8, device="cuda")
    scale = torch.ones(1, dtype=torch.float32, device="cuda")
    out = torch.empty(rows, 2 * inter, dtype=torch.bfloat16, device="cuda")
    work = torch.empty(64 << 20, dtype=torch.uint8, device="cuda")
    tokens = torch.empty(rows, dtype=torch.int32, device="cuda")
    keys = torch.empty(rows, dtype=torch.int64, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    calls = []
    for index, layer in enumerate(config.layers):
        prefix = f"layer.{index}."
        calls += [(prefix + "qkv", hidden, layer.packed_width()),
                  (prefix + "o", layer.query_width(), hidden),
                  (prefix + "gate_up", hidden, 2 * inter), (prefix + "down", inter, hidden)]

    def sweep():
        for name, k, n in calls:
            check(library.carat_b200_fp8_linear(
                x.data_ptr(), scale.data_ptr(), fp8.at(name).data_ptr(), fp8.scale(name).data_ptr(),
                out.data_ptr(), rows, k, n, work.data_ptr(), work.numel(), stream))
        check(library.carat_b200_fp8_linear_argmax(
            x.data_ptr(), scale.data_ptr(), fp8.at("token_embedding").data_ptr(),
            fp8.scale("token_embedding").data_ptr(), tokens.data_ptr(), keys.data_ptr(), rows,
            hidden, config.vocabulary_size, stream))

    sweep()
    torch.cuda.synchronize()
    times = []
    for _ in range(3):
        begin = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        begin.record()
        sweep()
        end.record()
        torch.cuda.synchronize()
        times.append(begin.elapsed_time(end))
    elapsed_ms = sorted(times)[1]
    total = sum(linear_bytes(rows, k, n) for _, k, n in calls)
    total += linear_bytes(rows, hidden, config.vocabulary_size, fused_argmax=True)
    launches = len(calls) + 1
    achieved = total / elapsed_ms / 1e6
    return {"bound": "hbm", "kernel": "fp8_linear_kernel (all 241 target linears of one verify step)",
            "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
            "bytes_per_launch": total / launches, "ms_per_launch": elapsed_ms / launches,
            # DRAM bytes per launch. One ncu capture of the 120 x 5376 -> 43008 launch
            # (profiles/fp8_linear_gate_up_120x5376x43008.md) read 231.91 MB and wrote 6.53 MB
            # against 242.18 MB algorithmic (part of the bf16 output was still in L2 when the
            # counters stopped); every weight byte is read exactly once whatever the shape, so the
            # figure is scaled to the sweep's mean launch by algorithmic bytes.
            "traffic": total / launches * NCU_GATE_UP_DRAM_BYTES / NCU_GATE_UP_ALGORITHMIC_BYTES,
            "traffic_source": "profiles/fp8_linear_gate_up_120x5376x43008.md (ncu capture of the "
                              "gate_up launch, 2026-11-25), scaled to the mean launch by "
                              "algorithmic bytes"}


# --------------------------------------------------------------------------- library baseline
def library_baseline(config, fp8, peaks):
    """The reference's own algorithm on the same GPU: its Fp8Linear (cuBLASLt) on the seven linear
    shapes of the model at 120 rows, and its unfused LM-head chain (quantise -> FP8 GEMM ->
    row argmax, cuda/batch_model_runner.cu:840-853,938-940), next to this repository's kernels on
    the same weights. Each shape rotates over the weights of several layers so that every call
    starts with a cold L2. The reference side is oracle/_ref/libref_cuda.so (the reference's
    sources compiled unmodified for sm_100a); without it the object says so."""
    path = os.path.join(ROOT, "oracle", "_ref", "libref_cuda.so")
    if not os.path.exists(path):
        return {"unavailable": "oracle/_ref/libref_cuda.so is not built"}
    import carat_b200
    from carat_b200.capi import check
    ours = carat_b200.library()
    theirs = ctypes.CDLL(path, mode=os.RTLD_NOW)
    P, I = ctypes.c_void_p, ctypes.c_int
    theirs.ref_fp8_linear_launch.argtypes = [P, P, P, P, P, I, I, I]
    theirs.ref_quantize_argmax_launch.argtypes = [P, P, P, P, P, P, P, P, I, I, I]
    theirs.ref_argmax_bf16_workspace_bytes.restype = ctypes.c_size_t
    theirs.ref_argmax_bf16_workspace_bytes.argtypes = [I]
    theirs.ref_last_error.restype = ctypes.c_char_p
    rows = SLOTS * DEPTH
    hidden, inter = config.hidden_size, config.intermediate_size
    sliding = [i for i, layer in enumerate(config.layers) if layer.attention == "sliding"]
    global_ = [i for i, layer in enumerate(config.layers) if layer.attention == "global"]
    first_sliding, first_global = config.layers[sliding[0]], config.layers[global_[0]]
    shapes = [("sliding_qkv", "qkv", sliding, hidden, first_sliding.packed_width()),
              ("sliding_o", "o", sliding, first_sliding.query_width(), hidden),
              ("global_qkv", "qkv", global_, hidden, first_global.packed_width()),
              ("global_o", "o", global_, first_global.query_width(), hidden),
              ("gate_up", "gate_up", sliding, hidden, 2 * inter),
              ("down", "down", sliding, inter, hidden)]
    widest = max(inter, first_global.query_width())
    x = torch.randint(0, 120, (rows, widest), dtype=torch.uint8, device="cuda")
    scale = torch.ones(1, dtype=torch.float32, device="cuda")
    out = torch.empty(rows, max(2 * inter, 4096), dtype=torch.bfloat16, device="cuda")
    work = torch.empty(64 << 20, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def timed(call, count):
        call(0)
        call(1)
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for index in range(count):
            call(index)
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end) / count * 1e3

    result = {"rows": rows, "unit": "us per call", "shapes": {}}
    for label, segment, layers, k, n in shapes:
        names = [f"layer.{index}.{segment}" for index in layers[:10]]

        def reference_call(index, names=names, k=k, n=n):
            name = names[index % len(names)]
            if theirs.ref_fp8_linear_launch(x.data_ptr(), scale.data_ptr(),
                                            fp8.at(name).data_ptr(), fp8.scale(name).data_ptr(),
                                            out.data_ptr(), rows, k, n) != 0:
                raise RuntimeError(theirs.ref_last_error().decode())

        def our_call(index, names=names, k=k, n=n):
            name = names[index % len(names)]
            check(ours.carat_b200_fp8_linear(
                x.data_ptr(), scale.data_ptr(), fp8.at(name).data_ptr(),
                fp8.scale(name).data_ptr(), out.data_ptr(), rows, k, n, work.data_ptr(),
                work.numel(), stream))

        count = 2 * len(names)
        try:
            reference_us = timed(reference_call, count)
        except RuntimeError as error:
            result["shapes"][label] = {"k": k, "n": n, "reference_error": str(error)}
            continue
        ours_us = timed(our_call, count)
        result["shapes"][label] = {"k": k, "n": n, "cublaslt_us": reference_us, "ours_us": ours_us,
                                   "cublaslt_weight_gbs": k * n / reference_us / 1e3,
                                   "ours_weight_gbs": k * n / ours_us / 1e3}
    # LM head: the reference's three launches (and 63 MB of logits) against the fused epilogue.
    vocabulary = config.vocabulary_size
    final_hidden = torch.randn(rows, hidden, device="cuda").to(torch.bfloat16)
    quantised = torch.empty(rows, hidden, dtype=torch.uint8, device="cuda")
    quantised_scale = torch.zeros(1, dtype=torch.float32, device="cuda")
    scratch = torch.zeros(1, dtype=torch.int32, device="cuda")
    logits = torch.empty(rows, vocabulary, dtype=torch.bfloat16, device="cuda")
    tokens = torch.empty(rows, dtype=torch.int32, device="cuda")
    keys = torch.empty(rows, dtype=torch.int64, device="cuda")
    argmax_work = torch.empty(theirs.ref_argmax_bf16_workspace_bytes(vocabulary) * rows,
                              dtype=torch.uint8, device="cuda")
    head, head_scale = fp8.at("token_embedding"), fp8.scale("token_embedding")

    def reference_head(_):
        if theirs.ref_quantize_argmax_launch(
                final_hidden.data_ptr(), quantised.data_ptr(), quantised_scale.data_ptr(),
                head.data_ptr(), head_scale.data_ptr(), logits.data_ptr(), tokens.data_ptr(),
                argmax_work.data_ptr(), rows, hidden, vocabulary) != 0:
            raise RuntimeError(theirs.ref_last_error().decode())

    def our_head(_):
        check(ours.carat_b200_quantize_bf16_to_fp8(
            final_hidden.data_ptr(), quantised.data_ptr(), quantised_scale.data_ptr(),
            scratch.data_ptr(), rows, hidden, stream))
        check(ours.carat_b200_fp8_linear_argmax(
            quantised.data_ptr(), quantised_scale.data_ptr(), head.data_ptr(),
            head_scale.data_ptr(), tokens.data_ptr(), keys.data_ptr(), rows, hidden, vocabulary,
            stream))

    try:
        result["lm_head_chain"] = {"k": hidden, "n": vocabulary,
                                   "reference_unfused_us": timed(reference_head, 4),
                                   "ours_fused_us": timed(our_head, 4)}
    except RuntimeError as error:
        result["lm_head_chain"] = {"reference_error": str(error)}
    return result


# --------------------------------------------------------------------------- CPU arm
def bookkeeping_sample():
    """Seconds one step's host bookkeeping takes (acceptance_cap + commit_speculation for 24
    slots), with the reference's own compiled speculation.cpp when oracle/_ref holds it."""
    from oracle import carat_semantics as cs
    reference = os.path.join(ROOT, "oracle", "_ref", "libref_speculation.so")
    begin = time.perf_counter()
    if os.path.exists(reference):
        library = ctypes.CDLL(reference)
        proposals = (ctypes.c_int * DEPTH)(*range(10, 10 + DEPTH))
        stops = (ctypes.c_int * 1)(1)
        resident = (ctypes.c_int * (DEPTH + 1))()
        emitted = (ctypes.c_int * (DEPTH + 1))()
        counts = [ctypes.c_int(), ctypes.c_int(), ctypes.c_int()]
        for _ in range(SLOTS):
            cap = library.ref_acceptance_cap(DEPTH, 100, proposals, DEPTH, stops, 1)
            library.ref_commit_speculation(10, proposals, max(cap - 1, 0), 20, stops, 1, resident,
                                           ctypes.byref(counts[0]), emitted,
                                           ctypes.byref(counts[1]), ctypes.byref(counts[2]))
        return time.perf_counter() - begin, "reference speculation.cpp (oracle/_ref)"
    for _ in range(SLOTS):
        cap = cs.acceptance_cap(DEPTH, 100, list(range(10, 10 + DEPTH)), {1})
        cs.commit_speculation(10, list(range(11, 10 + cap)), 20, {1})
    return time.perf_counter() - begin, "oracle port of speculation.cpp"


def cpu_sample(config, lengths, kind_only):
    """The reference's CPU path on a bounded sample: the oracle's restatement of one sliding layer,
    one global layer and the LM head of the verify forward at the benchmark's 120 rows and context
    lengths (PyTorch CPU, all host threads), extrapolated 50 / 10 / 1 to a full step, plus the
    reference's own C++ acceptance / commit logic when oracle/_ref is built."""
    from oracle import carat_semantics as cs
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    full = cs.gemma4_31b_config(MAX_CONTEXT)
    positions = context_lengths(seed=3)
    generator = torch.Generator().manual_seed(0)

    def matrix(rows, cols):
        return cs.bf16(torch.empty(rows, cols).normal_(0.0, 0.02, generator=generator))

    timings = {}
    hidden = cs.bf16(torch.randn(SLOTS * DEPTH, full.hidden, generator=generator))
    for kind, index in (("sliding", 0), ("global", 5)):
        layer = full.layers[index]
        sample = cs.ModelConfig(full.hidden, full.intermediate, 8, full.window, MAX_CONTEXT, full.eps,
                                [layer])
        weights = {"token_embedding": torch.zeros(8, full.hidden), "final_norm": torch.ones(full.hidden)}
        prefix = "layer.0."
        for name, width in (("input_norm", full.hidden), ("q_norm", layer.head_dim),
                            ("k_norm", layer.head_dim), ("post_attention_norm", full.hidden),
                            ("pre_mlp_norm", full.hidden), ("post_mlp_norm", full.hidden)):
            weights[prefix + name] = torch.ones(width)
        weights[prefix + "scalar"] = torch.ones(1)
        weights[prefix + "qkv"] = matrix(layer.packed_width, full.hidden)
        weights[prefix + "o"] = matrix(full.hidden, layer.query_width)
        weights[prefix + "gate_up"] = matrix(2 * full.intermediate, full.hidden)
        weights[prefix + "down"] = matrix(full.hidden, full.intermediate)
        runner = cs.OracleRunner(sample, weights, SLOTS)
        runner.positions = list(positions)
        begin = time.perf_counter()
        runner._verify_layer(0, hidden, list(range(SLOTS)), positions, DEPTH)
        timings[kind] = time.perf_counter() - begin
        del runner, weights
    head = cs.quantize_e4m3(matrix(full.vocab // 8, full.hidden))   # one eighth of the LM head
    begin = time.perf_counter()
    xq, xs = cs.quantize_e4m3(hidden)
    logits = cs.fp8_linear(xq, xs, head[0], head[1])
    cs.argmax_lowest_index(logits)
    timings["lm_head"] = (time.perf_counter() - begin) * 8
    timings["bookkeeping"], bookkeeping = bookkeeping_sample()
    step_seconds = 50 * timings["sliding"] + 10 * timings["global"] + timings["lm_head"] + \
        timings["bookkeeping"]
    mean_tokens = float(lengths.float().mean()) * SLOTS
    return {"value": mean_tokens / step_seconds, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": "verify forward of 1 sliding layer + 1 global layer + 1/8 of the LM head at "
                      "120 rows, 24 slots, the benchmark's context lengths (PyTorch CPU restatement "
                      f"of the reference's CUDA numerics), extrapolated x50 / x10 / x8; {bookkeeping}; "
                      "the drafter is not included",
            "extrapolated": True,
            "seconds_per_step_extrapolated": step_seconds,
            "seconds_sampled": {k: round(v, 3) for k, v in timings.items()}}


def hf_bf16_sample(lengths):
    """The PyTorch CPU forward the reference's fixture tools run (Hugging Face Gemma4 text model,
    BF16, eager attention; tools/generate_layer_fixture.py:57-86, tools/compare_gemma4_assistant.py)
    on a bounded sample of the verify step: one sliding + one global decoder layer at the 31B
    widths over 24 slots x (k+1) rows, attending a seeded random KV cache (1023 ring rows; the
    benchmark's mean context length for the global layer, uniform because the model wants a
    rectangular batch), and one eighth of the LM head. Extrapolated x50 / x10 / x8."""
    from transformers import DynamicCache
    from transformers.models.gemma4.configuration_gemma4 import Gemma4TextConfig
    from transformers.models.gemma4.modeling_gemma4 import Gemma4TextModel

    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    positions = context_lengths(seed=3)
    context = sum(positions) // len(positions)
    hidden, vocabulary = 5376, 262144
    generator = torch.Generator().manual_seed(0)

    def model_of(kinds):
        config = Gemma4TextConfig(
            vocab_size=4096, hidden_size=hidden, intermediate_size=21504,
            num_hidden_layers=len(kinds), num_attention_heads=32, num_key_value_heads=16,
            head_dim=256, global_head_dim=512, num_global_key_value_heads=4, attention_k_eq_v=True,
            sliding_window=1024, layer_types=kinds, rms_norm_eps=1e-6,
            hidden_size_per_layer_input=0, num_kv_shared_layers=0,
            max_position_embeddings=MAX_CONTEXT, final_logit_softcapping=None,
            tie_word_embeddings=True, attention_bias=False,
            rope_parameters={
                "sliding_attention": {"rope_type": "default", "rope_theta": 10000.0},
                "full_attention": {"rope_type": "proportional", "partial_rotary_factor": 0.25,
                                   "rope_theta": 1000000.0}})
        config._attn_implementation = "eager"
        return config, Gemma4TextModel(config).to(torch.bfloat16).eval()

    def causal(keys):
        mask = torch.zeros(SLOTS, 1, DEPTH, keys, dtype=torch.bfloat16)
        for row in range(DEPTH):
            mask[:, :, row, keys - DEPTH + row + 1:] = float("-inf")
        return mask

    # One forward through a [sliding, global] pair; each decoder layer is timed by hooks.
    kinds = ["sliding_attention", "full_attention"]
    config, model = model_of(kinds)
    started, spent = {}, {0: [], 1: []}
    for index, layer in enumerate(model.layers):
        layer.register_forward_pre_hook(
            lambda module, inputs, index=index: started.__setitem__(index, time.perf_counter()))
        layer.register_forward_hook(
            lambda module, inputs, output, index=index:
            spent[index].append(time.perf_counter() - started[index]))
    with torch.inference_mode():
        for _ in range(2):
            cache = DynamicCache(config=config)
            for index, kind in enumerate(kinds):
                heads, dim, rows = (16, 256, 1023) if kind == "sliding_attention" else \
                    (4, 512, context)
                cache.update(torch.randn(SLOTS, heads, rows, dim, generator=generator)
                             .to(torch.bfloat16),
                             torch.randn(SLOTS, heads, rows, dim, generator=generator)
                             .to(torch.bfloat16), index)
            ids = torch.randint(3, 4096, (SLOTS, DEPTH), generator=generator)
            position_ids = (context + torch.arange(DEPTH))[None, :].expand(SLOTS, DEPTH)
            model(input_ids=ids, past_key_values=cache, position_ids=position_ids, use_cache=True,
                  attention_mask={"full_attention": causal(context + DEPTH),
                                  "sliding_attention": causal(1023 + DEPTH)})
    del model
    sliding_seconds, global_seconds = min(spent[0]), min(spent[1])
    head = torch.randn(vocabulary // 8, hidden, generator=generator).to(torch.bfloat16)
    rows = torch.randn(SLOTS * DEPTH, hidden, generator=generator).to(torch.bfloat16)
    begin = time.perf_counter()
    (rows @ head.t()).argmax(dim=1)
    head_seconds = (time.perf_counter() - begin) * 8
    bookkeeping_seconds, bookkeeping = bookkeeping_sample()
    step_seconds = 50 * sliding_seconds + 10 * global_seconds + head_seconds + bookkeeping_seconds
    mean_tokens = float(lengths.float().mean()) * SLOTS
    import transformers
    return {"value": mean_tokens / step_seconds, "unit": UNIT, "cores": cores, "kind": "reference",
            "sample": "Hugging Face Gemma4TextModel BF16 eager forward (transformers "
                      f"{transformers.__version__}; the reference's fixture tools pin 5.19.0) of "
                      "one sliding and one global 31B-width decoder layer (each timed by hooks) over "
                      "24 slots x "
                      f"{DEPTH} rows with a random KV cache (1023 ring rows / {context} global "
                      "rows, the benchmark's mean context) and 1/8 of the BF16 LM head, best of 2, "
                      f"extrapolated x50 / x10 / x8; {bookkeeping}; the drafter is not included",
            "extrapolated": True,
            "seconds_per_step_extrapolated": step_seconds,
            "seconds_sampled": {"sliding": round(sliding_seconds, 3),
                                "global": round(global_seconds, 3),
                                "lm_head": round(head_seconds, 3),
                                "bookkeeping": round(bookkeeping_seconds, 6)}}


def run_reference(args, rank, world):
    if rank != 0:
        return
    lengths = accept_lengths(args.steps + args.warmup, seed=7)
    import carat_b200
    config = carat_b200.Gemma4Config.gemma4_31b()
    # One extrapolated sample stands for every step: a full 60-layer CPU step takes tens of
    # seconds, so `steps` of them would not end in minutes. steps_run says what was executed.
    port = cpu_sample(config, lengths, kind_only=True)
    try:
        best = hf_bf16_sample(lengths)
        best["fp8_restatement"] = {key: port[key] for key in ("value", "kind", "sample",
                                                             "seconds_per_step_extrapolated")}
    except Exception as error:   # transformers without Gemma4, or too little host memory
        best = port
        best["hf_bf16_forward"] = f"skipped: {type(error).__name__}: {error}"
    line = {"impl": "reference", "metric": METRIC, "value": best["value"], "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "steps_run": 0,
            "extrapolated": True,
            "ms_per_step": best["seconds_per_step_extrapolated"] * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 (Hugging Face CPU forward)" if best["kind"] == "reference"
            else "fp8_e4m3 values in fp32 arithmetic",
            "data": "synthetic", "config": workload_config(args), "cpu_baseline": best,
            "e2e": {"value": best["value"], "unit": UNIT, "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- multi-process plumbing
def barrier(world):
    if world > 1:
        torch.distributed.barrier()


def reduce_max_and_sum(world, maxima, sums):
    if world == 1:
        return maxima, sums
    # NCCL reduces device tensors; the CPU tests of this plumbing run it over gloo.
    device = "cuda" if torch.distributed.get_backend() == "nccl" else "cpu"
    m = torch.tensor(maxima, dtype=torch.float64, device=device)
    s = torch.tensor(sums, dtype=torch.float64, device=device)
    torch.distributed.all_reduce(m, op=torch.distributed.ReduceOp.MAX)
    torch.distributed.all_reduce(s, op=torch.distributed.ReduceOp.SUM)
    return m.tolist(), s.tolist()


def gather_rows(world, row):
    """Every rank's row of floats, in rank order, on every rank."""
    if world == 1:
        return [row]
    device = "cuda" if torch.distributed.get_backend() == "nccl" else "cpu"
    mine = torch.tensor(row, dtype=torch.float64, device=device)
    rows = [torch.empty_like(mine) for _ in range(world)]
    torch.distributed.all_gather(rows, mine)
    return [entry.tolist() for entry in rows]


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--drafts", type=int, default=4, choices=[2, 4, 8],
                        help="k, drafted tokens per slot and step (the headline metric is k = 4)")
    parser.add_argument("--skip-int4", action="store_true",
                        help="leave the int4_mlp object (the step with INT4 weight-only MLP "
                             "linears, N = 1 only) out")
    parser.add_argument("--same-seeds", action="store_true",
                        help="N > 1: every rank gets the very same slot-by-slot assignment instead of "
                             "the same work in an order of its own "
                             "(separates workload skew from machine effects)")
    parser.add_argument("--skip-cpu", action="store_true",
                        help="leave the cpu_baseline object out (profiling runs)")
    parser.add_argument("--case", nargs="+", metavar="WORD",
                        help="run one small single-kernel workload instead (bench_cases.py): "
                             "NAME [launches [K N [rows]]]")
    args = parser.parse_args()
    if args.case:
        import bench_cases
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        bench_cases.run_case(args.case)
        return
    global DRAFTS, DEPTH
    DRAFTS = args.drafts
    DEPTH = DRAFTS + 1
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl")
    try:
        run_ours(args, rank, world)
    finally:
        if world > 1:
            torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
