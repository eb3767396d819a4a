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
                    "context lengths uniform in [128, 6144] (seeded), zero-filled KV, accept "
                    "lengths injected from a seeded geometric distribution with mean 2.5",
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


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.device_index = device_index
        self.process = None
        self.path = None

    def start(self):
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
        if self.process is None:
            return result
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        clocks, reasons, maximum = [], set(), None
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
        if clocks:
            clocks.sort()
            busy = clocks[len(clocks) // 2:]   # upper half: samples taken under load
            result["sm_mhz"] = busy[len(busy) // 2]
            result["sm_max_mhz"] = maximum
            result["reasons"] = sorted(reasons)
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
                                               a_fp8, assistant_config)
    return config, runner, fp8


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
    lengths = accept_lengths(args.steps + args.warmup, seed=7 + rank)
    generator = torch.Generator().manual_seed(11 + rank)
    slots = list(range(SLOTS))
    start_positions = context_lengths(seed=3 + rank)
    runner.seed_slot_positions(start_positions)
    last_tokens = torch.randint(3, config.vocabulary_size, (SLOTS,), generator=generator).tolist()
    next_tokens = torch.randint(3, config.vocabulary_size, (SLOTS,), generator=generator).tolist()

    def one_step(step):
        nonlocal last_tokens, next_tokens
        if any(runner.slot_position(slot) + DEPTH > MAX_CONTEXT for slot in slots):
            runner.seed_slot_positions(start_positions)
        proposals = runner.draft_four(last_tokens, slots, next_tokens, DEPTH)
        caps = lengths[step].tolist()
        result = runner.verify_greedy_proposals(proposals, next_tokens, slots, caps,
                                                carat_b200.VERIFY_ASSUME_MATCH)
        verify_ms, draft_ms = runner.last_device_ms()
        verify_launches, draft_launches = runner.last_launches()
        last_tokens = [proposals[r][result.accepted_tokens[r] - 1] for r in range(SLOTS)]
        next_tokens = result.next_tokens
        return sum(result.accepted_tokens), verify_ms, draft_ms, verify_launches + draft_launches

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
        wall_start = time.perf_counter()
        for step in range(args.warmup, args.warmup + args.steps):
            accepted, verify_ms, draft_ms, step_launches = one_step(step)
            tokens += accepted
            device_ms += verify_ms + draft_ms
            verify_total_ms += verify_ms
            launches += step_launches
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - wall_start) * 1e3
        clocks = sampler.stop()
        barrier(world)
        return positions, tokens, device_ms, verify_total_ms, launches, wall_ms, clocks

    (positions_at_start, tokens, device_ms, verify_total_ms, launches, wall_ms,
     clocks) = timed_run()

    totals = reduce_max_and_sum(world, [device_ms, wall_ms], [float(tokens)])
    device_ms_max, wall_ms_max = totals[0]
    tokens_all = totals[1][0]
    if rank != 0:
        return
    peaks = measured_peaks()
    weight_bytes = step_weight_bytes(config)
    kv_bytes = step_kv_bytes(config, positions_at_start)
    verify_ms_step = verify_total_ms / args.steps
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
    }
    line["roofline"] = linear_roofline(library, config, fp8, peaks)
    if world == 1 and args.int4_mlp:
        line["int4_mlp"] = int4_variant(config, runner, timed_run, args, weight_bytes)
    if world == 1 and not args.skip_cpu:
        line["cpu_baseline"] = cpu_sample(config, lengths, kind_only=False)
    print(json.dumps(line), flush=True)


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
        _, tokens, device_ms, verify_total_ms, launches, wall_ms, _ = timed_run()
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


NCU_GATE_UP_DRAM_BYTES = 231.912192e6 + 6.525696e6
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
            "traffic_source": "ncu capture of the gate_up launch, scaled by algorithmic bytes"}


# --------------------------------------------------------------------------- CPU arm
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
    # Host bookkeeping with the reference's own compiled logic when available.
    bookkeeping = "oracle port"
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
        bookkeeping = "reference speculation.cpp (oracle/_ref)"
    else:
        for _ in range(SLOTS):
            cap = cs.acceptance_cap(DEPTH, 100, list(range(10, 10 + DEPTH)), {1})
            cs.commit_speculation(10, list(range(11, 10 + cap)), 20, {1})
    timings["bookkeeping"] = time.perf_counter() - begin
    step_seconds = 50 * timings["sliding"] + 10 * timings["global"] + timings["lm_head"] + \
        timings["bookkeeping"]
    mean_tokens = float(lengths.float().mean()) * SLOTS
    return {"value": mean_tokens / step_seconds, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": "verify forward of 1 sliding layer + 1 global layer + 1/8 of the LM head at "
                      "120 rows, 24 slots, the benchmark's context lengths (PyTorch CPU restatement "
                      f"of the reference's CUDA numerics), extrapolated x50 / x10 / x8; {bookkeeping}; "
                      "the drafter is not included",
            "seconds_per_step_extrapolated": step_seconds,
            "seconds_sampled": {k: round(v, 3) for k, v in timings.items()}}


def run_reference(args, rank, world):
    if rank != 0:
        return
    lengths = accept_lengths(args.steps + args.warmup, seed=7)
    import carat_b200
    config = carat_b200.Gemma4Config.gemma4_31b()
    samples = []
    for _ in range(max(1, min(args.steps, 2))):
        samples.append(cpu_sample(config, lengths, kind_only=True))
    best = max(samples, key=lambda sample: sample["value"])
    line = {"impl": "reference", "metric": METRIC, "value": best["value"], "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": best["seconds_per_step_extrapolated"] * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 values in fp32 arithmetic",
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


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--drafts", type=int, default=4, choices=[2, 4, 8],
                        help="k, drafted tokens per slot and step (the headline metric is k = 4)")
    parser.add_argument("--int4-mlp", action="store_true",
                        help="also time the step with INT4 weight-only MLP linears (N = 1 only)")
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
