"""Small, self-ending single-kernel workloads of bench.py (`python bench.py --case NAME ...`): one
kernel family each, a few launches, inputs larger than the 126 MB L2 but well under a few GB on
the device, so a profiler capture of them ends by itself.

    python bench.py --case linear      # FP8 linear 120 x 5376 -> 43008 (231 MB weights)
    python bench.py --case int4        # INT4 weight-only linear, same shape (116 MB of codes)
    python bench.py --case lm_head     # fused LM head 120 x 5376 -> 262144 (1.4 GB)
    python bench.py --case attention   # sliding verify attention, 24 slots, full ring
    python bench.py --case global      # global verify attention, 24 slots, 4096 context

Optional numbers after the name: launches [K N [rows]].
"""
from __future__ import annotations

import ctypes

import torch

from carat_b200 import capi
from carat_b200.capi import check


def _ptr(tensor):
    return ctypes.c_void_p(tensor.data_ptr()) if tensor is not None else None


def _fp8(rows, cols, seed):
    generator = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randint(0, 120, (rows, cols), dtype=torch.uint8, device="cuda", generator=generator)


def linear(rows=120, k=5376, n=43008, launches=4):
    library = capi.library()
    x, w = _fp8(rows, k, 0), _fp8(n, k, 1)
    scale = torch.full((1,), 0.01, dtype=torch.float32, device="cuda")
    out = torch.empty(rows, n, dtype=torch.bfloat16, device="cuda")
    need = library.carat_b200_fp8_linear_workspace_bytes(rows, k, n)
    work = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    for launch in range(launches):
        if launch == 1:
            start.record()
        check(library.carat_b200_fp8_linear(_ptr(x), _ptr(scale), _ptr(w), _ptr(scale), _ptr(out),
                                            rows, k, n, _ptr(work), need, None))
    stop.record()
    torch.cuda.synchronize()
    if launches > 1:
        micro = start.elapsed_time(stop) / (launches - 1) * 1e3
        print(f"linear {rows}x{k}x{n}: {micro:.1f} us per call, {k * n / micro / 1e6:.2f} TB/s of weights")


def gated(rows=120, k=5376, n=21504, launches=4):
    """gate_up with GeGLU in the epilogue; n is the gated (intermediate) width."""
    library = capi.library()
    weight, activation = _fp8(2 * n, k, 1), _fp8(rows, k, 2)
    weight_scale = activation_scale = torch.full((1,), 0.01, dtype=torch.float32, device="cuda")
    needed = library.carat_b200_fp8_linear_geglu_workspace_bytes(rows, k, n)
    workspace = torch.empty(needed, dtype=torch.uint8, device="cuda")
    activated = torch.empty(rows, n, dtype=torch.bfloat16, device="cuda")
    amax = torch.zeros(1, dtype=torch.int32, device="cuda")
    quantised = torch.empty(rows, n, dtype=torch.uint8, device="cuda")
    out_scale = torch.zeros(1, dtype=torch.float32, device="cuda")
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    for launch in range(launches):
        if launch == 1:
            start.record()
        check(library.carat_b200_fp8_linear_geglu(
            _ptr(activation), _ptr(activation_scale), _ptr(weight), _ptr(weight_scale),
            _ptr(activated), _ptr(amax), _ptr(quantised), _ptr(out_scale), rows, k, n,
            _ptr(workspace), needed, None))
    stop.record()
    torch.cuda.synchronize()
    if launches > 1:
        micro = start.elapsed_time(stop) / (launches - 1) * 1e3
        print(f"gated linear {rows}x{k}x2*{n}: {micro:.1f} us per call (with two small memsets), "
              f"{2 * k * n / micro / 1e6:.2f} TB/s of weights")


def int4(rows=120, k=5376, n=43008, launches=4, group_width=128):
    library = capi.library()
    generator = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(rows, k, device="cuda", generator=generator).to(torch.bfloat16)
    codes = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda", generator=generator)
    scales = torch.full((k // group_width, n), 0.003, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(rows, n, dtype=torch.bfloat16, device="cuda")
    need = library.carat_b200_int4_linear_workspace_bytes(rows, k, n)
    work = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    for launch in range(launches):
        if launch == 1:
            start.record()
        check(library.carat_b200_int4_linear(_ptr(x), _ptr(codes), _ptr(scales), _ptr(out), rows, k,
                                             n, group_width, _ptr(work), need, None))
    stop.record()
    torch.cuda.synchronize()
    if launches > 1:
        micro = start.elapsed_time(stop) / (launches - 1) * 1e3
        weight_bytes = k * n / 2 + (k // group_width) * n * 2
        print(f"int4 linear {rows}x{k}x{n}: {micro:.1f} us per call, "
              f"{weight_bytes / micro / 1e6:.2f} TB/s of codes and scales, "
              f"{2 * rows * k * n / micro / 1e6:.0f} TFLOP/s")


def lm_head(rows=120, k=5376, n=262144, launches=3):
    library = capi.library()
    x, w = _fp8(rows, k, 0), _fp8(n, k, 1)
    scale = torch.full((1,), 0.01, dtype=torch.float32, device="cuda")
    tokens = torch.empty(rows, dtype=torch.int32, device="cuda")
    keys = torch.empty(rows, dtype=torch.int64, device="cuda")
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    for launch in range(launches):
        if launch == 1:
            start.record()
        check(library.carat_b200_fp8_linear_argmax(_ptr(x), _ptr(scale), _ptr(w), _ptr(scale),
                                                   _ptr(tokens), _ptr(keys), rows, k, n, None))
    stop.record()
    torch.cuda.synchronize()
    if launches > 1:
        micro = start.elapsed_time(stop) / (launches - 1) * 1e3
        print(f"lm head {rows}x{k}x{n}: {micro:.1f} us per call, {k * n / micro / 1e6:.2f} TB/s of weights")


def attention(head_dim=256, heads=32, kv_heads=16, window=1024, capacity=1024, position=3000,
              requests=24, depth=5, launches=3, contexts=None):
    library = capi.library()
    generator = torch.Generator(device="cuda").manual_seed(0)

    def normal(*shape):
        return (torch.randn(*shape, device="cuda", generator=generator) * 0.3).to(torch.bfloat16)

    queries = normal(requests, heads, depth, head_dim)
    keys = normal(requests, kv_heads, capacity, head_dim)
    values = normal(requests, kv_heads, capacity, head_dim)
    staged = window > 0
    new_keys = normal(requests, kv_heads, depth, head_dim) if staged else None
    new_values = normal(requests, kv_heads, depth, head_dim) if staged else None
    if contexts is not None:
        position = max(contexts)
    rows = min(position, capacity) if staged else position + depth
    stride = 16 + (rows + 127) // 128 * 128
    positions = torch.full((requests,), position, dtype=torch.int32, device="cuda")
    if contexts is not None:
        positions = torch.tensor(list(contexts), dtype=torch.int32, device="cuda")
    out = torch.empty(requests * depth, heads * head_dim, dtype=torch.bfloat16, device="cuda")
    scores = torch.empty(requests * heads * depth * stride, dtype=torch.bfloat16, device="cuda")
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    for launch in range(launches):
        if launch == 1:
            start.record()
        check(library.carat_b200_verify_attention(
            _ptr(queries), _ptr(keys), _ptr(values), _ptr(new_keys), _ptr(new_values),
            _ptr(positions), _ptr(out), _ptr(scores), stride, requests, depth, heads, kv_heads,
            head_dim, capacity, window, position, None))
    stop.record()
    torch.cuda.synchronize()
    if launches > 1:
        micro = start.elapsed_time(stop) / (launches - 1) * 1e3
        each = positions.clamp(max=capacity) if staged else positions + depth
        moved = int(each.sum()) * kv_heads * head_dim * 2 * 2
        print(f"attention head_dim={head_dim}: {micro:.1f} us per call over {launches - 1} calls, "
              f"{moved / 1e6:.0f} MB of K and V, {moved / micro / 1e6:.2f} TB/s")


def global_attention(launches=3):
    attention(head_dim=512, heads=32, kv_heads=4, window=0, capacity=8192, position=4096,
              launches=launches)


def global_ragged(launches=3):
    """Global layer at the benchmark's ragged contexts (128..6144 tokens, seed of rank 0)."""
    import bench
    attention(head_dim=512, heads=32, kv_heads=4, window=0, capacity=8192,
              contexts=bench.context_lengths(seed=3), launches=launches)


def _period_model(slots, max_context, with_assistant):
    """One period of the 31B layer pattern (five sliding layers and one global layer at the real
    widths, vocabulary 262144) with bf16 and e4m3 weights, and the reference-shaped drafter."""
    import carat_b200
    generator = torch.Generator(device="cuda").manual_seed(0)

    def matrix(rows, cols, std=0.02):
        out = torch.empty(rows, cols, dtype=torch.bfloat16, device="cuda")
        step = max(1, (64 << 20) // cols)
        for start in range(0, rows, step):
            stop = min(rows, start + step)
            out[start:stop] = (torch.randn(stop - start, cols, device="cuda", generator=generator)
                               * std).to(torch.bfloat16)
        return out

    def ones(width):
        return torch.ones(width, dtype=torch.bfloat16, device="cuda")

    layers = [carat_b200.Gemma4LayerConfig("sliding", 32, 16, 256, 1e4, False) for _ in range(5)]
    layers.append(carat_b200.Gemma4LayerConfig("global", 32, 4, 512, 1e6, True))
    config = carat_b200.Gemma4Config(5376, 21504, 262144, 1024, 1e-6, layers)
    hidden, inter = config.hidden_size, config.intermediate_size
    bf16 = {"token_embedding": matrix(config.vocabulary_size, hidden), "final_norm": ones(hidden)}
    weight_bytes = 0
    for index, layer in enumerate(layers):
        prefix = f"layer.{index}."
        for name, width in (("input_norm", hidden), ("q_norm", layer.head_dimension),
                            ("k_norm", layer.head_dimension), ("post_attention_norm", hidden),
                            ("pre_mlp_norm", hidden), ("post_mlp_norm", hidden), ("scalar", 1)):
            bf16[prefix + name] = ones(width)
        for name, rows, cols in (("qkv", layer.packed_width(), hidden),
                                 ("o", hidden, layer.query_width()),
                                 ("gate_up", 2 * inter, hidden), ("down", hidden, inter)):
            bf16[prefix + name] = matrix(rows, cols)
            weight_bytes += 2 * rows * cols
    weights = carat_b200.DeviceWeightArena(bf16)
    fp8 = carat_b200.Fp8WeightArena.quantize(weights)
    if not with_assistant:
        runner = carat_b200.Gemma4BatchModelRunner(config, weights, slots, max_context, fp8)
        return config, runner, weight_bytes, (weights, fp8)
    assistant_config = carat_b200.Gemma4AssistantConfig()
    a_hidden, a_inter = assistant_config.hidden_size, assistant_config.intermediate_size
    a = {"token_embedding": matrix(config.vocabulary_size, a_hidden, 0.05),
         "pre_projection": matrix(a_hidden, 2 * hidden),
         "post_projection": matrix(hidden, a_hidden, 0.05), "final_norm": ones(a_hidden)}
    for index, kind in enumerate(assistant_config.layers):
        prefix = f"layer.{index}."
        head_dim = 512 if kind == "global" else 256
        for name, width in (("input_norm", a_hidden), ("q_norm", head_dim),
                            ("post_attention_norm", a_hidden), ("pre_mlp_norm", a_hidden),
                            ("post_mlp_norm", a_hidden), ("scalar", 1)):
            a[prefix + name] = ones(width)
        a[prefix + "q"] = matrix(assistant_config.query_heads * head_dim, a_hidden, 0.05)
        a[prefix + "o"] = matrix(a_hidden, assistant_config.query_heads * head_dim)
        a[prefix + "gate_up"] = matrix(2 * a_inter, a_hidden, 0.05)
        a[prefix + "down"] = matrix(a_hidden, a_inter)
    a_weights = carat_b200.DeviceWeightArena(a)
    a_fp8 = carat_b200.Fp8WeightArena.quantize(a_weights)
    runner = carat_b200.Gemma4BatchModelRunner(config, weights, slots, max_context, fp8, a_weights,
                                               a_fp8, assistant_config)
    return config, runner, weight_bytes, (weights, fp8, a_weights, a_fp8)


def prefill(launches=6, slots=24, chunk=8, context=1024):
    """BF16 prompt prefill on one period of the 31B layer pattern: `slots` prompts advance `chunk`
    tokens a call from `context` resident tokens. Prints the device time per call, the same figure
    for the 60-layer model (ten periods: extrapolated, the LM head is outside the timed calls) and
    the share of the bf16 weight stream's roofline."""
    # A multiple of 128 rows, like the server's 8192: the tensor-core attention needs that.
    max_context = (context + chunk * (launches + 2) + 64 + 127) // 128 * 128
    config, runner, weight_bytes, keep = _period_model(slots, max_context, with_assistant=False)
    runner.seed_empty_cache_for_benchmark(context)
    tokens = torch.randint(3, config.vocabulary_size, (slots, max_context),
                           generator=torch.Generator().manual_seed(1)).tolist()
    live = list(range(slots))
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    resident = context
    device_ms = 0.0
    for launch in range(launches):
        if launch == 1:
            start.record()
        # Every prompt is longer than what becomes resident, so no call ends with the LM head.
        runner.prefill_slots_chunks(live, [row[:max_context] for row in tokens], chunk)
        resident += chunk
        if launch >= 1:
            device_ms += runner.last_device_ms()[0]
    stop.record()
    torch.cuda.synchronize()
    assert runner.slot_position(0) == resident
    if launches > 1:
        wall = start.elapsed_time(stop) / (launches - 1)
        period = device_ms / (launches - 1)
        rows = slots * chunk
        roofline = weight_bytes / 1e9 / (period / 1e3)
        print(f"bf16 prefill, {slots} slots x {chunk} tokens from context {context}: {period:.2f} ms "
              f"of device time per call over 6 layers ({weight_bytes / 1e9:.2f} GB of bf16 weights "
              f"= {roofline:.0f} GB/s; {wall:.2f} ms wall clock through the Python mirror); x10 for "
              f"60 layers (extrapolated): {10 * period:.1f} ms, "
              f"{rows / (10 * period / 1e3):.0f} prompt tokens/s")
    runner.close()


def prefill_prompt(launches=3, slots=24):
    """Whole prompts from empty slots on one period of the 31B layer pattern: a lone 512-token
    prompt and `slots` of them together (the rings stay unwrapped: a step takes up to 256 rows,
    many eight-token pieces of one prompt), then a lone 3,072-token prompt and four of them
    together (past the first 1,024 tokens the sliding layers go wave by wave). Wall clock through
    the Python mirror, best of `launches`, and the same for ten periods (extrapolated)."""
    import time
    config, runner, weight_bytes, keep = _period_model(slots, 3200, with_assistant=False)
    generator = torch.Generator().manual_seed(2)
    for count, length in ((1, 512), (slots, 512), (1, 3072), (4, 3072)):
        prompts = torch.randint(3, config.vocabulary_size, (count, length),
                                generator=generator).tolist()
        best = None
        for _ in range(launches):
            for slot in range(count):
                runner.reset_slot(slot)
            torch.cuda.synchronize()
            begin = time.perf_counter()
            calls = 0
            pending = list(range(count))
            while pending:
                done = runner.prefill_slots_chunks(pending, [prompts[slot] for slot in pending],
                                                   length)
                calls += 1
                pending = [slot for slot, first in zip(pending, done) if first is None]
            wall = (time.perf_counter() - begin) * 1e3
            if best is None or wall < best:
                best = wall
        print(f"{count} prompt(s) of {length} tokens from empty slots: {best:.1f} ms wall clock over "
              f"6 layers ({count * length / best * 1e3:.0f} prompt tokens/s); x10 for 60 layers "
              f"(extrapolated): {10 * best:.0f} ms to the first token, "
              f"{count * length / (10 * best) * 1e3:.0f} prompt tokens/s")
    runner.close()


def single(launches=1, slots=24):
    """One request alone, as the batch-1 configuration describes it: a 512-token prompt, k = 4,
    256 new tokens with real greedy acceptance, through the scheduler loop (BF16 prefill, then
    draft -> verify -> commit), on one period of the 31B layer pattern with the real drafter.
    Prints the time to the first token and the decode rate of this 6-layer model."""
    import random
    import time
    from carat_b200.dispatcher import ReplicaScheduler, Request
    config, runner, _, keep = _period_model(slots, 1024, with_assistant=True)
    generator = random.Random(5)
    for attempt in range(launches + 1):                # the first pass warms plans and maps up
        for slot in range(slots):
            runner.reset_slot(slot)
        scheduler = ReplicaScheduler(runner, slots, depth=5, chunk_tokens=512)
        prompt = [generator.randrange(3, config.vocabulary_size) for _ in range(512)]
        scheduler.admit(Request(attempt, prompt, 256), 0, None, 0)
        torch.cuda.synchronize()
        begin = time.perf_counter()
        first_token_at = None
        emitted = 0
        while not scheduler.idle():
            tokens, _ = scheduler.tick()
            emitted += sum(len(row) for row in tokens.values())
            if first_token_at is None and emitted > 0:
                first_token_at = time.perf_counter() - begin
        total = time.perf_counter() - begin
    metrics = scheduler.metrics
    print(f"one request, prompt 512, 256 new tokens, k = 4 on a 6-layer 31B-width replica: first "
          f"token after {first_token_at * 1e3:.1f} ms, {emitted} tokens in {total * 1e3:.0f} ms "
          f"({(emitted - 1) / (total - first_token_at):.0f} tokens/s after the first), "
          f"{metrics['speculative_cycles']} speculative cycles, {metrics['accepted_tokens']} rows "
          f"accepted of {metrics['proposed_tokens']} proposed")
    assert emitted == 256 and runner.slot_position(0) == len(scheduler.slots[0].cached_tokens)
    runner.close()


def serving(launches=72, slots=24):
    """A request mix through the dispatcher and one replica's scheduler loop on one period of the
    31B layer pattern with the real drafter: `launches` requests, prompts of 128..1536 tokens of
    which half share a 512-token prefix, 16..96 new tokens each with real greedy acceptance, a
    third of them second turns of finished conversations; closed loop (a request is admitted as
    soon as the router finds it a slot), BF16 prefill in quanta of 64 tokens between decode steps.
    It shows the path's callers working together at the real widths; its tokens/s belong to a
    6-layer model, not to the 31B one."""
    import random
    import time
    from carat_b200.dispatcher import (Dispatcher, LocalChannel, ReplicaScheduler, ReplicaWorker,
                                       Request)
    max_context = 2048
    config, runner, _, keep = _period_model(slots, max_context, with_assistant=True)
    generator = random.Random(3)

    def tokens(count):
        return [generator.randrange(3, config.vocabulary_size) for _ in range(count)]

    shared = tokens(512)
    channel = LocalChannel()
    front = Dispatcher(channel, 1, slots)
    worker = ReplicaWorker(channel, 0, ReplicaScheduler(runner, slots, depth=5, chunk_tokens=64))
    first_turns = launches - launches // 3
    waiting = []
    for request_id in range(first_turns):
        length = generator.randint(128, 1536)
        prompt = (shared + tokens(length - 512)) if request_id % 2 and length > 512 else tokens(length)
        waiting.append(Request(request_id, prompt, generator.randint(16, 96)))
    second_turns = launches - first_turns
    prompt_tokens = sum(len(request.input_ids) for request in waiting)
    torch.cuda.synchronize()
    begin = time.perf_counter()
    for request in waiting:
        front.submit(request)
    followed = set()
    next_id = first_turns
    rounds = 0
    while not front.finished() or len(followed) < second_turns:
        front.poll()
        worker.step()
        rounds += 1
        for request_id, output in list(front.completed.items()):
            if request_id < first_turns and request_id not in followed and len(followed) < second_turns:
                parent = front.origin[request_id]
                history = parent.input_ids + output
                if len(history) + 8 + 64 < max_context - 16:
                    followed.add(request_id)
                    turn = Request(next_id, history + tokens(8), generator.randint(16, 64))
                    prompt_tokens += len(turn.input_ids)
                    front.submit(turn)
                    next_id += 1
                elif request_id not in followed:
                    followed.add(request_id)      # too long to continue: counts as handled
        if rounds > 200000:
            raise RuntimeError("the request mix did not drain")
    front.poll()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - begin
    emitted = sum(len(output) for output in front.completed.values())
    metrics = front.aggregate_metrics()
    print(f"serving mix on a 6-layer 31B-width replica: {len(front.completed)} requests, "
          f"{prompt_tokens} prompt tokens ({metrics['prefill_tokens']} prefilled, "
          f"{metrics['prefix_tokens_reused']} reused from cache, {metrics['kv_clones']} slot clones), "
          f"{emitted} tokens emitted in {seconds:.2f} s = {emitted / seconds:.0f} tokens/s; "
          f"{metrics['decode_steps']} decode steps, {metrics['accepted_tokens']} verify rows accepted "
          f"of {metrics['proposed_tokens']} proposed, {metrics['first_token_rejections']} "
          f"first-token rejections")
    for index, slot in enumerate(worker.scheduler.slots):
        if slot.cached_tokens:
            assert runner.slot_position(index) == len(slot.cached_tokens), index
    runner.close()


CASES = {"prefill": prefill, "prefill_prompt": prefill_prompt, "single": single, "serving": serving, "linear": linear, "gated": gated, "int4": int4, "lm_head": lm_head, "attention": attention, "global": global_attention,
         "global_ragged": global_ragged}



def run_case(words):
    """words = [name, launches, K, N, rows] (all but the name optional)."""
    name = words[0] if words else "linear"
    numbers = [int(word) for word in words[1:]]
    if len(numbers) > 3:
        CASES[name](launches=numbers[0], k=numbers[1], n=numbers[2], rows=numbers[3])
    elif len(numbers) > 2:
        CASES[name](launches=numbers[0], k=numbers[1], n=numbers[2])
    elif len(numbers) > 0:
        CASES[name](launches=numbers[0])
    else:
        CASES[name]()
    print(f"case {name} done")
