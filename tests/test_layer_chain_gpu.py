"""One decoder layer, stage by stage: every device operator is fed the oracle's exact input for
that stage (taken from a verify step with a populated KV cache) and must reproduce the oracle's
output of the stage. Localises a discrepancy to one operator."""
import ctypes

import pytest
import torch

import carat_b200
from carat_b200.capi import check
from oracle import carat_semantics as cs

pytestmark = pytest.mark.gpu

_alive = []


@pytest.fixture(autouse=True)
def _release():
    yield
    _alive.clear()


def dev(tensor, dtype=torch.bfloat16):
    moved = tensor.to(device="cuda", dtype=dtype).contiguous()
    _alive.append(moved)
    return moved


def ptr(tensor):
    return ctypes.c_void_p(tensor.data_ptr()) if tensor is not None else None


def fp8_dev(values):
    return dev(values.to(torch.float8_e4m3fn).view(torch.uint8), torch.uint8)


def scale_dev(scale):
    return dev(scale.reshape(1), torch.float32)


def mismatch(got, want):
    got = got.float().cpu().reshape(want.shape)
    return float((got != want).float().mean()), float((got - want).abs().max())


def run_linear(lib, xq, xs, wq, ws, rows, k, n):
    out = torch.empty(rows, n, dtype=torch.bfloat16, device="cuda")
    need = lib.carat_b200_fp8_linear_workspace_bytes(rows, k, n)
    work = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    check(lib.carat_b200_fp8_linear(ptr(fp8_dev(xq)), ptr(scale_dev(xs)), ptr(fp8_dev(wq)),
                                    ptr(scale_dev(ws)), ptr(out), rows, k, n, ptr(work), need, None))
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("layer_index", [0, 1, 2, 3])
def test_layer_stage_by_stage(cuda_device, layer_index):
    lib = carat_b200.library()
    config = cs.tiny_config(512)
    weights = cs.golden_tiny_weights(config)
    oracle = cs.OracleRunner(config, weights, 1)
    generator = torch.Generator().manual_seed(0)
    tokens = torch.randint(3, config.vocab, (24,), generator=generator).tolist()
    oracle.prefill_slot_fp8(0, tokens[:16])
    position, depth = 16, 8
    part = tokens[16:24]
    # Input of the layer under test: run the oracle on a copy and take the previous layer's output.
    import copy
    scout = copy.deepcopy(oracle)
    _, _, trace = scout.verify_greedy_proposals([part], [part[0]], [0], assume_match=True, trace=True)
    if layer_index == 0:
        x = cs.embedding(weights["token_embedding"], torch.tensor(part), config.hidden)
    else:
        x = trace.layer_outputs[layer_index - 1]
    layer = config.layers[layer_index]
    prefix = f"layer.{layer_index}."
    w = weights
    fw = oracle.fp8_weights
    rows, hidden, dim = depth, config.hidden, layer.head_dim
    heads, kv_heads = layer.query_heads, layer.kv_heads
    report = {}

    # a. input norm + quantise
    normalized = cs.rms_norm(x, w[prefix + "input_norm"], config.eps)
    xq, xs = cs.quantize_e4m3(normalized)
    out = torch.empty(rows, hidden, dtype=torch.uint8, device="cuda")
    scale = torch.zeros(1, dtype=torch.float32, device="cuda")
    scratch = torch.zeros(1, dtype=torch.int32, device="cuda")
    check(lib.carat_b200_rms_norm_quantize(ptr(dev(x)), ptr(dev(w[prefix + "input_norm"])), None,
                                           ptr(out), ptr(scale), ptr(scratch), rows, hidden,
                                           config.eps, None))
    torch.cuda.synchronize()
    report["a.norm_quant"] = mismatch(out.view(torch.float8_e4m3fn), xq)
    assert float(scale.cpu()) == float(xs)

    # b. qkv linear
    wq, ws = fw[prefix + "qkv"]
    packed = cs.fp8_linear(xq, xs, wq, ws)
    got = run_linear(lib, xq, xs, wq, ws, rows, hidden, layer.packed_width)
    report["b.qkv"] = mismatch(got, packed)

    # c. qkv post
    cos, sin = oracle.rope[(layer.kind, dim)]
    row_positions = torch.arange(position, position + depth)
    q_raw = packed[:, :layer.query_width].reshape(rows, heads, dim)
    k_raw = packed[:, layer.query_width:layer.query_width + layer.kv_width].reshape(rows, kv_heads, dim)
    v_raw = k_raw if layer.key_equals_value else packed[:, layer.query_width + layer.kv_width:].reshape(
        rows, kv_heads, dim)
    queries = cs.norm_rope(q_raw, w[prefix + "q_norm"], cos[row_positions], sin[row_positions], config.eps)
    new_k = cs.norm_rope(k_raw, w[prefix + "k_norm"], cos[row_positions], sin[row_positions], config.eps)
    new_v = cs.rms_norm(v_raw, None, config.eps)
    d_q = torch.empty(1, heads, depth, dim, dtype=torch.bfloat16, device="cuda")
    d_k = torch.empty(1, kv_heads, depth, dim, dtype=torch.bfloat16, device="cuda")
    d_v = torch.empty_like(d_k)
    d_cos = torch.empty(config.max_context, dim, dtype=torch.bfloat16, device="cuda")
    d_sin = torch.empty_like(d_cos)
    check(lib.carat_b200_rope_tables(ptr(d_cos), ptr(d_sin), config.max_context, dim,
                                     layer.rope_theta, 1 if layer.kind == "global" else 0, None))
    check(lib.carat_b200_qkv_postprocess(
        ptr(dev(packed)), ptr(dev(w[prefix + "q_norm"])), ptr(dev(w[prefix + "k_norm"])), ptr(d_cos),
        ptr(d_sin), ptr(d_q), ptr(d_k), ptr(d_v), ptr(dev(torch.tensor([position]), torch.int32)), 1,
        depth, heads, kv_heads, dim, 1 if layer.key_equals_value else 0, config.max_context,
        config.eps, None))
    torch.cuda.synchronize()
    report["c.q"] = mismatch(d_q.permute(0, 2, 1, 3), queries.reshape(1, depth, heads, dim))
    report["c.k"] = mismatch(d_k.permute(0, 2, 1, 3), new_k.reshape(1, depth, kv_heads, dim))
    report["c.v"] = mismatch(d_v.permute(0, 2, 1, 3), new_v.reshape(1, depth, kv_heads, dim))

    # d. attention
    window = config.window if layer.kind == "sliding" else 0
    capacity = config.capacity(layer_index)
    attention = cs.verify_attention(
        queries.reshape(1, depth, heads, dim), [oracle.keys[layer_index][0]],
        [oracle.values[layer_index][0]], new_k.reshape(1, depth, kv_heads, dim),
        new_v.reshape(1, depth, kv_heads, dim), [position], window)
    cache_rows = min(position, capacity) if window > 0 else position + depth
    stride = 16 + (cache_rows + 127) // 128 * 128
    if window > 0:
        cache_k, cache_v = dev(oracle.keys[layer_index][0:1]), dev(oracle.values[layer_index][0:1])
        side_k = dev(new_k.reshape(1, depth, kv_heads, dim).permute(0, 2, 1, 3))
        side_v = dev(new_v.reshape(1, depth, kv_heads, dim).permute(0, 2, 1, 3))
    else:
        filled_k = oracle.keys[layer_index][0:1].clone()
        filled_v = oracle.values[layer_index][0:1].clone()
        filled_k[0, :, position:position + depth] = new_k.reshape(depth, kv_heads, dim).permute(1, 0, 2)
        filled_v[0, :, position:position + depth] = new_v.reshape(depth, kv_heads, dim).permute(1, 0, 2)
        cache_k, cache_v, side_k, side_v = dev(filled_k), dev(filled_v), None, None
    d_out = torch.empty(depth, heads * dim, dtype=torch.bfloat16, device="cuda")
    d_scores = torch.zeros(heads * depth * stride, dtype=torch.bfloat16, device="cuda")
    check(lib.carat_b200_verify_attention(
        ptr(dev(queries.reshape(1, depth, heads, dim).permute(0, 2, 1, 3))),
        ptr(cache_k), ptr(cache_v), ptr(side_k), ptr(side_v),
        ptr(dev(torch.tensor([position]), torch.int32)), ptr(d_out), ptr(d_scores), stride, 1, depth,
        heads, kv_heads, dim, capacity, window, position, None))
    torch.cuda.synchronize()
    attention_rows = attention.reshape(rows, heads * dim)
    report["d.attention"] = mismatch(d_out, attention_rows)

    # e. attention quantise, f. o linear
    aq, a_s = cs.quantize_e4m3(attention_rows)
    check(lib.carat_b200_quantize_bf16_to_fp8(ptr(dev(attention_rows)), ptr(out), ptr(scale),
                                              ptr(scratch), rows, heads * dim, None))
    torch.cuda.synchronize()
    report["e.quant"] = mismatch(out.view(torch.float8_e4m3fn)[:, :heads * dim], aq)
    wq, ws = fw[prefix + "o"]
    projected = cs.fp8_linear(aq, a_s, wq, ws)
    report["f.o"] = mismatch(run_linear(lib, aq, a_s, wq, ws, rows, heads * dim, hidden), projected)

    # g. post-attention norms
    first, pre_mlp = cs.rms_norm_add_and_norm(projected, w[prefix + "post_attention_norm"], x,
                                              w[prefix + "pre_mlp_norm"], config.eps)
    mq, m_s = cs.quantize_e4m3(pre_mlp)
    d_first = torch.empty(rows, hidden, dtype=torch.bfloat16, device="cuda")
    check(lib.carat_b200_rms_norm_add_and_norm_quantize(
        ptr(dev(projected)), ptr(dev(w[prefix + "post_attention_norm"])), ptr(dev(x)),
        ptr(dev(w[prefix + "pre_mlp_norm"])), ptr(d_first), ptr(out), ptr(scale), ptr(scratch), rows,
        hidden, config.eps, None))
    torch.cuda.synchronize()
    report["g.first"] = mismatch(d_first, first)
    report["g.quant"] = mismatch(out.view(torch.float8_e4m3fn), mq)

    # h. gate_up, i. geglu, j. down
    wq, ws = fw[prefix + "gate_up"]
    gate_up = cs.fp8_linear(mq, m_s, wq, ws)
    report["h.gate_up"] = mismatch(run_linear(lib, mq, m_s, wq, ws, rows, hidden,
                                              2 * config.intermediate), gate_up)
    activated = cs.gelu_tanh_gate(gate_up, config.intermediate)
    gq, g_s = cs.quantize_e4m3(activated)
    wide = torch.empty(rows, config.intermediate, dtype=torch.uint8, device="cuda")
    check(lib.carat_b200_gelu_gate_quantize(ptr(dev(gate_up)), ptr(wide), ptr(scale), ptr(scratch),
                                            rows, config.intermediate, None))
    torch.cuda.synchronize()
    report["i.geglu"] = mismatch(wide.view(torch.float8_e4m3fn), gq)
    wq, ws = fw[prefix + "down"]
    down = cs.fp8_linear(gq, g_s, wq, ws)
    report["j.down"] = mismatch(run_linear(lib, gq, g_s, wq, ws, rows, config.intermediate, hidden),
                                down)

    # k. layer output + next norm
    output = cs.rms_norm_add_scale(down, w[prefix + "post_mlp_norm"], first, w[prefix + "scalar"],
                                   config.eps)
    d_output = torch.empty(rows, hidden, dtype=torch.bfloat16, device="cuda")
    check(lib.carat_b200_rms_norm_add_scale_then_norm_quantize(
        ptr(dev(down)), ptr(dev(w[prefix + "post_mlp_norm"])), ptr(dev(first)),
        ptr(dev(w[prefix + "scalar"])), ptr(d_output), ptr(dev(w["final_norm"])), None, ptr(out),
        ptr(scale), ptr(scratch), rows, hidden, config.eps, None))
    torch.cuda.synchronize()
    report["k.output"] = mismatch(d_output, output)
    report["k.vs_trace"] = mismatch(d_output, trace.layer_outputs[layer_index])

    print(f"layer {layer_index}: " + ", ".join(f"{k}={v[0]:.4f}/{v[1]:.4g}" for k, v in report.items()))
    for name, (fraction, worst) in report.items():
        assert fraction < 0.01, (name, fraction, worst)
