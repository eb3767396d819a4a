"""CPU restatement of the Carat speculative-decoding step (TEST INFRASTRUCTURE, not product code).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this module; the
product path (carat_b200/) never does.

Every function restates, rounding point by rounding point, what the reference's CUDA path computes
and cites the reference file:line it follows (paths inside the Gradiated/carat tree). Tensors are
torch float32 holding values that are exactly representable in the storage type the reference uses
at that point (bf16 or e4m3), so `bf16(x)` below marks each place the reference rounds.

Pinning: the integer logic is checked against the reference's own known-answer tests
(tests/speculation_tests.cpp, tests/cuda_ops_tests.cu argmax tie rule) and against the reference's
compiled speculation.cpp (oracle/_ref); the floating-point layer math is checked in BF16 mode
against the Hugging Face Gemma4 text model that the reference's fixture tools use
(tools/generate_layer_fixture.py). The FP8 path, the verify accept loop, the ring rollback and the
drafter have no reference test that runs without the real checkpoint: for those parts parity is
pinned only to this restatement ("parity unpinned" beyond what is listed above).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

E4M3_MAX = 448.0


# --------------------------------------------------------------------------- configuration
@dataclass
class LayerConfig:
    """One decoder layer's attention shape (include/carat/gemma4_config.h:14-26)."""

    kind: str  # "sliding" | "global"
    query_heads: int
    kv_heads: int
    head_dim: int
    rope_theta: float
    key_equals_value: bool

    @property
    def query_width(self) -> int:
        return self.query_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.kv_heads * self.head_dim

    @property
    def packed_width(self) -> int:
        return self.query_width + self.kv_width * (1 if self.key_equals_value else 2)


@dataclass
class ModelConfig:
    hidden: int
    intermediate: int
    vocab: int
    window: int
    max_context: int
    eps: float
    layers: List[LayerConfig]

    def capacity(self, layer: int) -> int:
        # cuda/batch_model_runner.cu:330-342: sliding layers keep min(context, window) rows.
        if self.layers[layer].kind == "sliding":
            return min(self.max_context, self.window)
        return self.max_context


@dataclass
class AssistantConfig:
    """Drafter shape. The reference fixes hidden 1024, FFN 8192, 32 query heads, 4 layers with the
    last one global (cuda/assistant_runner.cu:22-27,166-170); here it is a parameter so the small
    test configurations can use the same code."""

    hidden: int
    intermediate: int
    query_heads: int
    layers: List[str]  # "sliding" | "global" per layer; attends the target's shared KV of that kind
    eps: float = 1e-6


def gemma4_31b_config(max_context: int = 8192) -> ModelConfig:
    """Gemma-4-31B text shapes (src/fp8_linear_benchmark.cu:346-351, cuda/layer_runner.cu:162-176);
    a 5 sliding : 1 global repeat is assumed for the layer order."""
    layers = []
    for index in range(60):
        if index % 6 == 5:
            layers.append(LayerConfig("global", 32, 4, 512, 1e6, True))
        else:
            layers.append(LayerConfig("sliding", 32, 16, 256, 1e4, False))
    return ModelConfig(5376, 21504, 262144, 1024, max_context, 1e-6, layers)


def tiny_config(max_context: int = 512) -> ModelConfig:
    """The CPU-runnable plumbing case: 3 sliding (window 128) + 1 global layer, hidden 256,
    4 query / 2 KV heads, head_dim 64, FFN 1024, vocab 4096."""
    layers = [LayerConfig("sliding", 4, 2, 64, 1e4, False) for _ in range(3)]
    layers.append(LayerConfig("global", 4, 2, 64, 1e6, True))
    return ModelConfig(256, 1024, 4096, 128, max_context, 1e-6, layers)


def tiny_assistant() -> AssistantConfig:
    return AssistantConfig(hidden=256, intermediate=1024, query_heads=4, layers=["global"])


# --------------------------------------------------------------------------- rounding helpers
def bf16(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even to bfloat16, returned as float32 (__float2bfloat16_rn)."""
    return x.to(torch.float32).to(torch.bfloat16).to(torch.float32)


def e4m3(x: torch.Tensor) -> torch.Tensor:
    """Saturating round to e4m3 (the __nv_fp8_e4m3 constructor), returned as float32."""
    clamped = torch.clamp(x.to(torch.float32), -E4M3_MAX, E4M3_MAX)
    return clamped.to(torch.float8_e4m3fn).to(torch.float32)


def f32(value: float) -> torch.Tensor:
    return torch.tensor(value, dtype=torch.float32)


# --------------------------------------------------------------------------- elementwise ops
def embedding(weight: torch.Tensor, tokens: torch.Tensor, hidden: int) -> torch.Tensor:
    """cuda/ops.cu:321-335, launch :1140-1153: bf16(W[token] * bf16(sqrt(hidden)))."""
    scale = bf16(f32(math.sqrt(float(hidden))))
    return bf16(weight[tokens.long()] * scale)


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float,
             residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """cuda/ops.cu:27-68: fp32 sum of squares, rsqrt(mean + eps), x*inv*w (+ residual), one bf16
    rounding. weight None is the unweighted V norm of cuda/qkv.cu:528-529."""
    width = x.shape[-1]
    inverse = torch.rsqrt((x * x).sum(dim=-1, keepdim=True) / f32(float(width)) + f32(eps))
    y = x * inverse
    if weight is not None:
        y = y * weight
    if residual is not None:
        y = y + residual
    return bf16(y)


def rms_norm_add_and_norm(x, weight, residual, next_weight, eps):
    """cuda/ops.cu:87-179: r = bf16(norm(x)*w + residual); y = bf16(norm(r)*w2), r re-read as bf16."""
    first = rms_norm(x, weight, eps, residual)
    return first, rms_norm(first, next_weight, eps)


def rms_norm_add_scale(x, weight, residual, scalar, eps):
    """cuda/ops.cu:181-217: bf16(bf16(norm(x)*w + residual) * scalar)."""
    return bf16(rms_norm(x, weight, eps, residual) * scalar)


def gelu_tanh_gate(packed: torch.Tensor, width: int) -> torch.Tensor:
    """cuda/ops.cu:228-252: bf16(gelu_tanh(gate) * up) from rows packed as [gate | up]."""
    gate, up = packed[:, :width], packed[:, width:]
    inner = f32(0.7978845608028654) * (gate + f32(0.044715) * gate * gate * gate)
    return bf16(f32(0.5) * gate * (f32(1.0) + torch.tanh(inner)) * up)


def quantize_e4m3(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """cuda/linear.cu:76-115 (and :117-153, :155-189, same contract): amax over the whole tensor,
    scale = amax/448 (1 when amax == 0), value = e4m3(x * (1/scale)) with 1/scale rounded once."""
    amax = x.abs().max().to(torch.float32)
    scale = amax / f32(E4M3_MAX) if float(amax) > 0.0 else f32(1.0)
    inverse = f32(1.0) / scale
    return e4m3(x * inverse), scale


def fp8_linear(xq, x_scale, wq, w_scale) -> torch.Tensor:
    """cuda/linear.cu:645-803: bf16((sx*sw) * Xq . Wq^T) with fp32 accumulation (order unspecified)."""
    return bf16((xq @ wq.t()) * (x_scale * w_scale))


def bf16_linear(x, w) -> torch.Tensor:
    """cuda/linear.cu:534-643: bf16(X . W^T), fp32 accumulation."""
    return bf16(x @ w.t())


def int4_quantize(weight: torch.Tensor, group_width: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """cuda/int4_bf16_linear.cu:95-136: per output row and K-local group, scale = bf16(max|w| / 7)
    (1 when the group is all zero), code = clamp(rint(w / float(scale)), -7, 7).
    Returns (codes int8 [N, K], scales bf16-exact float [K / group, N], group-major)."""
    rows, width = weight.shape
    groups = width // group_width
    grouped = weight.float().reshape(rows, groups, group_width)
    maximum = grouped.abs().amax(dim=2)
    scale = bf16(torch.where(maximum > 0, maximum / f32(7.0), torch.ones_like(maximum)))
    codes = torch.clamp(torch.round(grouped / scale[:, :, None]), -7, 7)
    return codes.reshape(rows, width).to(torch.int8), scale.t().contiguous()


def int4_pack(codes: torch.Tensor) -> torch.Tensor:
    """Two codes a byte, even K in the low nibble (cuda/int4_bf16_linear.cu:126-134)."""
    nibbles = (codes.to(torch.int16) & 0xF).to(torch.uint8)
    return nibbles[:, 0::2] | (nibbles[:, 1::2] << 4)


def int4_dequantize(codes: torch.Tensor, scales: torch.Tensor, group_width: int) -> torch.Tensor:
    """The weight the linear multiplies with: bf16(code * scale)
    (tests/cuda_ops_tests.cu:824-843)."""
    per_element = scales.t().repeat_interleave(group_width, dim=1)
    return bf16(codes.float() * per_element)


def int4_bf16_linear(x, codes, scales, group_width: int) -> torch.Tensor:
    """Int4Bf16Linear::run (include/carat/linear.h:70-90): bf16(X . W^T) over the dequantised
    weights, fp32 accumulation."""
    return bf16_linear(x, int4_dequantize(codes, scales, group_width))


def argmax_lowest_index(values: torch.Tensor) -> torch.Tensor:
    """cuda/ops.cu:890-981: maximum with ties to the lowest index (rows of bf16 logits)."""
    maximum = values.max(dim=-1, keepdim=True).values
    width = values.shape[-1]
    index = torch.arange(width).expand_as(values)
    return torch.where(values == maximum, index, torch.full_like(index, width)).min(dim=-1).values.to(
        torch.int32)


# --------------------------------------------------------------------------- RoPE and QKV post
def rope_tables(positions: int, head_dim: int, theta: float, proportional: bool):
    """cuda/qkv.cu:44-64: bf16 cos/sin of position * theta^(-2i/D); global layers keep only the first
    D/8 frequencies (the rest are angle 0). Returns [positions, head_dim] tables, both halves equal."""
    half = head_dim // 2
    index = torch.arange(half, dtype=torch.float32)
    frequency = torch.pow(f32(theta), f32(-2.0) * index / f32(float(head_dim)))
    if proportional:
        frequency = torch.where(index < head_dim // 8, frequency, torch.zeros_like(frequency))
    angle = torch.arange(positions, dtype=torch.float32)[:, None] * frequency[None, :]
    cos = bf16(torch.cos(angle))
    sin = bf16(torch.sin(angle))
    return torch.cat([cos, cos], dim=1), torch.cat([sin, sin], dim=1)


def norm_rope(x: torch.Tensor, weight: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
              eps: float) -> torch.Tensor:
    """cuda/qkv.cu:387-422: per-head bf16(norm*w), then bf16(n*cos + rotate_half(n)*sin).
    x: [rows, heads, D]; cos/sin: [rows, D]."""
    normalized = rms_norm(x, weight, eps)
    half = x.shape[-1] // 2
    rotated = torch.cat([-normalized[..., half:], normalized[..., :half]], dim=-1)
    return bf16(normalized * cos[:, None, :] + rotated * sin[:, None, :])


# --------------------------------------------------------------------------- verify attention
def verify_attention(queries, old_keys, old_values, new_keys, new_values, positions, window):
    """Attention of `depth` proposal rows per request over that request's cache plus the proposals.

    queries [requests, depth, Hq, D]; old_keys/old_values: per request [Hkv, capacity, D] holding
    logical position p in physical row p % capacity (cuda/qkv.cu:509); new_keys/new_values
    [requests, depth, Hkv, D]; positions[request] = first proposal's logical position;
    window = 0 for global (causal) layers, else the sliding window (keys p-window+1 .. p).

    Follows cuda/prefill_gemm_attention.cu:165-349,552-730: query t sees proposals 0..t, the
    pre-write rows of later proposal slots and the untouched remainder; scale 1.0; scores rounded
    to bf16; fp32 max/exp/sum; probabilities rounded to bf16; fp32 PV rounded to bf16 once.
    Returns [requests, depth, Hq, D]."""
    requests, depth, heads, dim = queries.shape
    kv_heads = new_keys.shape[2]
    group = heads // kv_heads
    output = torch.zeros(requests, depth, heads, dim)
    for request in range(requests):
        position = positions[request]
        capacity = old_keys[request].shape[1]
        for t in range(depth):
            query_position = position + t
            first = max(0, query_position - (window - 1)) if window > 0 else 0
            physical = [p % capacity for p in range(first, position)]
            k_ctx = torch.cat([old_keys[request][:, physical, :],
                               new_keys[request, : t + 1].transpose(0, 1)], dim=1)
            v_ctx = torch.cat([old_values[request][:, physical, :],
                               new_values[request, : t + 1].transpose(0, 1)], dim=1)
            q = queries[request, t].reshape(kv_heads, group, dim)
            scores = bf16(torch.einsum("hgd,hkd->hgk", q, k_ctx))
            maximum = scores.max(dim=-1, keepdim=True).values
            exponent = torch.exp(scores - maximum)
            probabilities = bf16(exponent * (f32(1.0) / exponent.sum(dim=-1, keepdim=True)))
            output[request, t] = bf16(torch.einsum("hgk,hkd->hgd", probabilities,
                                                   v_ctx)).reshape(heads, dim)
    return output


# --------------------------------------------------------------------------- weights
def random_weights(config: ModelConfig, seed: int, std: float = 0.02,
                   norm_jitter: float = 0.0) -> Dict[str, torch.Tensor]:
    """Random-init weights under the reference's segment names (src/weight_plan.cpp:37-82):
    matrices N(0, std) rounded to bf16, norm weights 1 (+ optional jitter), layer scalar 1."""
    generator = torch.Generator().manual_seed(seed)

    def matrix(rows, cols):
        return bf16(torch.randn(rows, cols, generator=generator) * std)

    def norm(width):
        if norm_jitter == 0.0:
            return torch.ones(width)
        return bf16(1.0 + torch.randn(width, generator=generator) * norm_jitter)

    weights = {"token_embedding": matrix(config.vocab, config.hidden)}
    for index, layer in enumerate(config.layers):
        prefix = f"layer.{index}."
        weights[prefix + "input_norm"] = norm(config.hidden)
        weights[prefix + "q_norm"] = norm(layer.head_dim)
        weights[prefix + "k_norm"] = norm(layer.head_dim)
        weights[prefix + "qkv"] = matrix(layer.packed_width, config.hidden)
        weights[prefix + "o"] = matrix(config.hidden, layer.query_width)
        weights[prefix + "post_attention_norm"] = norm(config.hidden)
        weights[prefix + "pre_mlp_norm"] = norm(config.hidden)
        weights[prefix + "gate_up"] = matrix(2 * config.intermediate, config.hidden)
        weights[prefix + "down"] = matrix(config.hidden, config.intermediate)
        weights[prefix + "post_mlp_norm"] = norm(config.hidden)
        weights[prefix + "scalar"] = torch.ones(1)
    weights["final_norm"] = norm(config.hidden)
    return weights


def golden_tiny_weights(config: ModelConfig) -> Dict[str, torch.Tensor]:
    """Seed-0 weights with non-trivial norm weights and layer scalars, used by the committed
    Hugging Face fixture (tests/golden/make_hf_golden.py) and the tests that read it."""
    weights = random_weights(config, 0, norm_jitter=0.1)
    generator = torch.Generator().manual_seed(1234)
    for index, layer in enumerate(config.layers):
        weights[f"layer.{index}.scalar"] = bf16(0.5 + 0.5 * torch.rand(1, generator=generator))
        # With unit q/k norm weights a random-init model has |q||k| = head_dim and attention logits
        # so large that bf16 rounding of the scores decides the output; trained checkpoints do not
        # behave like that. Scale the norms so logits have a standard deviation near one.
        for name in ("q_norm", "k_norm"):
            weights[f"layer.{index}.{name}"] = bf16(
                0.35 + 0.035 * torch.randn(layer.head_dim, generator=generator))
    return weights


def random_assistant_weights(config: ModelConfig, assistant: AssistantConfig, seed: int,
                             std: float = 0.02) -> Dict[str, torch.Tensor]:
    """Drafter segments (src/weight_plan.cpp:84-128)."""
    generator = torch.Generator().manual_seed(seed)

    def matrix(rows, cols):
        return bf16(torch.randn(rows, cols, generator=generator) * std)

    hidden = assistant.hidden
    weights = {
        "token_embedding": matrix(config.vocab, hidden),
        "pre_projection": matrix(hidden, 2 * config.hidden),
        "post_projection": matrix(config.hidden, hidden),
    }
    for index, kind in enumerate(assistant.layers):
        head_dim = shared_layer(config, kind)[1].head_dim
        query = assistant.query_heads * head_dim
        prefix = f"layer.{index}."
        weights[prefix + "input_norm"] = torch.ones(hidden)
        weights[prefix + "q_norm"] = torch.ones(head_dim)
        weights[prefix + "q"] = matrix(query, hidden)
        weights[prefix + "o"] = matrix(hidden, query)
        weights[prefix + "post_attention_norm"] = torch.ones(hidden)
        weights[prefix + "pre_mlp_norm"] = torch.ones(hidden)
        weights[prefix + "gate_up"] = matrix(2 * assistant.intermediate, hidden)
        weights[prefix + "down"] = matrix(hidden, assistant.intermediate)
        weights[prefix + "post_mlp_norm"] = torch.ones(hidden)
        weights[prefix + "scalar"] = torch.ones(1)
    weights["final_norm"] = torch.ones(hidden)
    return weights


def quantize_weights(weights: Dict[str, torch.Tensor]):
    """cuda/device_weights.cu:200-263: every 2-D segment gets e4m3 bytes + one fp32 scale."""
    return {name: quantize_e4m3(value) for name, value in weights.items() if value.dim() == 2}


def shared_layer(config: ModelConfig, kind: str) -> Tuple[int, LayerConfig]:
    """The drafter reads the target's last layer of each kind (cuda/batch_model_runner.cu:560-566)."""
    for index in range(len(config.layers) - 1, -1, -1):
        if config.layers[index].kind == kind:
            return index, config.layers[index]
    raise ValueError(f"target has no {kind} layer")


# --------------------------------------------------------------------------- the runner
@dataclass
class VerifyTrace:
    """Intermediate values of one verify call, kept for kernel-level parity tests."""

    final_hidden: torch.Tensor  # [rows, hidden] after final norm
    logits: torch.Tensor  # [rows, vocab] bf16 logits
    predictions: torch.Tensor  # [rows] int32
    top2_margin: torch.Tensor  # [rows] float32, top-1 minus top-2 logit
    layer_outputs: List[torch.Tensor] = field(default_factory=list)


class OracleRunner:
    """Slots, KV arenas and the verify / draft entry points of Gemma4BatchModelRunner
    (include/carat/batch_model_runner.h:22-77), restated on CPU."""

    def __init__(self, config: ModelConfig, weights, slots: int,
                 assistant: Optional[AssistantConfig] = None, assistant_weights=None,
                 fp8: bool = True, assistant_fp8: bool = True):
        self.config = config
        self.weights = weights
        self.fp8 = fp8
        self.fp8_weights = quantize_weights(weights) if fp8 else None
        self.slots = slots
        self.positions = [0] * slots
        # KV arenas: per layer [slot, kv_head, capacity, D], zero-filled
        # (cuda/batch_model_runner.cu:330-342,574-577,608-622).
        self.keys = []
        self.values = []
        for index, layer in enumerate(config.layers):
            shape = (slots, layer.kv_heads, config.capacity(index), layer.head_dim)
            self.keys.append(torch.zeros(shape))
            self.values.append(torch.zeros(shape))
        self.rope = {}
        for layer in config.layers:
            key = (layer.kind, layer.head_dim)
            if key not in self.rope:
                self.rope[key] = rope_tables(config.max_context, layer.head_dim, layer.rope_theta,
                                             layer.kind == "global")
        self.target_hidden = torch.zeros(slots, config.hidden)
        self.assistant = assistant
        self.assistant_weights = assistant_weights
        self.assistant_fp8 = assistant_fp8
        self.assistant_fp8_weights = (quantize_weights(assistant_weights)
                                      if assistant is not None and assistant_fp8 else None)

    def use_int4_mlp(self, group_width: int = 128):
        """The target's gate_up and down projections become weight-only INT4 linears over bf16
        activations (quantiser rule of cuda/int4_bf16_linear.cu:95-136 at the given group width;
        the reference itself has this linear but never selects it for the MLP, so this variant is
        defined here: no e4m3 quantisation of pre_mlp / activated, everything else unchanged)."""
        self.int4_group = group_width
        self.int4_weights = {}
        for index in range(len(self.config.layers)):
            for name in (f"layer.{index}.gate_up", f"layer.{index}.down"):
                self.int4_weights[name] = int4_quantize(self.weights[name], group_width)

    # ---- linears
    def _linear(self, x, name, weights=None, fp8_weights=None, use_fp8=None):
        if (weights is None or weights is self.weights) and name in getattr(self, "int4_weights", {}):
            codes, scales = self.int4_weights[name]
            return int4_bf16_linear(x, codes, scales, self.int4_group)
        weights = self.weights if weights is None else weights
        fp8_weights = self.fp8_weights if fp8_weights is None else fp8_weights
        use_fp8 = self.fp8 if use_fp8 is None else use_fp8
        if not use_fp8:
            return bf16_linear(x, weights[name])
        xq, x_scale = quantize_e4m3(x)
        wq, w_scale = fp8_weights[name]
        return fp8_linear(xq, x_scale, wq, w_scale)

    # ---- one verify layer (cuda/layer_runner.cu:730-1041 run_prefill_chunks, uniform FP8 path)
    def _verify_layer(self, index, hidden, slots, positions, depth):
        config = self.config
        layer = config.layers[index]
        prefix = f"layer.{index}."
        w = self.weights
        rows = hidden.shape[0]
        heads, kv_heads, dim = layer.query_heads, layer.kv_heads, layer.head_dim
        capacity = config.capacity(index)
        # run_qkv_projection (cuda/layer_runner.cu:241-262)
        normalized = rms_norm(hidden, w[prefix + "input_norm"], config.eps)
        packed = self._linear(normalized, prefix + "qkv")
        row_positions = torch.tensor([positions[r // depth] + r % depth for r in range(rows)])
        cos, sin = self.rope[(layer.kind, dim)]
        cos, sin = cos[row_positions], sin[row_positions]
        # run_prefill_uniform_direct (cuda/qkv.cu:387-422,477-530)
        q_raw = packed[:, :layer.query_width].reshape(rows, heads, dim)
        k_raw = packed[:, layer.query_width:layer.query_width + layer.kv_width].reshape(
            rows, kv_heads, dim)
        if layer.key_equals_value:
            v_raw = k_raw
        else:
            v_raw = packed[:, layer.query_width + layer.kv_width:].reshape(rows, kv_heads, dim)
        queries = norm_rope(q_raw, w[prefix + "q_norm"], cos, sin, config.eps)
        new_keys = norm_rope(k_raw, w[prefix + "k_norm"], cos, sin, config.eps)
        new_values = rms_norm(v_raw, None, config.eps)
        window = config.window if layer.kind == "sliding" else 0
        attention = verify_attention(
            queries.reshape(len(slots), depth, heads, dim),
            [self.keys[index][slot] for slot in slots], [self.values[index][slot] for slot in slots],
            new_keys.reshape(len(slots), depth, kv_heads, dim),
            new_values.reshape(len(slots), depth, kv_heads, dim), positions, window)
        attention = attention.reshape(rows, heads, dim)
        hidden_out = self._project(index, hidden, attention.reshape(rows, heads * dim))
        return hidden_out, new_keys, new_values

    def _project(self, index, residual, attention_states, weights=None, fp8_weights=None,
                 use_fp8=None, intermediate=None, eps=None):
        """cuda/layer_runner.cu:264-354 Implementation::project."""
        w = self.weights if weights is None else weights
        intermediate = self.config.intermediate if intermediate is None else intermediate
        eps = self.config.eps if eps is None else eps
        prefix = f"layer.{index}."
        projected = self._linear(attention_states, prefix + "o", w, fp8_weights, use_fp8)
        first, pre_mlp = rms_norm_add_and_norm(projected, w[prefix + "post_attention_norm"],
                                               residual, w[prefix + "pre_mlp_norm"], eps)
        gate_up = self._linear(pre_mlp, prefix + "gate_up", w, fp8_weights, use_fp8)
        activated = gelu_tanh_gate(gate_up, intermediate)
        down = self._linear(activated, prefix + "down", w, fp8_weights, use_fp8)
        return rms_norm_add_scale(down, w[prefix + "post_mlp_norm"], first, w[prefix + "scalar"],
                                  eps)

    # ---- verify (cuda/batch_model_runner.cu:1617-1810)
    def verify_greedy_proposals(self, proposals: Sequence[Sequence[int]],
                                target_first_tokens: Sequence[int], slots: Sequence[int],
                                maximum_accepted_tokens: Sequence[int] = (),
                                assume_match: bool = False, trace: bool = False,
                                allow_empty_slot: bool = False):
        config = self.config
        requests = len(proposals)
        depth = len(proposals[0]) if requests else 0
        if (requests <= 0 or requests > self.slots or depth <= 0
                or len(target_first_tokens) != requests or len(slots) != requests):
            raise RuntimeError("invalid greedy verification batch")
        if maximum_accepted_tokens and len(maximum_accepted_tokens) != requests:
            raise RuntimeError("speculative acceptance caps do not match request count")
        seen = set()
        positions = []
        for request in range(requests):
            slot = slots[request]
            if slot < 0 or slot >= self.slots or slot in seen or len(proposals[request]) != depth:
                raise RuntimeError("invalid or repeated speculative slot")
            seen.add(slot)
            position = self.positions[slot]
            if (position <= 0 and not allow_empty_slot) or position + depth > config.max_context:
                raise RuntimeError("speculative slot is empty or lacks context capacity")
            positions.append(position)
            for token in proposals[request]:
                if token < 0 or token >= config.vocab:
                    raise RuntimeError("speculative proposal contains an invalid token")
        tokens = torch.tensor([t for row in proposals for t in row], dtype=torch.int64)
        hidden = embedding(self.weights["token_embedding"], tokens, config.hidden)
        staged = []
        layer_outputs = []
        for index in range(len(config.layers)):
            hidden, new_keys, new_values = self._verify_layer(index, hidden, slots, positions, depth)
            staged.append((new_keys, new_values))
            if trace:
                layer_outputs.append(hidden.clone())
        final_hidden = rms_norm(hidden, self.weights["final_norm"], config.eps)
        # run_decode_lm_head (cuda/batch_model_runner.cu:840-853): tied embedding as LM head.
        logits = self._linear(final_hidden, "token_embedding")
        predictions = argmax_lowest_index(logits)
        accepted, next_tokens = greedy_prefix_accept(
            [list(row) for row in proposals], list(target_first_tokens), predictions.tolist(),
            list(maximum_accepted_tokens), depth, assume_match)
        # Commit: rows t < accepted become resident; rows t >= accepted leave the ring exactly as
        # it was (cuda/ops.cu:849-871); global rows beyond the new position are unreachable.
        for index, layer in enumerate(config.layers):
            capacity = config.capacity(index)
            new_keys, new_values = staged[index]
            for request, slot in enumerate(slots):
                limit = accepted[request] if layer.kind == "sliding" else depth
                for t in range(limit):
                    row = (positions[request] + t) % capacity
                    self.keys[index][slot][:, row, :] = new_keys[request * depth + t]
                    self.values[index][slot][:, row, :] = new_values[request * depth + t]
        for request, slot in enumerate(slots):
            if accepted[request] > 0:
                # cuda/batch_model_runner.cu:1761-1783: final-normed row (accepted-1) -> slot table.
                self.target_hidden[slot] = final_hidden[request * depth + accepted[request] - 1]
            self.positions[slot] += accepted[request]
        if trace:
            top2 = torch.topk(logits, 2, dim=-1).values
            return accepted, next_tokens, VerifyTrace(final_hidden, logits, predictions,
                                                      top2[:, 0] - top2[:, 1], layer_outputs)
        return accepted, next_tokens

    # ---- drafter (cuda/assistant_runner.cu:162-338, cuda/batch_model_runner.cu:1812-1836)
    def draft(self, last_tokens: Sequence[int], slots: Sequence[int],
              forced_first_tokens: Sequence[int] = (), depth: int = 4, trace: bool = False):
        if self.assistant is None or len(last_tokens) != len(slots) or not last_tokens:
            raise RuntimeError("assistant is not configured or draft batch is invalid")
        if forced_first_tokens and len(forced_first_tokens) != len(last_tokens):
            raise RuntimeError("forced assistant first tokens do not match draft batch")
        config, assistant, w = self.config, self.assistant, self.assistant_weights
        context_positions = []
        for slot in slots:
            if slot < 0 or slot >= self.slots or self.positions[slot] <= 0:
                raise RuntimeError("assistant slot is empty or invalid")
            context_positions.append(self.positions[slot] - 1)
        active = len(slots)
        previous_hidden = self.target_hidden[list(slots)].clone()
        tokens = torch.tensor(list(last_tokens), dtype=torch.int64)
        proposals = [[0] * depth for _ in range(active)]
        traces = []

        def linear(x, name):
            return self._linear(x, name, w, self.assistant_fp8_weights, self.assistant_fp8)

        for draft_index in range(depth):
            emb = embedding(self.weights["token_embedding"], tokens, config.hidden)
            hidden = linear(torch.cat([emb, previous_hidden], dim=1), "pre_projection")
            for index, kind in enumerate(assistant.layers):
                shared_index, shared = shared_layer(config, kind)
                capacity = config.capacity(shared_index)
                dim, kv_heads = shared.head_dim, shared.kv_heads
                heads = assistant.query_heads
                group = heads // kv_heads
                prefix = f"layer.{index}."
                normalized = rms_norm(hidden, w[prefix + "input_norm"], assistant.eps)
                projected = linear(normalized, prefix + "q").reshape(active, heads, dim)
                cos, sin = self.rope[(kind, dim)]
                query_positions = torch.tensor([p + draft_index for p in context_positions])
                queries = norm_rope(projected, w[prefix + "q_norm"], cos[query_positions],
                                    sin[query_positions], assistant.eps)
                attention = torch.zeros(active, heads, dim)
                for row, slot in enumerate(slots):
                    # cuda/gemm_attention.cu:88-132: the first min(position+1, capacity) physical
                    # rows are valid; the key set does not change across draft steps.
                    valid = min(context_positions[row] + 1, capacity)
                    k_ctx = self.keys[shared_index][slot][:, :valid, :]
                    v_ctx = self.values[shared_index][slot][:, :valid, :]
                    q = queries[row].reshape(kv_heads, group, dim)
                    scores = bf16(torch.einsum("hgd,hkd->hgk", q, k_ctx))
                    maximum = scores.max(dim=-1, keepdim=True).values
                    exponent = torch.exp(scores - maximum)
                    probabilities = bf16(exponent * (f32(1.0) / exponent.sum(dim=-1, keepdim=True)))
                    attention[row] = bf16(torch.einsum("hgk,hkd->hgd", probabilities,
                                                       v_ctx)).reshape(heads, dim)
                hidden = self._project(index, hidden, attention.reshape(active, heads * dim), w,
                                       self.assistant_fp8_weights, self.assistant_fp8,
                                       assistant.intermediate, assistant.eps)
            final_hidden = rms_norm(hidden, w["final_norm"], assistant.eps)
            margin = None
            if draft_index == 0 and forced_first_tokens:
                tokens = torch.tensor(list(forced_first_tokens), dtype=torch.int64)
            else:
                logits = linear(final_hidden, "token_embedding")
                tokens = argmax_lowest_index(logits).long()
                top2 = torch.topk(logits, 2, dim=-1).values
                margin = top2[:, 0] - top2[:, 1]
            previous_hidden = linear(final_hidden, "post_projection")
            traces.append((final_hidden, previous_hidden, margin))
            for row in range(active):
                proposals[row][draft_index] = int(tokens[row])
        if trace:
            return proposals, traces
        return proposals

    def prefill_slot_fp8(self, slot: int, tokens: Sequence[int], chunk: int = 8) -> int:
        """Makes `tokens` resident in `slot` by running them through the FP8 verify forward in
        chunks with every row accepted, and returns the greedy next token. (The reference prefills
        in BF16, cuda/batch_model_runner.cu:1274-1275; this interim form only has to build the same
        state on both sides of a parity test.)"""
        next_token = -1
        for start in range(0, len(tokens), chunk):
            part = list(tokens[start:start + chunk])
            _, next_tokens = self.verify_greedy_proposals([part], [part[0]], [slot],
                                                          assume_match=True, allow_empty_slot=True)
            next_token = next_tokens[0]
        return next_token

    def append_ragged(self, token_ids: Sequence[int], slots: Sequence[int]) -> List[int]:
        """Plain decode, one token per listed slot (cuda/batch_model_runner.cu:1544-1615): the
        token becomes resident at the slot's position, the position advances by one, and the
        greedy next token comes back. The forward is the verify forward with one row per slot
        (same norms, tensor-scale e4m3 linears, ring attention and tied LM head; the reference's
        decode kernels differ from its verify kernels only in launch shape), so it is restated
        as a depth-1 verification whose single proposal is the forced token itself."""
        active = len(token_ids)
        if active <= 0 or active > self.slots or len(slots) != active:
            raise RuntimeError("invalid ragged token batch")
        seen = set()
        for token, slot in zip(token_ids, slots):
            if (slot < 0 or slot >= self.slots or slot in seen or token < 0
                    or token >= self.config.vocab):
                raise RuntimeError("invalid or repeated ragged slot")
            seen.add(slot)
            if self.positions[slot] <= 0 or self.positions[slot] >= self.config.max_context:
                raise RuntimeError("ragged slot is empty or full")
        _, next_tokens = self.verify_greedy_proposals([[token] for token in token_ids],
                                                      list(token_ids), list(slots))
        return next_tokens

    def clone_slot(self, source_slot: int, destination_slot: int) -> int:
        """cuda/batch_model_runner.cu:1507-1542: resident KV rows, hand-off hidden row and position
        of one slot copied to another; returns the KV bytes copied."""
        if (source_slot < 0 or source_slot >= self.slots or destination_slot < 0
                or destination_slot >= self.slots or source_slot == destination_slot):
            raise RuntimeError("invalid cache slot clone")
        position = self.positions[source_slot]
        if position <= 0 or position >= self.config.max_context:
            raise RuntimeError("source cache slot is empty or full")
        copied = 0
        for index, layer in enumerate(self.config.layers):
            resident = min(position, self.config.capacity(index))
            for cache in (self.keys[index], self.values[index]):
                cache[destination_slot][:, :resident, :] = cache[source_slot][:, :resident, :]
                copied += 2 * resident * layer.kv_width
        self.target_hidden[destination_slot] = self.target_hidden[source_slot]
        self.positions[destination_slot] = position
        return copied

    def seed_empty_cache_for_benchmark(self, position: int):
        """cuda/batch_model_runner.cu seed_empty_cache_for_benchmark: zero KV, advance positions."""
        for index in range(len(self.config.layers)):
            self.keys[index].zero_()
            self.values[index].zero_()
        self.positions = [position] * self.slots


# --------------------------------------------------------------------------- integer logic
def greedy_prefix_accept(proposals: List[List[int]], target_first: List[int],
                         predictions: List[int], caps: List[int], depth: int,
                         assume_match: bool = False) -> Tuple[List[int], List[int]]:
    """cuda/batch_model_runner.cu:1735-1759. predictions is row-major [request * depth + t].
    assume_match (not in the reference) treats every proposal as matching, so the cap alone sets
    the accepted length; throughput runs use it to inject accept lengths."""
    accepted_tokens, next_tokens = [], []
    for request, row in enumerate(proposals):
        cap = depth if not caps else max(0, min(caps[request], depth))
        accepted = 0
        start = request * depth
        while accepted < cap:
            expected = target_first[request] if accepted == 0 else predictions[start + accepted - 1]
            if not assume_match and row[accepted] != expected:
                break
            accepted += 1
        accepted_tokens.append(accepted)
        next_tokens.append(target_first[request] if accepted == 0
                           else predictions[start + accepted - 1])
    return accepted_tokens, next_tokens


def acceptance_cap(depth: int, remaining: int, proposals: Sequence[int], stop_ids) -> int:
    """src/runtime/speculation.cpp:7-18."""
    cap = min(depth, remaining)
    inspected = min(cap, len(proposals))
    for index in range(1, inspected):
        if proposals[index] in stop_ids:
            return index + 1
    return cap


def commit_speculation(forced_token: int, accepted_drafts: Sequence[int], next_token: int,
                       stop_ids):
    """src/runtime/speculation.cpp:20-36. Returns (resident, emitted, next_token, stopped)."""
    resident, emitted = [forced_token], []
    for token in accepted_drafts:
        resident.append(token)
        emitted.append(token)
        if token in stop_ids:
            return resident, emitted, next_token, True
    emitted.append(next_token)
    return resident, emitted, next_token, False


def backup_kv_ring_spans(keys, values, positions, depth):
    """cuda/ops.cu:827-847: backup[req, head, t, :] = cache[req][head, (pos+t) % cap, :]."""
    capacity = keys[0].shape[1]
    rows = [[(p + t) % capacity for t in range(depth)] for p in positions]
    backup_k = torch.stack([keys[r][:, rows[r], :] for r in range(len(positions))])
    backup_v = torch.stack([values[r][:, rows[r], :] for r in range(len(positions))])
    return backup_k, backup_v


def restore_kv_ring_suffixes(backup_k, backup_v, keys, values, positions, accepted, depth):
    """cuda/ops.cu:849-871: rows t >= accepted[req] get their saved contents back."""
    capacity = keys[0].shape[1]
    for request, position in enumerate(positions):
        for t in range(accepted[request], depth):
            row = (position + t) % capacity
            keys[request][:, row, :] = backup_k[request][:, t, :]
            values[request][:, row, :] = backup_v[request][:, t, :]
