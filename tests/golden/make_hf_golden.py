"""Generates tests/golden/hf_tiny_bf16.npz: BF16 outputs of the Hugging Face Gemma4 text model (the
model the reference's fixture tools run, tools/generate_layer_fixture.py:57-86) on the tiny
plumbing configuration with the oracle's seed-0 random weights.

Run from the repository root in the build container (needs transformers with Gemma4):
    python tests/golden/make_hf_golden.py
The fixture pins the BF16 layer math of oracle/carat_semantics.py (norm placement, RoPE incl. the
proportional global variant, sliding-window and causal attention, GeGLU, residual/scalar order).
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import carat_semantics as cs  # noqa: E402

from transformers.models.gemma4.configuration_gemma4 import Gemma4TextConfig  # noqa: E402
from transformers.models.gemma4.modeling_gemma4 import Gemma4TextModel  # noqa: E402

TOKENS = 165  # longer than the 128-token window so the sliding mask is exercised
SEED = 0


def main():
    config = cs.tiny_config(512)
    weights = cs.golden_tiny_weights(config)
    hf_config = Gemma4TextConfig(
        vocab_size=config.vocab, hidden_size=config.hidden, intermediate_size=config.intermediate,
        num_hidden_layers=len(config.layers), num_attention_heads=4, num_key_value_heads=2,
        head_dim=64, global_head_dim=64, num_global_key_value_heads=2, attention_k_eq_v=True,
        sliding_window=config.window,
        layer_types=["sliding_attention" if l.kind == "sliding" else "full_attention"
                     for l in config.layers],
        rms_norm_eps=config.eps, hidden_size_per_layer_input=0, num_kv_shared_layers=0,
        max_position_embeddings=config.max_context, final_logit_softcapping=None,
        tie_word_embeddings=True, attention_bias=False,
        rope_parameters={
            "sliding_attention": {"rope_type": "default", "rope_theta": 10000.0},
            "full_attention": {"rope_type": "proportional", "partial_rotary_factor": 0.25,
                               "rope_theta": 1000000.0}})
    hf_config._attn_implementation = "eager"
    model = Gemma4TextModel(hf_config).eval()
    state = {"embed_tokens.weight": weights["token_embedding"], "norm.weight": weights["final_norm"]}
    names = {"input_norm": "input_layernorm.weight", "q_norm": "self_attn.q_norm.weight",
             "k_norm": "self_attn.k_norm.weight", "o": "self_attn.o_proj.weight",
             "post_attention_norm": "post_attention_layernorm.weight",
             "pre_mlp_norm": "pre_feedforward_layernorm.weight", "down": "mlp.down_proj.weight",
             "post_mlp_norm": "post_feedforward_layernorm.weight", "scalar": "layer_scalar"}
    for index, layer in enumerate(config.layers):
        prefix = f"layer.{index}."
        for ours, theirs in names.items():
            state[f"layers.{index}.{theirs}"] = weights[prefix + ours]
        qkv = weights[prefix + "qkv"]
        state[f"layers.{index}.self_attn.q_proj.weight"] = qkv[:layer.query_width]
        state[f"layers.{index}.self_attn.k_proj.weight"] = qkv[layer.query_width:
                                                               layer.query_width + layer.kv_width]
        if not layer.key_equals_value:
            state[f"layers.{index}.self_attn.v_proj.weight"] = qkv[layer.query_width + layer.kv_width:]
        gate_up = weights[prefix + "gate_up"]
        state[f"layers.{index}.mlp.gate_proj.weight"] = gate_up[:config.intermediate]
        state[f"layers.{index}.mlp.up_proj.weight"] = gate_up[config.intermediate:]
    missing, unexpected = model.load_state_dict(state, strict=False)
    missing = [name for name in missing if "embed_scale" not in name]
    assert not missing and not unexpected, (missing, unexpected)
    model = model.to(torch.bfloat16)
    generator = torch.Generator().manual_seed(SEED)
    tokens = torch.randint(3, config.vocab, (TOKENS,), generator=generator)
    with torch.inference_mode():
        output = model(input_ids=tokens[None, :], use_cache=False)
        hidden = output.last_hidden_state[0].float()
        logits = (output.last_hidden_state[0] @ model.embed_tokens.weight.t()).float()
    np.savez_compressed(
        os.path.join(os.path.dirname(os.path.abspath(__file__)), "hf_tiny_bf16.npz"),
        tokens=tokens.numpy().astype(np.int32),
        final_hidden_tail=hidden[-8:].numpy().astype(np.float32),
        logits_tail_top=logits[-8:].topk(8, dim=-1).indices.numpy().astype(np.int32),
        logits_tail_values=logits[-8:].topk(8, dim=-1).values.numpy().astype(np.float32),
        note=np.array("transformers " + __import__("transformers").__version__))
    print("wrote fixture; last-row argmax", logits[-1].argmax().item())


if __name__ == "__main__":
    main()
