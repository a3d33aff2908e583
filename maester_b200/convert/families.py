"""Conversion tables of the supported model families and their architecture descriptors.

Key names on the native side are the models' parameter FQNs (the keys under ``"model"`` in a DCP
checkpoint).  Reference key maps: scripts/convert/llama/to_dcp.py:30-44, gemma/to_dcp.py:142-248,
deepseek/to_dcp.py:158-235, glm4/to_dcp.py:100-180.
"""
from __future__ import annotations

from maester_b200.convert.rules import (
    FamilySpec, Fuse, Rule, Stack, rope_rows_half_to_interleaved, rope_rows_interleaved_to_half,
)

_L = "model.layers.{L}."

# ------------------------------------------------------------------------------------------ Llama / Mistral
LLAMA = FamilySpec(
    name="llama",
    entries=[
        Rule("model.embed_tokens.weight", "tok_embeddings.weight"),
        Rule(_L + "self_attn.q_proj.weight", "layers.{L}.attention.wq.weight",
             rope_rows_half_to_interleaved("n_heads"), rope_rows_interleaved_to_half("n_heads")),
        Rule(_L + "self_attn.k_proj.weight", "layers.{L}.attention.wk.weight",
             rope_rows_half_to_interleaved("n_kv_heads"), rope_rows_interleaved_to_half("n_kv_heads")),
        Rule(_L + "self_attn.v_proj.weight", "layers.{L}.attention.wv.weight"),
        Rule(_L + "self_attn.o_proj.weight", "layers.{L}.attention.wo.weight"),
        Rule(_L + "self_attn.rotary_emb.inv_freq", None),
        Rule(_L + "mlp.gate_proj.weight", "layers.{L}.feed_forward.w1.weight"),
        Rule(_L + "mlp.up_proj.weight", "layers.{L}.feed_forward.w3.weight"),
        Rule(_L + "mlp.down_proj.weight", "layers.{L}.feed_forward.w2.weight"),
        Rule(_L + "input_layernorm.weight", "layers.{L}.attention_norm.weight"),
        Rule(_L + "post_attention_layernorm.weight", "layers.{L}.ffn_norm.weight"),
        Rule("model.norm.weight", "norm.weight"),
        Rule("lm_head.weight", "output.weight"),
    ],
)


# ------------------------------------------------------------------------------------------ Gemma 3 (text)
def _gemma_qkv_sizes(arch):
    return [arch["n_heads"] * arch["head_dim"], arch["n_kv_heads"] * arch["head_dim"],
            arch["n_kv_heads"] * arch["head_dim"]]


GEMMA = FamilySpec(
    name="gemma",
    # multimodal checkpoints nest the text model; vision tower and projector are not converted
    strip_prefixes=("model.language_model.", "language_model.model.", "language_model."),
    ignore=(r"^(model\.)?vision_tower\.", r"^(model\.)?multi_modal_projector\.", r"^lm_head\.weight$",
            r"^model\.vision_tower\.", r"rotary_emb\.inv_freq$"),
    entries=[
        Rule("model.embed_tokens.weight", "tok_embeddings.weight"),
        Rule("embed_tokens.weight", "tok_embeddings.weight"),
        Fuse([_L + "self_attn.q_proj.weight", _L + "self_attn.k_proj.weight", _L + "self_attn.v_proj.weight"],
             _L + "self_attn.qkv_proj.weight", _gemma_qkv_sizes),
        Rule(_L + "self_attn.o_proj.weight", _L + "self_attn.o_proj.weight"),
        Rule(_L + "self_attn.q_norm.weight", _L + "self_attn.query_norm.weight"),
        Rule(_L + "self_attn.k_norm.weight", _L + "self_attn.key_norm.weight"),
        Rule(_L + "mlp.gate_proj.weight", _L + "mlp.gate_proj.weight"),
        Rule(_L + "mlp.up_proj.weight", _L + "mlp.up_proj.weight"),
        Rule(_L + "mlp.down_proj.weight", _L + "mlp.down_proj.weight"),
        Rule(_L + "input_layernorm.weight", _L + "input_layernorm.weight"),
        Rule(_L + "post_attention_layernorm.weight", _L + "post_attention_layernorm.weight"),
        Rule(_L + "pre_feedforward_layernorm.weight", _L + "pre_feedforward_layernorm.weight"),
        Rule(_L + "post_feedforward_layernorm.weight", _L + "post_feedforward_layernorm.weight"),
        Rule("model.norm.weight", "model.norm.weight"),
    ],
)
# a stripped multimodal key loses its "model." prefix: accept both spellings on import
GEMMA.entries.extend([])


# ------------------------------------------------------------------------------------------ DeepSeek V2/V3
def _moe_entries(hf_layer: str, native_layer: str) -> list:
    return [
        Rule(hf_layer + "mlp.gate.weight", native_layer + "moe.router.gate.weight"),
        Rule(hf_layer + "mlp.gate.e_score_correction_bias", native_layer + "moe.expert_bias"),
        Rule(hf_layer + "mlp.shared_experts.gate_proj.weight", native_layer + "moe.shared_experts.w1.weight"),
        Rule(hf_layer + "mlp.shared_experts.up_proj.weight", native_layer + "moe.shared_experts.w3.weight"),
        Rule(hf_layer + "mlp.shared_experts.down_proj.weight", native_layer + "moe.shared_experts.w2.weight"),
        Stack(hf_layer + "mlp.experts.{E}.gate_proj.weight", native_layer + "moe.experts.w1"),
        Stack(hf_layer + "mlp.experts.{E}.up_proj.weight", native_layer + "moe.experts.w3"),
        Stack(hf_layer + "mlp.experts.{E}.down_proj.weight", native_layer + "moe.experts.w2"),
    ]


DEEPSEEK = FamilySpec(
    name="deepseek",
    ignore=(r"rotary_emb\.inv_freq$", r"^model\.layers\.\d+\.(embed_tokens|enorm|hnorm|eh_proj|shared_head)\."),
    entries=[
        Rule("model.embed_tokens.weight", "tok_embeddings.weight"),
        Rule("model.norm.weight", "norm.weight"),
        Rule("lm_head.weight", "output.weight"),
        Rule(_L + "self_attn.q_proj.weight", "layers.{L}.attention.wq.weight"),
        Rule(_L + "self_attn.q_a_proj.weight", "layers.{L}.attention.wq_a.weight"),
        Rule(_L + "self_attn.q_a_layernorm.weight", "layers.{L}.attention.q_norm.weight"),
        Rule(_L + "self_attn.q_b_proj.weight", "layers.{L}.attention.wq_b.weight"),
        Rule(_L + "self_attn.kv_a_proj_with_mqa.weight", "layers.{L}.attention.wkv_a.weight"),
        Rule(_L + "self_attn.kv_a_layernorm.weight", "layers.{L}.attention.kv_norm.weight"),
        Rule(_L + "self_attn.kv_b_proj.weight", "layers.{L}.attention.wkv_b.weight"),
        Rule(_L + "self_attn.o_proj.weight", "layers.{L}.attention.wo.weight"),
        Rule(_L + "mlp.gate_proj.weight", "layers.{L}.feed_forward.w1.weight"),
        Rule(_L + "mlp.up_proj.weight", "layers.{L}.feed_forward.w3.weight"),
        Rule(_L + "mlp.down_proj.weight", "layers.{L}.feed_forward.w2.weight"),
        Rule(_L + "input_layernorm.weight", "layers.{L}.attention_norm.weight"),
        Rule(_L + "post_attention_layernorm.weight", "layers.{L}.ffn_norm.weight"),
        *_moe_entries(_L, "layers.{L}."),
    ],
)

# ------------------------------------------------------------------------------------------ GLM-4.5 (MoE)
GLM4 = FamilySpec(
    name="glm4",
    ignore=(r"rotary_emb\.inv_freq$",),
    entries=[
        Rule("model.embed_tokens.weight", "tok_embeddings.weight"),
        Rule("model.norm.weight", "norm.weight"),
        Rule("lm_head.weight", "output.weight"),
        *[Rule(_L + f"self_attn.{p}_proj.{kind}", "layers.{L}." + f"self_attn.{p}_proj.{kind}")
          for p in ("q", "k", "v", "o") for kind in ("weight", "bias")],
        Rule(_L + "self_attn.q_norm.weight", "layers.{L}.self_attn.q_norm.weight"),
        Rule(_L + "self_attn.k_norm.weight", "layers.{L}.self_attn.k_norm.weight"),
        Rule(_L + "input_layernorm.weight", "layers.{L}.input_layernorm.weight"),
        Rule(_L + "post_attention_layernorm.weight", "layers.{L}.post_attention_layernorm.weight"),
        Rule(_L + "mlp.gate_proj.weight", "layers.{L}.mlp.gate_proj.weight"),
        Rule(_L + "mlp.up_proj.weight", "layers.{L}.mlp.up_proj.weight"),
        Rule(_L + "mlp.down_proj.weight", "layers.{L}.mlp.down_proj.weight"),
        *_moe_entries(_L, "layers.{L}."),
    ],
)

FAMILIES: dict[str, FamilySpec] = {
    "llama": LLAMA, "llama2": LLAMA, "llama3": LLAMA, "mistral": LLAMA,
    "gemma": GEMMA, "gemma3": GEMMA, "deepseek": DEEPSEEK, "glm4": GLM4,
}


# ---------------------------------------------------------------------------------------------------
def arch_from_hf_config(family: str, cfg: dict) -> dict:
    """Head counts and sizes the transforms need, from an HF ``config.json`` dict."""
    cfg = cfg.get("text_config", cfg)
    heads = cfg.get("num_attention_heads", 0)
    arch = {
        "n_heads": heads,
        "n_kv_heads": cfg.get("num_key_value_heads", heads),
        "dim": cfg.get("hidden_size", 0),
        "n_layers": cfg.get("num_hidden_layers", 0),
    }
    arch["head_dim"] = cfg.get("head_dim") or (arch["dim"] // heads if heads else 0)
    if FAMILIES[family] is LLAMA and cfg.get("rope_scaling"):
        raise ValueError("the checkpoint uses scaled RoPE, which the Llama model here does not implement")
    return arch


def arch_from_model_args(family: str, args) -> dict:
    """The same descriptor from a native ``ModelArgs``."""
    heads = args.n_heads
    kv = getattr(args, "n_kv_heads", None) or getattr(args, "num_key_value_heads", None) or heads
    hd = getattr(args, "head_dim", None) or args.dim // heads
    return {"n_heads": heads, "n_kv_heads": kv, "dim": args.dim, "n_layers": args.n_layers, "head_dim": hd}
