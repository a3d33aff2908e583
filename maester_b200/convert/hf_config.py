"""Hugging Face ``config.json`` contents for exported checkpoints, built from native model args.

The reference's ``from_dcp`` scripts recover the architecture from the training job's
``config.json`` and write an HF config next to the safetensors
(scripts/convert/gemma/from_dcp.py:147-190, llama/from_dcp.py).
"""
from __future__ import annotations


def _llama(a, mup: bool) -> dict:
    from maester_b200.models.llama.model import swiglu_hidden_dim
    kv = a.n_kv_heads or a.n_heads
    cfg = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "hidden_size": a.dim, "intermediate_size": swiglu_hidden_dim(a.dim, a.multiple_of, a.ffn_dim_multiplier),
        "num_hidden_layers": a.n_layers, "num_attention_heads": a.n_heads, "num_key_value_heads": kv,
        "head_dim": a.dim // a.n_heads, "vocab_size": a.vocab_size, "rms_norm_eps": a.norm_eps,
        "rope_theta": float(a.rope_theta), "max_position_embeddings": a.max_seq_len, "hidden_act": "silu",
        "tie_word_embeddings": bool(a.tied_embeddings), "attention_bias": False, "mlp_bias": False,
        "torch_dtype": "bfloat16",
    }
    if mup or a.enable_mup:
        cfg.update({"architectures": ["MupLlamaForCausalLM"], "model_type": "mup_llama",
                    "mup_input_alpha": a.mup_input_alpha, "mup_output_alpha": a.mup_output_alpha,
                    "mup_width_mul": a.mup_width_mul})
    return cfg


def _gemma(a) -> dict:
    types = a.attn_types or ["global"]
    layer_types = ["sliding_attention" if types[i % len(types)] == "local_sliding" else "full_attention"
                   for i in range(a.n_layers)]
    wl = a.rope_wave_length or {}
    cfg = {
        "architectures": ["Gemma3ForCausalLM"], "model_type": "gemma3_text",
        "hidden_size": a.dim, "intermediate_size": a.intermediate_size, "num_hidden_layers": a.n_layers,
        "num_attention_heads": a.n_heads, "num_key_value_heads": a.num_key_value_heads, "head_dim": a.head_dim,
        # the model was trained with the window INCLUSIVE of both ends (a query sees keys q-W .. q, W + 1 of them, as
        # the reference's mask does: maester/models/gemma/model.py:206-214); transformers counts the keys, so the
        # exported window is one larger and the exported model computes what was trained
        "vocab_size": a.vocab_size, "rms_norm_eps": a.rms_norm_eps, "sliding_window": a.sliding_window_size + 1,
        "layer_types": layer_types, "sliding_window_pattern": len(types),
        "query_pre_attn_scalar": a.query_pre_attn_scalar or a.head_dim,
        "rope_theta": float(wl.get("global", 1_000_000)), "rope_local_base_freq": float(wl.get("local_sliding", 10_000)),
        "max_position_embeddings": a.max_seq_len, "hidden_activation": "gelu_pytorch_tanh",
        "tie_word_embeddings": True, "attention_bias": False, "pad_token_id": a.pad_token_id,
        "bos_token_id": a.bos_token_id, "eos_token_id": a.eos_token_id, "torch_dtype": "bfloat16",
    }
    if a.rope_scaling:
        cfg["rope_scaling"] = {"rope_type": "linear", "factor": float(a.rope_scaling.get("factor", 1.0))}
    return cfg


def _deepseek(a) -> dict:
    m = a.moe_args
    v3 = m.score_func == "sigmoid"
    return {
        "architectures": ["DeepseekV3ForCausalLM" if v3 else "DeepseekV2ForCausalLM"],
        "model_type": "deepseek_v3" if v3 else "deepseek_v2",
        "hidden_size": a.dim, "intermediate_size": a.inter_dim, "moe_intermediate_size": a.moe_intermediate_size,
        "num_hidden_layers": a.n_layers, "first_k_dense_replace": a.n_dense_layers,
        "num_attention_heads": a.n_heads, "num_key_value_heads": a.n_heads, "vocab_size": a.vocab_size,
        "n_routed_experts": m.num_experts, "n_shared_experts": m.num_shared_experts,
        "num_experts_per_tok": m.top_k, "routed_scaling_factor": m.route_scale, "norm_topk_prob": m.route_norm,
        # one routing group holding every expert: this model family has no group-limited routing
        "n_group": 1, "topk_group": 1, "topk_method": "noaux_tc" if v3 else "greedy",
        "scoring_func": m.score_func, "q_lora_rank": a.q_lora_rank or None, "kv_lora_rank": a.kv_lora_rank,
        "qk_nope_head_dim": a.qk_nope_head_dim, "qk_rope_head_dim": a.qk_rope_head_dim, "v_head_dim": a.v_head_dim,
        "rms_norm_eps": a.norm_eps, "rope_theta": float(a.rope_theta), "max_position_embeddings": a.max_seq_len,
        "rope_scaling": ({"type": "yarn", "factor": float(a.rope_factor),
                          "original_max_position_embeddings": a.original_seq_len, "beta_fast": float(a.beta_fast),
                          "beta_slow": float(a.beta_slow), "mscale": a.mscale, "mscale_all_dim": a.mscale}
                         if a.max_seq_len > a.original_seq_len else None),
        "tie_word_embeddings": bool(a.tied_embeddings), "hidden_act": "silu", "torch_dtype": "bfloat16",
    }


def _glm4(a) -> dict:
    m = a.moe_args
    return {
        "architectures": ["Glm4MoeForCausalLM"], "model_type": "glm4_moe",
        "hidden_size": a.dim, "intermediate_size": a.intermediate_size, "moe_intermediate_size": a.moe_intermediate_size,
        "num_hidden_layers": a.n_layers, "first_k_dense_replace": a.first_k_dense_replace,
        "num_attention_heads": a.n_heads, "num_key_value_heads": a.n_kv_heads, "head_dim": a.head_dim,
        "partial_rotary_factor": a.partial_rotary_factor, "vocab_size": a.vocab_size,
        "n_routed_experts": m.num_experts, "n_shared_experts": m.num_shared_experts, "num_experts_per_tok": m.top_k,
        "routed_scaling_factor": m.route_scale, "norm_topk_prob": m.route_norm, "use_qk_norm": a.use_qk_norm,
        "attention_bias": a.attention_bias, "rms_norm_eps": a.rms_norm_eps, "rope_theta": float(a.rope_theta),
        "max_position_embeddings": a.max_position_embeddings, "hidden_act": a.hidden_act,
        "tie_word_embeddings": bool(a.tie_word_embeddings), "pad_token_id": a.pad_token_id,
        "eos_token_id": a.eos_token_id, "torch_dtype": "bfloat16",
    }


def hf_config_from_args(family: str, args, mup: bool = False) -> dict:
    if family in ("llama", "llama2", "llama3", "mistral"):
        return _llama(args, mup)
    if family in ("gemma", "gemma3"):
        return _gemma(args)
    if family == "deepseek":
        return _deepseek(args)
    if family == "glm4":
        return _glm4(args)
    raise KeyError(family)
