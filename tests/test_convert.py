"""Checkpoint converters: key maps on tiny random models, logits parity with transformers, DCP I/O."""
import copy
import json

import pytest
import torch

from maester_b200.convert import FAMILIES, arch_from_hf_config, arch_from_model_args, to_hf, to_native
from maester_b200.convert.cli import convert_from_dcp, convert_to_dcp
from maester_b200.convert.hf_config import hf_config_from_args
from maester_b200.convert.io import read_dcp_model, read_hf_dir, write_dcp, write_hf_dir
from maester_b200.models import model_name_to_cls, models_config

TINY = [("llama3", "tiny", "llama"), ("gemma3", "debug", "gemma"), ("deepseek", "debug_flex", "deepseek"),
        ("glm4", "debug", "glm4")]


def _native_model(name, flavor, vocab=512, **over):
    a = copy.deepcopy(models_config[name][flavor])
    if getattr(a, "vocab_size", 0) <= 0:
        a.vocab_size = vocab
    for k, v in over.items():
        setattr(a, k, v)
    torch.manual_seed(0)
    return a, model_name_to_cls[name].from_model_args(a)


@pytest.mark.parametrize("name,flavor,family", TINY)
def test_round_trip_is_identity(name, flavor, family):
    a, m = _native_model(name, flavor)
    sd = {k: torch.randn_like(v) for k, v in m.state_dict().items()}
    arch = arch_from_model_args(family, a)
    hf = to_hf(FAMILIES[family], sd, arch)
    assert all(k.startswith(("model.", "lm_head.")) for k in hf)
    back = to_native(FAMILIES[family], hf, arch)
    assert set(back) == set(sd)
    for k in sd:
        assert torch.equal(back[k], sd[k]), k


def test_unknown_keys_are_reported():
    a, m = _native_model("llama3", "tiny")
    with pytest.raises(KeyError):
        to_native(FAMILIES["llama"], {"model.layers.0.self_attn.bogus.weight": torch.zeros(1)},
                  arch_from_model_args("llama", a))


def test_llama_logits_match_transformers():
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=64, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=128, rms_norm_eps=1e-5, rope_theta=10000.0,
                      max_position_embeddings=64, tie_word_embeddings=False)
    torch.manual_seed(1)
    hf = LlamaForCausalLM(cfg).eval()
    from maester_b200.models.llama.model import ModelArgs, Transformer
    args = ModelArgs(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=128, multiple_of=256,
                     ffn_dim_multiplier=None, norm_eps=1e-5, rope_theta=10000.0, max_seq_len=64)
    # swiglu_hidden_dim(64, 256, None) = 256
    mine = Transformer(args).eval()
    native = to_native(FAMILIES["llama"], hf.state_dict(), arch_from_hf_config("llama", cfg.to_dict()))
    missing, unexpected = mine.load_state_dict(native, strict=False)
    assert not unexpected and all("rope" in k or "inv_freq" in k for k in missing)
    tok = torch.randint(0, 128, (2, 33))
    with torch.no_grad():
        want = hf(tok).logits
        got = mine(tok)
    assert (got.float() - want).abs().max().item() < 2e-4
    assert torch.equal(got.argmax(-1), want.argmax(-1))


def test_gemma3_logits_match_transformers():
    tr = pytest.importorskip("transformers")
    if not hasattr(tr, "Gemma3ForCausalLM"):
        pytest.skip("transformers without Gemma 3")
    from transformers import Gemma3ForCausalLM, Gemma3TextConfig
    _gemma3_against_transformers(max_seq_len=64)
    # every layer kind of the 5 local : 1 global pattern, a window shorter than the sequence (the native window counts
    # both ends, the exported one is a key count), scaled global RoPE, an explicit softmax scale
    _gemma3_against_transformers(max_seq_len=64, n_layers=7, sliding_window_size=16, rope_scaling={"factor": 8.0},
                                 query_pre_attn_scalar=24)


def _gemma3_against_transformers(**over):
    from transformers import Gemma3ForCausalLM, Gemma3TextConfig
    a, mine = _native_model("gemma3", "debug", **over)
    cfg = Gemma3TextConfig(**{k: v for k, v in hf_config_from_args("gemma3", a).items()
                              if k not in ("architectures", "model_type", "torch_dtype")})
    torch.manual_seed(2)
    hf = Gemma3ForCausalLM(cfg).eval()
    native = to_native(FAMILIES["gemma"], hf.state_dict(), arch_from_hf_config("gemma", cfg.to_dict()))
    missing, unexpected = mine.load_state_dict(native, strict=False)
    assert not unexpected, unexpected
    mine.eval()
    tok = torch.randint(0, a.vocab_size, (2, 48))
    with torch.no_grad():
        want = hf(tok).logits
        got = mine(tok)
    assert (got.float() - want).abs().max().item() < 1e-4
    assert (got.float() - want).abs().mean().item() < 1e-5


def test_dcp_and_safetensors_io(tmp_path):
    a, m = _native_model("llama3", "tiny")
    sd = {k: v.detach().clone() for k, v in m.state_dict().items()}
    write_dcp(tmp_path / "ckpt" / "step-5", sd)
    back = read_dcp_model(tmp_path / "ckpt" / "step-5")
    assert set(back) == set(sd) and all(torch.equal(back[k], sd[k]) for k in sd)
    # job config next to the checkpoint folder recovers the architecture
    (tmp_path / "config.json").write_text(json.dumps({"model_name": "llama3", "flavor": "tiny"}))
    # the tiny flavor takes its vocabulary from the checkpoint
    files = convert_from_dcp("llama", str(tmp_path / "ckpt" / "step-5"), str(tmp_path / "hf"), dtype=torch.float32,
                             max_shard_bytes=8 * 2**20)
    assert len(files) > 1 and (tmp_path / "hf" / "model.safetensors.index.json").is_file()
    hf_sd, hf_cfg = read_hf_dir(tmp_path / "hf")
    assert hf_cfg["model_type"] == "llama" and hf_cfg["vocab_size"] == sd["tok_embeddings.weight"].shape[0]
    native = convert_to_dcp("llama", str(tmp_path / "hf"), str(tmp_path / "dcp2"))
    again = read_dcp_model(tmp_path / "dcp2")
    for k in sd:
        assert torch.equal(native[k], sd[k]) and torch.equal(again[k], sd[k]), k


def test_mup_llama_export_matches_native_model(tmp_path):
    from maester_b200.models.hf.modeling_mup_llama import MupLlamaConfig, MupLlamaForCausalLM
    from maester_b200.models.llama.model import ModelArgs, Transformer
    args = ModelArgs(dim=256, n_layers=2, n_heads=2, n_kv_heads=2, vocab_size=96, multiple_of=64, norm_eps=1e-5,
                     max_seq_len=32, enable_mup=True, mup_output_alpha=2.0, mup_width_mul=2.0)
    torch.manual_seed(3)
    mine = Transformer(args).eval()
    hf_sd = to_hf(FAMILIES["llama"], {k: v for k, v in mine.state_dict().items()}, arch_from_model_args("llama", args))
    cfg_d = hf_config_from_args("llama", args)
    assert cfg_d["model_type"] == "mup_llama"
    cfg = MupLlamaConfig(**{k: v for k, v in cfg_d.items() if k not in ("architectures", "model_type", "torch_dtype")})
    hf = MupLlamaForCausalLM(cfg).eval()
    missing, unexpected = hf.load_state_dict(hf_sd, strict=False)
    assert not unexpected and not [k for k in missing if "inv_freq" not in k]
    tok = torch.randint(0, 96, (1, 20))
    with torch.no_grad():
        assert (mine(tok).float() - hf(tok).logits).abs().max().item() < 2e-4


def _hub_layout(state):
    """transformers keeps the routed experts of a layer as two stacked tensors in memory (``gate_up_proj`` [E, 2I, H],
    ``down_proj`` [E, H, I]); checkpoints on disk, which the converters read, hold one matrix per expert."""
    out = {}
    for k, v in state.items():
        if k.endswith("mlp.experts.gate_up_proj"):
            for e in range(v.shape[0]):
                gate, up = v[e].chunk(2, dim=0)
                out[k.replace("gate_up_proj", f"{e}.gate_proj.weight")] = gate
                out[k.replace("gate_up_proj", f"{e}.up_proj.weight")] = up
        elif k.endswith("mlp.experts.down_proj"):
            for e in range(v.shape[0]):
                out[k.replace("down_proj", f"{e}.down_proj.weight")] = v[e]
        else:
            out[k] = v
    return out


def _against_transformers(name, family, args, hf_cls, cfg_cls, tol=1e-4):
    cfg_d = hf_config_from_args(family, args)
    cfg = cfg_cls(**{k: v for k, v in cfg_d.items() if k not in ("architectures", "model_type", "torch_dtype")})
    torch.manual_seed(1)
    hf = hf_cls(cfg).eval()
    with torch.no_grad():   # the selection bias is zero after construction: give it values so that it matters
        for n, p in list(hf.named_parameters()) + list(hf.named_buffers()):
            if "e_score_correction_bias" in n:
                p.copy_(0.1 * torch.randn_like(p))
    mine = model_name_to_cls[name].from_model_args(args).eval()
    mine.init_weights()
    native = to_native(FAMILIES[family], _hub_layout(hf.state_dict()), arch_from_hf_config(family, cfg.to_dict()))
    missing, unexpected = mine.load_state_dict(native, strict=False)
    assert not unexpected and not [k for k in missing if "expert_bias" not in k], (missing, unexpected)
    tok = torch.randint(0, args.vocab_size, (2, 40))
    with torch.no_grad():
        want, got = hf(tok).logits, mine(tok).float()
    assert (got - want).abs().max().item() < tol * max(1.0, want.abs().max().item())
    assert torch.equal(got.argmax(-1), want.argmax(-1))


def test_glm4_moe_logits_match_transformers():
    """Partial rotary embedding, sigmoid router with the selection bias, renormalised top-k, shared expert."""
    from transformers import Glm4MoeConfig, Glm4MoeForCausalLM
    for qk_norm in (False, True):
        a = copy.deepcopy(models_config["glm4"]["debug"])
        a.vocab_size, a.use_qk_norm, a.attention_bias = 512, qk_norm, qk_norm
        _against_transformers("glm4", "glm4", a, Glm4MoeForCausalLM, Glm4MoeConfig)


@pytest.mark.parametrize("variant", ["v3_sigmoid_yarn", "v3_low_rank_queries", "v2_softmax"])
def test_deepseek_logits_match_transformers(variant):
    """Latent attention (with and without low-rank queries), YaRN with its softmax-scale correction, both routers.
    The experts' outputs are weighted AFTER the experts, as DeepSeek does (``score_before_experts=False``; the
    reference's own DeepSeek flavors weight the inputs instead, which is a different function).  The softmax (V2)
    variant runs without YaRN: transformers' V2 port leaves the softmax-scale correction out."""
    import transformers
    a = copy.deepcopy(models_config["deepseek"]["debug_flex"])
    a.vocab_size, a.moe_args.score_before_experts, a.moe_args.load_balance_coeff = 512, False, 1e-3
    if variant == "v2_softmax":
        a.max_seq_len = a.original_seq_len
        cls, cfg = transformers.DeepseekV2ForCausalLM, transformers.DeepseekV2Config
    else:
        a.moe_args.score_func, a.moe_args.route_norm = "sigmoid", True
        assert a.max_seq_len > a.original_seq_len
        if variant == "v3_low_rank_queries":
            a.q_lora_rank = 64
        cls, cfg = transformers.DeepseekV3ForCausalLM, transformers.DeepseekV3Config
    _against_transformers("deepseek", "deepseek", a, cls, cfg)
