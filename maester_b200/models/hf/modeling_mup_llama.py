"""``mup_llama``: a transformers model type for Llama checkpoints trained with muP.

Same role as the reference's maester/models/hf/modeling_mup_llama.py:16-287 (``MupLlamaConfig``,
``MupLlamaModel``, ``MupLlamaForCausalLM`` registered with the Auto classes), built differently: the
classes derive from transformers' Llama implementation (HF weight layout, KV cache, generation,
attention back ends) and only add what muP changes at inference time:

* attention logits are scaled by ``1 / head_dim`` instead of ``1 / sqrt(head_dim)``;
* the final hidden states are multiplied by ``mup_output_alpha / mup_width_mul`` before the head;
* token embeddings are multiplied by ``mup_input_alpha`` when ``mup_scale_embeddings`` is set (the
  training model leaves them unscaled, so the default is off).

Importing this module registers the classes: ``AutoModelForCausalLM.from_pretrained(dir)`` then works
for exports whose ``config.json`` has ``"model_type": "mup_llama"``.
"""
from __future__ import annotations

from transformers import AutoConfig, AutoModel, AutoModelForCausalLM
from transformers.models.llama.configuration_llama import LlamaConfig
from transformers.models.llama.modeling_llama import LlamaForCausalLM, LlamaModel


class MupLlamaConfig(LlamaConfig):
    model_type = "mup_llama"

    def __init__(self, mup_input_alpha: float = 1.0, mup_output_alpha: float = 1.0, mup_width_mul: float = 1.0,
                 mup_scale_embeddings: bool = False, **kwargs):
        self.mup_input_alpha = mup_input_alpha
        self.mup_output_alpha = mup_output_alpha
        self.mup_width_mul = mup_width_mul
        self.mup_scale_embeddings = mup_scale_embeddings
        super().__init__(**kwargs)


def _apply_mup(model: LlamaModel, config: MupLlamaConfig) -> None:
    head_dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
    for layer in model.layers:
        layer.self_attn.scaling = 1.0 / head_dim
    out_scale = config.mup_output_alpha / config.mup_width_mul
    model.norm.register_forward_hook(lambda _m, _inp, out: out * out_scale)
    if config.mup_scale_embeddings and config.mup_input_alpha != 1.0:
        model.embed_tokens.register_forward_hook(lambda _m, _inp, out: out * config.mup_input_alpha)


class MupLlamaModel(LlamaModel):
    config_class = MupLlamaConfig

    def __init__(self, config: MupLlamaConfig):
        super().__init__(config)
        _apply_mup(self, config)


class MupLlamaForCausalLM(LlamaForCausalLM):
    config_class = MupLlamaConfig

    def __init__(self, config: MupLlamaConfig):
        super().__init__(config)
        _apply_mup(self.model, config)


def register() -> None:
    """Idempotent registration with the Auto classes."""
    try:
        AutoConfig.register("mup_llama", MupLlamaConfig)
    except ValueError:
        return
    AutoModel.register(MupLlamaConfig, MupLlamaModel)
    AutoModelForCausalLM.register(MupLlamaConfig, MupLlamaForCausalLM)


register()
