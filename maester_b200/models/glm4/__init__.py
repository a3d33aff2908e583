"""GLM-4.5 MoE flavors (shapes as in maester/models/glm4/__init__.py:6-111)."""
from maester_b200.models.glm4.model import Glm4MoeTextModel, ModelArgs
from maester_b200.models.moe import MoEArgs

__all__ = ["Glm4MoeTextModel", "ModelArgs", "glm4_configs"]


def _glm(dim, inter, layers, heads, kv, hd, moe_inter, E, top_k, theta=100000, eps=1e-6, bias=False,
         pad=0, eos=(2,)) -> ModelArgs:
    return ModelArgs(
        vocab_size=151_552, dim=dim, intermediate_size=inter, n_layers=layers, n_heads=heads, n_kv_heads=kv,
        head_dim=hd, hidden_act="silu", attention_dropout=0.0, max_position_embeddings=131_072,
        initializer_range=0.02, rms_norm_eps=eps, tie_word_embeddings=False, rope_theta=theta, rope_scaling=None,
        pad_token_id=pad, eos_token_id=list(eos), bos_token_id=1, attention_bias=bias, tied_embeddings=False,
        moe_args=MoEArgs(num_experts=E, score_func="sigmoid", route_norm=True, top_k=top_k, num_shared_experts=1,
                         score_before_experts=False, use_grouped_mm=True),
        moe_intermediate_size=moe_inter, first_k_dense_replace=1, use_qk_norm=False,
    )


glm4_configs = {
    "debug": _glm(512, 1024, 4, 8, 2, 64, 256, 8, 2),
    "small": _glm(2048, 5376, 32, 64, 8, 128, 1024, 64, 8),
    "106B": _glm(2048, 10944, 20, 96, 8, 128, 1408, 128, 8, theta=1_000_000, eps=1e-5, bias=True, pad=151329,
                 eos=(151329, 151336, 151338)),
}
