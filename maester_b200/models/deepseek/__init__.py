"""DeepSeek flavors (shapes as in maester/models/deepseek/__init__.py:7-164)."""
from maester_b200.models.deepseek.args import DeepSeekModelArgs
from maester_b200.models.deepseek.model import DeepSeekModel
from maester_b200.models.deepseek.optimizer import build_deepseek_optimizers
from maester_b200.models.moe import MoEArgs

__all__ = ["DeepSeekModel", "DeepSeekModelArgs", "build_deepseek_optimizers", "deepseek_configs"]


def _moe(E, top_k, shared=2, scale=1.0, **kw) -> MoEArgs:
    return MoEArgs(num_experts=E, num_shared_experts=shared, top_k=top_k, score_func="softmax", route_scale=scale,
                   use_grouped_mm=True, load_balance_coeff=None, **kw)


def _ds(vocab, dim, inter, moe_inter, layers, heads, moe, dense=1, q_lora=0, mscale=0.70, flex=True, **kw):
    return DeepSeekModelArgs(vocab_size=vocab, dim=dim, inter_dim=inter, moe_intermediate_size=moe_inter,
                             n_layers=layers, first_k_dense_replace=dense, n_heads=heads, moe_args=moe,
                             q_lora_rank=q_lora, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64,
                             v_head_dim=128, mscale=mscale, use_flex_attn=flex, attn_mask_type="causal", **kw)


deepseek_configs = {
    "debug": _ds(129280, 512, 2048, 512, 8, 16, _moe(8, 3), flex=False, max_batch_size=32),
    "debug_flex": _ds(2000, 256, 1024, 256, 3, 16, _moe(8, 3)),
    "debug_flex_gate_after": _ds(2000, 256, 1024, 256, 3, 16, _moe(8, 3, score_before_experts=False)),
    "16B": _ds(102400, 2048, 10944, 1408, 27, 16, _moe(64, 6)),
    "45B_custom": _ds(102400, 3072, 8192, 1408, 20, 128, _moe(160, 6, scale=16.0), q_lora=1536),
    "236B": _ds(102400, 5120, 12288, 1536, 60, 128, _moe(160, 6, scale=16.0), q_lora=1536),
    "685B": _ds(129280, 7168, 18432, 2048, 61, 128, _moe(256, 8, shared=1, scale=2.5), dense=3, q_lora=1536,
                mscale=1.0),
    # 16-layer MoE used as a benchmark configuration: 64 routed experts (ffn 1408) + 2 shared, top-6
    "bench16L": _ds(102400, 2048, 10944, 1408, 16, 16, _moe(64, 6), max_seq_len=4096),
    # the same block at 6 layers: fits one GPU with fp32 master weights and Adam state (no expert parallelism)
    "bench6L": _ds(102400, 2048, 10944, 1408, 6, 16, _moe(64, 6), max_seq_len=4096),
}
