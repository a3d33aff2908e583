"""Gemma 3 flavors (shapes as in maester/models/gemma/__init__.py:5-105)."""
from maester_b200.models.gemma.model import GemmaTextModel, ModelArgs

__all__ = ["GemmaTextModel", "ModelArgs", "gemma3_configs"]

_PATTERN = ["local_sliding"] * 5 + ["global"]  # 5 local : 1 global
_ROPE = {"local_sliding": 10_000, "global": 1_000_000}


def _g3(vocab, dim, layers, heads, kv, hd, ffn, window, scaled, qscalar=None) -> ModelArgs:
    return ModelArgs(
        vocab_size=vocab, dim=dim, n_layers=layers, n_heads=heads, num_key_value_heads=kv, head_dim=hd,
        intermediate_size=ffn, attn_types=list(_PATTERN), use_post_ffw_norm=True, use_pre_ffw_norm=True,
        sliding_window_size=window, rope_wave_length=dict(_ROPE),
        rope_scaling={"factor": 8.0} if scaled else None, query_pre_attn_scalar=qscalar,
        use_qk_norm=True, vision_config=None,
    )


gemma3_configs = {
    #              vocab    dim  L  H  KV  hd   ffn   win  scaled
    "270M": _g3(262_144, 640, 18, 4, 1, 256, 2048, 512, False),
    "1B": _g3(262_144, 1152, 26, 4, 1, 256, 6912, 512, False),
    "4B": _g3(262_208, 2560, 34, 8, 4, 256, 10240, 1024, True),
    "12B": _g3(262_208, 3840, 48, 16, 8, 256, 15360, 1024, True),
    "27B": _g3(262_208, 5376, 62, 32, 16, 128, 21504, 1024, True, qscalar=168),
    # small shapes for tests and CPU runs
    "debug": _g3(32_000, 256, 2, 4, 1, 64, 1024, 128, False),
    "debug_gqa": _g3(32_000, 256, 2, 4, 2, 64, 1024, 128, False),  # two key / value heads: splits over 2 TP ranks
}
