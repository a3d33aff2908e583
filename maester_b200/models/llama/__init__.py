"""Llama 2 / Llama 3 / Mistral flavors (shapes as in maester/models/llama/__init__.py:14-135)."""
from maester_b200.models.llama.model import ModelArgs, Transformer

__all__ = ["Transformer", "ModelArgs", "llama2_configs", "llama3_configs", "mistral_configs"]


def _m(dim, layers, heads, kv=None, mult=None, mo=256, theta=10000, **kw) -> ModelArgs:
    return ModelArgs(dim=dim, n_layers=layers, n_heads=heads, n_kv_heads=kv, ffn_dim_multiplier=mult,
                     multiple_of=mo, rope_theta=theta, **kw)


llama2_configs = {
    "debugmodel": _m(256, 2, 16),
    "271M": _m(1024, 16, 8),
    "1B": _m(2048, 18, 16),
    "7B": _m(4096, 32, 32),
    "13B": _m(5120, 40, 40),
    "26B": _m(5120, 80, 40),
    "70B": _m(8192, 80, 64, kv=8, mult=1.3, mo=4096),
}

llama3_configs = {
    "debugmodel": _m(1024, 4, 16, theta=500000),
    "tiny": _m(768, 3, 8, mult=0.6, mo=256, max_batch_size=64, tied_embeddings=True),
    "430M": _m(1024, 24, 32, kv=8, mult=1.3, mo=1024, theta=500000),
    "500M": _m(1024, 14, 32, kv=8, mult=1.2, mo=512, theta=500000),
    "1B": _m(2048, 16, 32, kv=8, mult=1.3, mo=1024, theta=500000),
    "Munin-4B": _m(4096, 16, 32, kv=8, mult=1.3, mo=1024, theta=500000),
    "1B-v2": _m(1536, 24, 32, kv=8, mult=1.2, mo=512, theta=500000),
    "3B": _m(3072, 28, 24, kv=8, mult=1.0, mo=1024, theta=500000),
    "Comma7B": _m(4096, 32, 32, theta=100000.0, max_seq_len=4096, vocab_size=64256),
    "8B": _m(4096, 32, 32, kv=8, mult=1.3, mo=1024, theta=500000),
    "sweep": _m(4096, 4, 8, kv=8, mult=1.3, mo=256, theta=500000),
    "70B": _m(8192, 80, 64, kv=8, mult=1.3, mo=4096, theta=500000),
}

mistral_configs = {
    "debugmodel": _m(256, 2, 16),
    "7B": _m(4096, 32, 32, kv=8, mult=1.2, mo=2048, theta=10000),
}
