"""GLM-4.5 MoE text model (reference: maester/models/glm4/model.py).

HF-compatible layout: ``q_proj/k_proj/v_proj`` (optional bias) and ``o_proj``, optional per-head
QK-norm, partial rotary embedding (``partial_rotary_factor`` of the head, rotate-half pairing,
:155-231), causal GQA attention, first ``first_k_dense_replace`` layers with a dense SwiGLU
``mlp`` and the rest with the shared MoE block (sigmoid router, renormalised top-k, one shared
expert, scores applied after the experts, :422-464), ``Glm4MoeRMSNorm`` = weight * x̂ with fp32
statistics (:612-632).  ``document_ids`` are honoured by the attention kernel (the reference drops
them, :551).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn as nn

from maester_b200 import ops
from maester_b200.log_utils import logger
from maester_b200.models.layers import FusedWeight, Linear
from maester_b200.models.moe import MoE, MoEArgs
from maester_b200.models.norms import RMSNorm
from maester_b200.ops import reference as ref


@dataclass
class ModelArgs:
    vocab_size: int = 151552
    dim: int = 4096
    intermediate_size: int = 10944
    n_layers: int = 46
    n_heads: int = 96
    n_kv_heads: int = 8
    partial_rotary_factor: float = 0.5
    head_dim: int = 128
    hidden_act: str = "silu"
    attention_dropout: float = 0.0
    max_position_embeddings: int = 131072
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-05
    tie_word_embeddings: bool = False
    rope_theta: float = 10000.0
    rope_scaling: Optional[dict] = None
    pad_token_id: int = 151329
    eos_token_id: int | list[int] = field(default_factory=lambda: [151329, 151336, 151338])
    bos_token_id: Optional[int] = None
    attention_bias: bool = False
    tied_embeddings: bool = False
    attention_backend: str = "native"
    norm_type: str = "rmsnorm"
    moe_args: MoEArgs = field(default_factory=MoEArgs)
    moe_intermediate_size: int = 1408
    first_k_dense_replace: int = 1
    use_qk_norm: bool = False
    max_seq_len: int = 0  # RoPE table length / 2; 0 = max_position_embeddings
    selective_recompute: bool = False

    def get_nparams_and_flops(self, model: nn.Module, seq_len: int) -> tuple[int, int]:
        n_emb = n_dense = n_shared = n_experts = n_router = 0
        for name, p in model.named_parameters():
            if "embedding" in name:
                n_emb += p.numel()
                n_dense += p.numel()
            elif "moe.shared_experts" in name:
                n_shared += p.numel()
            elif "moe.router" in name:
                n_router += p.numel()
            elif "moe.experts" in name:
                n_experts += p.numel()
            else:
                n_dense += p.numel()
        total = n_dense + n_shared + n_experts + n_router
        active = n_shared + n_router + n_experts * self.moe_args.top_k // max(1, self.moe_args.num_experts)
        logger.info(f"Total parameter count: dense {n_dense:,}, sparse {total - n_dense:,}, active {n_dense + active:,}")
        l, h, t = self.n_layers, self.n_heads, seq_len
        return total, 6 * (n_dense - n_emb + active) + 12 * l * h * (self.dim // h) * t


Glm4MoeRMSNorm = RMSNorm


def rotary_dim_of(config: ModelArgs) -> int:
    r = int(config.head_dim * config.partial_rotary_factor)
    if r <= 0 or r > config.head_dim:
        r = config.head_dim
    if r % 2:
        r -= 1
    return max(r, 2)


class Glm4MoeAttention(nn.Module):
    def __init__(self, config: ModelArgs, layer_idx: int | None = None):
        super().__init__()
        self.config, self.layer_idx = config, layer_idx
        self.head_dim, self.n_heads, self.n_kv_heads = config.head_dim, config.n_heads, config.n_kv_heads
        self.attn_scale = self.head_dim ** -0.5
        b = config.attention_bias
        self.q_proj = Linear(config.dim, config.n_heads * self.head_dim, bias=b)
        self.k_proj = Linear(config.dim, config.n_kv_heads * self.head_dim, bias=b)
        self.v_proj = Linear(config.dim, config.n_kv_heads * self.head_dim, bias=b)
        self.o_proj = Linear(config.n_heads * self.head_dim, config.dim)
        self.use_qk_norm = config.use_qk_norm
        if self.use_qk_norm:
            self.q_norm = RMSNorm(self.head_dim, eps=config.rms_norm_eps)
            self.k_norm = RMSNorm(self.head_dim, eps=config.rms_norm_eps)
        self.rotary_dim = rotary_dim_of(config)
        self.eps = config.rms_norm_eps
        self._wqkv = FusedWeight([self.q_proj, self.k_proj, self.v_proj])

    def forward(self, x, position_ids, inv_freq, rope_cs, document_ids, residual=None):
        qkv = ops.linear(x, self._wqkv.get())
        if self.q_proj.bias is not None:
            qkv = qkv + torch.cat([self.q_proj.bias, self.k_proj.bias, self.v_proj.bias]).to(qkv.dtype)
        out = ops.attention_block(qkv, self.q_norm.weight if self.use_qk_norm else None,
                                  self.k_norm.weight if self.use_qk_norm else None, position_ids, inv_freq,
                                  rope_cs, document_ids, self.n_heads, self.n_kv_heads, self.head_dim,
                                  layout="half", eps=self.eps, unit_offset=False, scale=self.attn_scale,
                                  causal=True, window=None)
        return self.o_proj(out, residual=residual)

    def init_weights(self) -> None:
        for lin in (self.q_proj, self.k_proj, self.v_proj, self.o_proj):
            nn.init.normal_(lin.weight, mean=0.0, std=0.02)
            if lin.bias is not None:
                nn.init.zeros_(lin.bias)
        if self.use_qk_norm:
            self.q_norm.reset_parameters()
            self.k_norm.reset_parameters()


class Glm4MoeMLP(nn.Module):
    fused_param_order = ("gate_proj", "up_proj", "down_proj")

    def __init__(self, config: ModelArgs, intermediate_size: int | None = None):
        super().__init__()
        inter = intermediate_size or config.intermediate_size
        self.gate_proj = Linear(config.dim, inter)
        self.up_proj = Linear(config.dim, inter)
        self.down_proj = Linear(inter, config.dim)
        self._gate_up = FusedWeight([self.gate_proj, self.up_proj])

    def forward(self, x, residual=None):
        return self.down_proj(ops.glu(ops.linear(x, self._gate_up.get()), "silu"), residual=residual)

    def init_weights(self) -> None:
        for lin in (self.gate_proj, self.up_proj, self.down_proj):
            nn.init.normal_(lin.weight, mean=0.0, std=0.02)


class Glm4MoeDecoderLayer(nn.Module):
    def __init__(self, config: ModelArgs, layer_idx: int):
        super().__init__()
        self.hidden_size = config.dim
        self.self_attn = Glm4MoeAttention(config, layer_idx)
        self.moe_enabled = layer_idx >= config.first_k_dense_replace
        if self.moe_enabled:
            self.moe = MoE(config.moe_args, dim=config.dim, hidden_dim=config.moe_intermediate_size)
        else:
            self.mlp = Glm4MoeMLP(config)
        self.input_layernorm = RMSNorm(config.dim, eps=config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.dim, eps=config.rms_norm_eps)
        self.selective_recompute = config.selective_recompute

    def forward(self, x, position_ids, inv_freq, rope_cs, document_ids):
        rc = self.selective_recompute
        x = self.self_attn(self.input_layernorm(x), position_ids, inv_freq, rope_cs,
                           document_ids, residual=x)
        h = self.post_attention_layernorm(x)
        if self.moe_enabled:
            return x + self.moe(h)
        return self.mlp(h, residual=x)

    def init_weights(self, buffer_device=None) -> None:
        self.self_attn.init_weights()
        if self.moe_enabled:
            self.moe.init_weights(init_std=0.02, buffer_device=buffer_device)
        else:
            self.mlp.init_weights()
        self.input_layernorm.reset_parameters()
        self.post_attention_layernorm.reset_parameters()


class Glm4MoeTextModel(nn.Module):
    def __init__(self, config: ModelArgs):
        super().__init__()
        self.config = config
        self.model_args = config
        self.vocab_size, self.n_layers = config.vocab_size, config.n_layers
        self.rotary_dim = rotary_dim_of(config)
        self.layers = nn.ModuleDict({str(i): Glm4MoeDecoderLayer(config, i) for i in range(config.n_layers)})
        self.norm = RMSNorm(config.dim, eps=config.rms_norm_eps)
        self.tok_embeddings = nn.Embedding(config.vocab_size, config.dim, padding_idx=config.pad_token_id)
        self.output = Linear(config.dim, config.vocab_size)
        if config.tie_word_embeddings:
            self.output.weight = self.tok_embeddings.weight
        self._build_rope_buffers()

    def _build_rope_buffers(self, device=None) -> None:
        n_pos = 2 * (self.config.max_seq_len or self.config.max_position_embeddings)
        inv = ref.rope_inv_freq(self.rotary_dim, self.config.rope_theta, device=device)
        self.register_buffer("inv_freq", inv, persistent=False)
        self.register_buffer("rope_cs", ops.rope_table(inv, n_pos), persistent=False)

    def init_weights(self, buffer_device: torch.device | None = None) -> None:
        dev = buffer_device or self.tok_embeddings.weight.device
        if dev.type != "meta":
            self._build_rope_buffers(device=dev)
        nn.init.normal_(self.tok_embeddings.weight, std=self.config.initializer_range)
        for layer in self.layers.values():
            layer.init_weights(buffer_device=dev)
        self.norm.reset_parameters()
        if not self.config.tie_word_embeddings:
            nn.init.normal_(self.output.weight, mean=0.0, std=self.config.initializer_range)

    def moe_layers(self):
        return [l.moe for l in self.layers.values() if l.moe_enabled]

    def set_attention_backend(self, backend: str) -> None:
        if backend.lower() not in {"native", "cudnn", "auto", "flash", "naive", "math"}:
            raise ValueError(f"Unsupported attention backend '{backend}'")

    def forward(self, tokens, labels=None, position_ids=None, document_ids=None):
        B, S = tokens.shape
        h = ops.embedding(tokens, self.tok_embeddings.weight)
        if position_ids is None:
            position_ids = torch.arange(S, device=tokens.device, dtype=torch.int32)[None].expand(B, S)
        elif position_ids.dim() == 1:
            position_ids = position_ids.unsqueeze(0)
        for layer in self.layers.values():
            h = layer(h, position_ids, self.inv_freq, self.rope_cs, document_ids)
        h = self.norm(h)
        w = self.tok_embeddings.weight if self.config.tie_word_embeddings else self.output.weight
        if labels is not None:
            loss = ops.linear_cross_entropy(h, w, labels)
            aux = [m.aux_loss for m in self.moe_layers() if m.aux_loss is not None]
            return loss + sum(aux) if aux else loss
        return ops.linear(h, w)

    # the two ends of forward(), for runners that stream the blocks through the GPU one group at a time
    def forward_embed(self, tokens: torch.Tensor) -> dict:
        B, S = tokens.shape
        pos = torch.arange(S, device=tokens.device, dtype=torch.int32)[None].expand(B, S)
        return {"h": ops.embedding(tokens, self.tok_embeddings.weight), "args": (pos, self.inv_freq, self.rope_cs, None)}

    def forward_head(self, h: torch.Tensor) -> torch.Tensor:
        w = self.tok_embeddings.weight if self.config.tie_word_embeddings else self.output.weight
        return ops.linear(self.norm(h), w)

    @classmethod
    def from_model_args(cls, model_args: ModelArgs) -> "Glm4MoeTextModel":
        return cls(model_args)
