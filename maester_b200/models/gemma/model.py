"""Gemma 3 text decoder.

Behaviour follows the reference (maester/models/gemma/model.py): sandwich norms around attention
and MLP (:478-510), RMSNorm ``x̂·(1+w)`` with zero-initialised weight (:135-175), fused ``qkv_proj``
with per-head QK-norm before RoPE (:309-372), half-split RoPE with a local (θ=10k, unscaled) and a
global (θ=1M, linearly scaled) table gathered by ``position_ids`` (:588-623, :744-747), attention
pattern ``attn_types[i % len]`` with an inclusive sliding window on local layers and same-document
masking from ``document_ids`` (:203-256, :532-538), tanh-GeGLU MLP (:177-195), embedding scaled by
√dim in the activation dtype (:672-678) and a tied LM head whose loss never materialises the full
logits (:759-772).  Module and parameter names equal the reference's, so checkpoints interchange.

What differs is the execution: each op is one native kernel (``maester_b200.ops``); gate/up
projections run as one GEMM over a fused weight view; masks are evaluated inside the attention
kernel from ``document_ids`` and per-block index ranges instead of materialised block masks.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from maester_b200 import ops
from maester_b200.log_utils import logger
from maester_b200.models.layers import Embedding, FusedWeight, Linear
from maester_b200.ops import reference as ref


@dataclass
class ModelArgs:
    vocab_size: int = 32000
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    num_key_value_heads: int = 32
    head_dim: int = 128
    intermediate_size: int = 11008
    max_seq_len: int = 8192
    layer_norm_eps: float = 1e-5
    initializer_range: float = 0.02
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2
    attn_types: list[str] | None = None
    query_pre_attn_scalar: float | None = None
    rms_norm_eps: float = 1e-6
    use_qk_norm: bool = True
    sliding_window_size: int = 512
    use_pre_ffw_norm: bool = True
    use_post_ffw_norm: bool = True
    rope_wave_length: dict[str, float] | None = None
    rope_scaling: dict[str, float] | None = None
    vision_config: dict | None = None
    tied_embeddings: bool = True
    init_std: float = 0.02
    norm_type: str = "rmsnorm"
    # execution options of this framework
    selective_recompute: bool = False  # per-op recomputation plan is active (parallel/parallelize.py::apply_ac)

    def get_nparams_and_flops(self, model: nn.Module, seq_len: int) -> tuple[int, int]:
        """Parameter count and FLOPs/token: ``6·(N − N_emb) + 12·L·H·(dim//H)·T`` (model.py:44-82)."""
        n_emb = sum(p.numel() for n, p in model.named_parameters() if "embedding" in n)
        n_all = sum(p.numel() for p in model.parameters())
        logger.info(f"Total parameter count: {n_all:,} (embeddings: {n_emb:,})")
        l, h, q, t = self.n_layers, self.n_heads, self.dim // self.n_heads, seq_len
        return n_all, 6 * (n_all - n_emb) + 12 * l * h * q * t


class RMSNorm(nn.Module):
    """fp32 RMS normalisation scaled by ``1 + weight`` (``weight`` alone if add_unit_offset=False)."""

    def __init__(self, dim: int, eps: float = 1e-6, add_unit_offset: bool = True):
        super().__init__()
        self.eps, self.add_unit_offset = eps, add_unit_offset
        self.weight = nn.Parameter(torch.zeros(dim))

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, self.add_unit_offset, residual)

    def fork(self, x: torch.Tensor):
        """(norm(x), x): the second value is the skip connection of the branch that the first one enters."""
        return ops.rmsnorm_fork(x, self.weight, self.eps, self.add_unit_offset)

    def reset_parameters(self) -> None:
        nn.init.zeros_(self.weight)


class GemmaMLP(nn.Module):
    def __init__(self, hidden_size: int, intermediate_size: int):
        super().__init__()
        self.gate_proj = Linear(hidden_size, intermediate_size)
        self.up_proj = Linear(hidden_size, intermediate_size)
        self.down_proj = Linear(intermediate_size, hidden_size)
        self._gate_up = FusedWeight([self.gate_proj, self.up_proj])

    tp_fused = None    # set by apply_tp when the fused tensor-parallel kernels are usable

    def forward(self, x: torch.Tensor, recompute_act: bool = False) -> torch.Tensor:
        w_gu = self._gate_up.get()
        if self.tp_fused is not None:  # x: this rank's token rows; returns this rank's token rows of the summed result
            from maester_b200.parallel.fused_tp import ag_linear, glu_mlp_tp, linear_rs
            if (w_gu.shape[0] // 2) % 128 == 0 and w_gu.is_contiguous() and ops.use_native(x, w_gu):
                return glu_mlp_tp(x, w_gu, self.down_proj.weight, "gelu_tanh", None, self.tp_fused)
            return linear_rs(ops.glu(ag_linear(x, w_gu, self.tp_fused), "gelu_tanh"), self.down_proj.weight, None,
                             self.tp_fused)
        # one autograd node: the gated activation lives in the GEMM epilogues (forward and backward)
        return ops.glu_mlp(x, w_gu, self.down_proj.weight, "gelu_tanh")

    def init_weights(self, init_std: float) -> None:
        for lin in (self.gate_proj, self.up_proj, self.down_proj):
            nn.init.normal_(lin.weight, mean=0.0, std=init_std)


class GemmaAttention(nn.Module):
    cp_capable = True  # context parallelism may set .cp on instances
    cp = None

    def __init__(self, config: ModelArgs, attn_type: str):
        super().__init__()
        self.num_heads = config.n_heads
        self.num_kv_heads = config.num_key_value_heads
        assert self.num_heads % self.num_kv_heads == 0
        self.hidden_size, self.head_dim = config.dim, config.head_dim
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        qs = config.query_pre_attn_scalar
        self.scaling = (qs if qs is not None else self.head_dim) ** -0.5
        self.qkv_proj = Linear(self.hidden_size, self.q_size + 2 * self.kv_size)
        self.o_proj = Linear(self.q_size, self.hidden_size)
        self.query_norm = RMSNorm(self.head_dim, eps=config.rms_norm_eps) if config.use_qk_norm else None
        self.key_norm = RMSNorm(self.head_dim, eps=config.rms_norm_eps) if config.use_qk_norm else None
        self.attn_type = attn_type
        self.sliding_window_size = config.sliding_window_size
        self.eps = config.rms_norm_eps

    tp_fused = None    # set by apply_tp when the fused tensor-parallel kernels are usable

    def forward(self, x, position_ids, inv_freq, rope_cs, document_ids):
        if self.tp_fused is not None:  # x is this rank's token shard: the all-gather lives in the projection
            from maester_b200.parallel.fused_tp import ag_linear, linear_rs
            qkv = ag_linear(x, self.qkv_proj.weight, self.tp_fused)
        else:
            qkv = self.qkv_proj(x)
        window = self.sliding_window_size if (self.attn_type == "local_sliding" and self.sliding_window_size) else None
        from maester_b200.parallel.context_parallel import attention as cp_aware_attention
        out = cp_aware_attention(
            self, qkv,
            self.query_norm.weight if self.query_norm is not None else None,
            self.key_norm.weight if self.key_norm is not None else None,
            position_ids, inv_freq, rope_cs, document_ids,
            self.num_heads, self.num_kv_heads, self.head_dim,
            layout="half", eps=self.eps, unit_offset=True, scale=self.scaling, causal=True, window=window,
        )
        if self.tp_fused is not None:  # GEMM + reduce-scatter over peer memory: this rank's token rows of the sum
            return linear_rs(out, self.o_proj.weight, None, self.tp_fused)
        return self.o_proj(out)

    def init_weights(self, init_std: float) -> None:
        nn.init.normal_(self.qkv_proj.weight, mean=0.0, std=init_std)
        nn.init.normal_(self.o_proj.weight, mean=0.0, std=init_std)
        for n in (self.query_norm, self.key_norm):
            if n is not None:
                n.reset_parameters()


class Gemma2DecoderLayer(nn.Module):
    """Decoder layer used by Gemma 2 and 3 (name kept for checkpoint/FQN compatibility)."""

    def __init__(self, config: ModelArgs, attn_type: str):
        super().__init__()
        self.attn_type = attn_type
        self.self_attn = GemmaAttention(config, attn_type)
        self.mlp = GemmaMLP(config.dim, config.intermediate_size)
        eps = config.rms_norm_eps
        self.input_layernorm = RMSNorm(config.dim, eps=eps)
        self.post_attention_layernorm = RMSNorm(config.dim, eps=eps)
        self.pre_feedforward_layernorm = RMSNorm(config.dim, eps=eps) if config.use_pre_ffw_norm else None
        self.post_feedforward_layernorm = RMSNorm(config.dim, eps=eps) if config.use_post_ffw_norm else None
        self.selective_recompute = config.selective_recompute

    tp = None  # set by apply_tp: the residual stream is then sharded along the flattened token dimension

    def forward(self, x, position_ids, inv_freq, rope_cs, document_ids):
        rc = self.selective_recompute
        if self.tp is not None:
            # sequence parallel: the four norms and the residual stream work on this rank's token rows; the
            # attention and MLP blocks see all tokens (all-gather in front) with this rank's heads / hidden slice and
            # return partial sums (reduce-scatter behind).  With the fused kernels the two collectives live inside
            # the blocks' first and last GEMM.
            from maester_b200.parallel.tensor_parallel import gather_seq, reduce_scatter_seq
            fused = self.self_attn.tp_fused is not None
            gather = (lambda t: t) if fused else (lambda t: gather_seq(t, self.tp))
            scatter = (lambda t: t) if fused else (lambda t: reduce_scatter_seq(t, self.tp))
            h, skip = self.input_layernorm.fork(x)
            a = scatter(self.self_attn(gather(h), position_ids, inv_freq, rope_cs, document_ids))
            x = self.post_attention_layernorm(a, residual=skip)
            h, skip = self.pre_feedforward_layernorm.fork(x) if self.pre_feedforward_layernorm is not None else (x, x)
            m = scatter(self.mlp(gather(h), recompute_act=rc))
            if self.post_feedforward_layernorm is not None:
                return self.post_feedforward_layernorm(m, residual=skip)
            return skip + m
        h, skip = self.input_layernorm.fork(x)
        h = self.self_attn(h, position_ids, inv_freq, rope_cs, document_ids)
        x = self.post_attention_layernorm(h, residual=skip)  # x + norm(attn)
        h, skip = self.pre_feedforward_layernorm.fork(x) if self.pre_feedforward_layernorm is not None else (x, x)
        h = self.mlp(h, recompute_act=rc)
        if self.post_feedforward_layernorm is not None:
            return self.post_feedforward_layernorm(h, residual=skip)
        return skip + h

    def init_weights(self, init_std: float) -> None:
        for n in (self.input_layernorm, self.post_attention_layernorm, self.pre_feedforward_layernorm,
                  self.post_feedforward_layernorm):
            if n is not None:
                n.reset_parameters()
        self.self_attn.init_weights(init_std)
        self.mlp.init_weights(init_std)


class GemmaModel(nn.Module):
    def __init__(self, config: ModelArgs):
        super().__init__()
        self.config = config
        self.layers = nn.ModuleList()
        for i in range(config.n_layers):
            t = config.attn_types[i % len(config.attn_types)] if config.attn_types else "global"
            self.layers.append(Gemma2DecoderLayer(config, t))
        self.norm = RMSNorm(config.dim, eps=config.rms_norm_eps)

    def init_weights(self, init_std: float) -> None:
        for layer in self.layers:
            layer.init_weights(init_std)
        self.norm.reset_parameters()


class GemmaTextModel(nn.Module):
    """``forward(tokens, labels=None, position_ids=None, document_ids=None)`` → loss or logits."""

    def __init__(self, config: ModelArgs):
        super().__init__()
        self.config = config
        self.model_args = config
        self.vocab_size, self.n_layers = config.vocab_size, config.n_layers
        self.tok_embeddings = Embedding(config.vocab_size, config.dim)
        self.model = GemmaModel(config)
        self._attention_backend = "native"
        self._build_rope_buffers()

    # -- rope -------------------------------------------------------------------------------
    def _rope_params(self):
        wl = self.config.rope_wave_length or {}
        factor = (self.config.rope_scaling or {}).get("factor", 1.0)
        # the scaling factor applies to global layers only
        return {"local_sliding": (wl.get("local_sliding", 10_000), 1.0), "global": (wl.get("global", 10_000), factor)}

    def _build_rope_buffers(self, device=None) -> None:
        hd, n_pos = self.config.head_dim, self.config.max_seq_len * 2
        for name, (theta, factor) in self._rope_params().items():
            inv = ref.rope_inv_freq(hd, theta, factor, device=device)
            self.register_buffer(f"{name}_inv_freq", inv, persistent=False)
            self.register_buffer(f"{name}_rope_cs", ops.rope_table(inv, n_pos), persistent=False)

    def init_weights(self) -> None:
        dev = self.tok_embeddings.weight.device
        if dev.type != "meta":
            self._build_rope_buffers(device=dev)  # RoPE tables are never in checkpoints
        nn.init.normal_(self.tok_embeddings.weight, std=self.config.init_std)
        self.model.init_weights(self.config.init_std)

    def set_attention_backend(self, backend: str) -> None:
        if backend not in {"native", "flex", "naive"}:
            raise ValueError(f"Unsupported attention backend: {backend}")
        self._attention_backend = backend

    # -- forward ----------------------------------------------------------------------------
    def forward(self, tokens, labels=None, position_ids=None, document_ids=None):
        B, S = tokens.shape
        tp = getattr(self, "tp", None)
        if tp is not None:   # this rank embeds its slice of the flattened tokens only (partial embedding gradient)
            from maester_b200.parallel.tensor_parallel import gather_seq, local_tokens, sum_over_group
            tp.batch = B
            x = self.tok_embeddings(local_tokens(tokens, tp), scale=self.config.dim ** 0.5)
        else:
            x = self.tok_embeddings(tokens, scale=self.config.dim ** 0.5)
        if position_ids is None:
            position_ids = torch.arange(S, device=tokens.device, dtype=torch.int32)[None].expand(B, S)
        tables = {
            t: (getattr(self, f"{t}_inv_freq"), getattr(self, f"{t}_rope_cs")) for t in ("local_sliding", "global")
        }
        for layer in self.model.layers:
            inv, cs = tables.get(layer.attn_type, tables["global"])
            x = layer(x, position_ids, inv, cs, document_ids)
        h = self.model.norm(x)
        w = self.tok_embeddings.weight
        if tp is not None:
            # tied, replicated head: every rank scores its own token slice against the whole vocabulary; the ranks'
            # partial losses (each divided by the global count of valid labels) add up to the mean
            if labels is not None:
                nvalid = (labels != -100).sum()
                return sum_over_group(ops.linear_cross_entropy(h, w, local_tokens(labels, tp), nvalid=nvalid), tp)
            return gather_seq(ops.linear(h, w), tp, same_grad=True)
        if labels is not None:
            return ops.linear_cross_entropy(h, w, labels)
        return ops.linear(h, w)

    @classmethod
    def from_model_args(cls, model_args: ModelArgs) -> "GemmaTextModel":
        return cls(model_args)


class Gemma3MultiModalModel(nn.Module):
    """Text tower of the multimodal checkpoint layout; the vision tower is not part of training
    here (the reference ships the same stub, model.py:780-882)."""

    def __init__(self, config: ModelArgs):
        super().__init__()
        if config.vision_config is not None:
            logger.warning("vision_config is ignored: only the language model is instantiated")
        self.language_model = GemmaTextModel(config)

    def forward(self, tokens, labels=None, position_ids=None, document_ids=None):
        return self.language_model(tokens, labels, position_ids, document_ids)

    def init_weights(self) -> None:
        self.language_model.init_weights()

    @classmethod
    def from_model_args(cls, model_args: ModelArgs) -> "Gemma3MultiModalModel":
        return cls(model_args)
