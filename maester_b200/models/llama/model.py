"""Llama 2/3 and Mistral decoder (reference: maester/models/llama/model.py).

Pre-norm blocks ``h = x + attn(norm(x)); out = h + ffn(norm(h))`` (:379-381), separate bias-free
``wq/wk/wv/wo`` (:213-220), interleaved-pair RoPE (:133-168), causal GQA attention with scale
``1/sqrt(hd)`` (``1/hd`` under muP, :221), SwiGLU with hidden size
``multiple_of * ceil(mult * int(8·dim/3) / multiple_of)`` (:298-309), optional tied output
(:427-430), muP init / output scaling (:358-361, :518-520).  Unlike the reference (which warns and
ignores them, :483-489) ``document_ids`` are honoured: the attention kernel masks across documents.

Execution: wq/wk/wv run as one GEMM over a fused weight view, w1/w3 likewise; RoPE is fused with
the attention input pass; the loss is the chunked linear-cross-entropy.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from maester_b200 import ops
from maester_b200.log_utils import logger
from maester_b200.models.layers import FusedWeight, Linear
from maester_b200.models.norms import create_norm
from maester_b200.ops import reference as ref


@dataclass
class ModelArgs:
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: Optional[int] = None
    vocab_size: int = -1  # taken from the tokenizer when <= 0
    multiple_of: int = 256
    ffn_dim_multiplier: Optional[float] = None
    norm_eps: float = 1e-5
    rope_theta: float = 10000
    init_std: float = 0.02
    tied_embeddings: bool = False
    max_batch_size: int = 32
    max_seq_len: int = 2048
    norm_type: str = "rmsnorm"
    enable_mup: bool = False
    mup_input_alpha: float = 1.0
    mup_output_alpha: float = 1.0
    mup_width_mul: float = 1.0
    selective_recompute: bool = False

    def get_nparams_and_flops(self, model: nn.Module, seq_len: int) -> tuple[int, int]:
        n_emb = sum(p.numel() for n, p in model.named_parameters() if "embedding" in n)
        n_all = sum(p.numel() for p in model.parameters())
        logger.info(f"Total parameter count: {n_all:,} (embeddings: {n_emb:,})")
        l, h, q, t = self.n_layers, self.n_heads, self.dim // self.n_heads, seq_len
        return n_all, 6 * (n_all - n_emb) + 12 * l * h * q * t


def swiglu_hidden_dim(dim: int, multiple_of: int, ffn_dim_multiplier: Optional[float]) -> int:
    hidden = int(2 * (4 * dim) / 3)
    if ffn_dim_multiplier is not None:
        hidden = int(ffn_dim_multiplier * hidden)
    return multiple_of * ((hidden + multiple_of - 1) // multiple_of)


class Attention(nn.Module):
    def __init__(self, args: ModelArgs):
        super().__init__()
        self.n_heads = args.n_heads
        self.n_kv_heads = args.n_heads if args.n_kv_heads is None else args.n_kv_heads
        self.n_rep = self.n_heads // self.n_kv_heads
        self.head_dim = args.dim // args.n_heads
        self.wq = Linear(args.dim, self.n_heads * self.head_dim)
        self.wk = Linear(args.dim, self.n_kv_heads * self.head_dim)
        self.wv = Linear(args.dim, self.n_kv_heads * self.head_dim)
        self.wo = Linear(self.n_heads * self.head_dim, args.dim)
        self.attn_scale = 1.0 / self.head_dim if args.enable_mup else 1.0 / math.sqrt(self.head_dim)
        self._wqkv = FusedWeight([self.wq, self.wk, self.wv])

    def init_weights(self, init_std: float) -> None:
        for lin in (self.wq, self.wk, self.wv, self.wo):
            nn.init.normal_(lin.weight, mean=0.0, std=init_std)

    def forward(self, x, position_ids, inv_freq, rope_cs, document_ids, residual=None):
        from maester_b200.parallel.context_parallel import attention as cp_aware_attention
        if self.tp_fused is not None:  # x is this rank's token shard: the all-gather lives in the projection
            from maester_b200.parallel.fused_tp import ag_linear, linear_rs
            qkv = ag_linear(x, self._wqkv.get(), self.tp_fused)
        else:
            qkv = ops.linear(x, self._wqkv.get())
        out = cp_aware_attention(self, qkv, None, None, position_ids, inv_freq, rope_cs, document_ids,
                                 self.n_heads, self.n_kv_heads, self.head_dim, layout="interleaved",
                                 scale=self.attn_scale, causal=True, window=None)
        if self.tp_fused is not None:  # GEMM + reduce-scatter + residual in one pass over peer memory
            return linear_rs(out, self.wo.weight, residual, self.tp_fused)
        return self.wo(out, residual=residual)

    cp_capable = True  # context parallelism may set .cp on instances
    cp = None
    tp_fused = None    # set by apply_tp when the fused tensor-parallel kernels are usable


class FeedForward(nn.Module):
    def __init__(self, dim: int, hidden_dim: int, multiple_of: int, ffn_dim_multiplier: Optional[float]):
        super().__init__()
        hidden = int(2 * hidden_dim / 3)
        if ffn_dim_multiplier is not None:
            hidden = int(ffn_dim_multiplier * hidden)
        hidden = multiple_of * ((hidden + multiple_of - 1) // multiple_of)
        self.w1 = Linear(dim, hidden)
        self.w2 = Linear(hidden, dim)
        self.w3 = Linear(dim, hidden)
        self._w13 = None

    def _fused(self) -> FusedWeight:
        # w1 and w3 are adjacent in a flat buffer only if w2 does not sit between them; the runtime
        # orders parameters by this list when it lays out the block
        if self._w13 is None:
            self._w13 = FusedWeight([self.w1, self.w3])
        return self._w13

    fused_param_order = ("w1", "w3", "w2")

    tp_fused = None

    def forward(self, x, residual=None, recompute_act: bool = False):
        if self.tp_fused is not None:
            from maester_b200.parallel.fused_tp import ag_linear, glu_mlp_tp, linear_rs
            w_gu = self._fused().get()
            if (w_gu.shape[0] // 2) % 128 == 0 and w_gu.is_contiguous() and ops.use_native(x, w_gu):
                return glu_mlp_tp(x, w_gu, self.w2.weight, "silu", residual, self.tp_fused)
            gate_up = ag_linear(x, w_gu, self.tp_fused)
            return linear_rs(ops.glu(gate_up, "silu"), self.w2.weight, residual, self.tp_fused)
        return ops.glu_mlp(x, self._fused().get(), self.w2.weight, "silu", residual=residual)

    def init_weights(self, init_std: float) -> None:
        for lin in (self.w1, self.w2, self.w3):
            nn.init.normal_(lin.weight, mean=0.0, std=init_std)


def _fork(norm: nn.Module, x: torch.Tensor):
    """(norm(x), x) with the two gradients merged in the norm's backward kernel where the norm supports it."""
    fork = getattr(norm, "fork", None)
    return fork(x) if fork is not None else (norm(x), x)


class TransformerBlock(nn.Module):
    def __init__(self, layer_id: int, args: ModelArgs):
        super().__init__()
        self.n_heads, self.dim = args.n_heads, args.dim
        self.attention = Attention(args)
        self.feed_forward = FeedForward(args.dim, 4 * args.dim, args.multiple_of, args.ffn_dim_multiplier)
        self.layer_id, self.num_layers = layer_id, args.n_layers
        self.attention_norm = create_norm(args.norm_type, dim=args.dim, eps=args.norm_eps)
        self.ffn_norm = create_norm(args.norm_type, dim=args.dim, eps=args.norm_eps)
        self.weight_init_std = args.init_std / math.sqrt(args.mup_width_mul) if args.enable_mup else args.init_std
        self.selective_recompute = args.selective_recompute

    tp = None  # set by apply_tp: the residual stream is then sharded along the sequence

    def forward(self, x, position_ids, inv_freq, rope_cs, document_ids):
        rc = self.selective_recompute
        if self.tp is not None and self.attention.tp_fused is None:
            from maester_b200.parallel.tensor_parallel import gather_seq, reduce_scatter_seq
            a_in = gather_seq(self.attention_norm(x), self.tp)
            h = x + reduce_scatter_seq(self.attention(a_in, position_ids, inv_freq, rope_cs, document_ids), self.tp)
            f_in = gather_seq(self.ffn_norm(h), self.tp)
            return h + reduce_scatter_seq(self.feed_forward(f_in, recompute_act=rc), self.tp)
        a_in, skip = _fork(self.attention_norm, x)
        h = self.attention(a_in, position_ids, inv_freq, rope_cs, document_ids, residual=skip)
        f_in, skip = _fork(self.ffn_norm, h)
        return self.feed_forward(f_in, residual=skip, recompute_act=rc)

    def init_weights(self) -> None:
        for norm in (self.attention_norm, self.ffn_norm):
            if hasattr(norm, "reset_parameters"):
                norm.reset_parameters()
        self.attention.init_weights(self.weight_init_std)
        self.feed_forward.init_weights(self.weight_init_std)


class TiedLinear(nn.Module):
    """Output projection that reuses the embedding matrix (reference: llama/tied_linear.py:16-49)."""

    def __init__(self, tied_module: nn.Module):
        super().__init__()
        object.__setattr__(self, "_tied", tied_module)  # not registered: no duplicate parameter

    @property
    def weight(self) -> torch.Tensor:
        return self._tied.weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self._tied.weight)


class Transformer(nn.Module):
    def __init__(self, model_args: ModelArgs):
        super().__init__()
        self.model_args = model_args
        self.vocab_size, self.n_layers = model_args.vocab_size, model_args.n_layers
        self.tok_embeddings = nn.Embedding(model_args.vocab_size, model_args.dim)
        self.layers = nn.ModuleDict({str(i): TransformerBlock(i, model_args) for i in range(model_args.n_layers)})
        self.norm = create_norm(model_args.norm_type, dim=model_args.dim, eps=model_args.norm_eps)
        if model_args.tied_embeddings:
            self.output = TiedLinear(self.tok_embeddings)
        else:
            self.output = Linear(model_args.dim, model_args.vocab_size)
        self._build_rope_buffers()
        if self.tok_embeddings.weight.device.type != "meta":
            self.init_weights()

    def _build_rope_buffers(self, device=None) -> None:
        hd = self.model_args.dim // self.model_args.n_heads
        inv = ref.rope_inv_freq(hd, self.model_args.rope_theta, device=device)
        self.register_buffer("inv_freq", inv, persistent=False)
        self.register_buffer("rope_cs", ops.rope_table(inv, self.model_args.max_seq_len * 2), persistent=False)

    def init_weights(self) -> None:
        dev = self.tok_embeddings.weight.device
        if dev.type != "meta":
            self._build_rope_buffers(device=dev)
        nn.init.normal_(self.tok_embeddings.weight, std=self.model_args.init_std)
        for layer in self.layers.values():
            layer.init_weights()
        if hasattr(self.norm, "reset_parameters"):
            self.norm.reset_parameters()
        if not self.model_args.tied_embeddings:
            nn.init.normal_(self.output.weight, std=self.model_args.init_std)

    def forward(self, tokens, labels=None, position_ids=None, document_ids=None):
        B, S = tokens.shape
        tp = getattr(self, "tp", None)
        if tp is not None:
            # sequence parallel: this rank embeds its slice of the flattened tokens only; the embedding's gradient
            # is therefore a partial sum, completed by the all-reduce of replicated parameters' gradients
            from maester_b200.parallel.tensor_parallel import (gather_seq, local_tokens, sum_over_group,
                                                                vocab_parallel_cross_entropy)
            tp.batch = B
            h = ops.embedding(local_tokens(tokens, tp), self.tok_embeddings.weight)
        else:
            h = ops.embedding(tokens, self.tok_embeddings.weight)
        if position_ids is not None and position_ids.dim() == 1:
            position_ids = position_ids.unsqueeze(0)
        if position_ids is None:
            position_ids = torch.arange(S, device=tokens.device, dtype=torch.int32)[None].expand(B, S)
        for layer in self.layers.values():
            h = layer(h, position_ids, self.inv_freq, self.rope_cs, document_ids)
        h = self.norm(h)
        if self.model_args.enable_mup:
            h = h * (self.model_args.mup_output_alpha / self.model_args.mup_width_mul)
        w = self.tok_embeddings.weight if self.model_args.tied_embeddings else self.output.weight
        if tp is not None:
            if self.model_args.tied_embeddings:
                # replicated head: every rank scores its own token slice against the whole vocabulary; the ranks'
                # partial losses (each divided by the global count of valid labels) add up to the mean
                if labels is not None:
                    nvalid = (labels != -100).sum()
                    part = ops.linear_cross_entropy(h, w, local_tokens(labels, tp), nvalid=nvalid)
                    return sum_over_group(part, tp)
                return gather_seq(ops.linear(h, w), tp, same_grad=True)   # [B, S, V], identical on every rank
            h = gather_seq(h, tp)   # backward sums the ranks' partial dH (one vocabulary slice each)
            if labels is not None:
                return vocab_parallel_cross_entropy(h, w, labels, tp)
            logits = ops.linear(h, w)  # vocabulary-sharded logits [B, S, V/tp]
            if tp.loss_parallel:
                return logits
            full = torch.empty(tp.size, *logits.shape, device=logits.device, dtype=logits.dtype)
            torch.distributed.all_gather_into_tensor(full.view(-1), logits.contiguous().view(-1), group=tp.group)
            return full.permute(1, 2, 0, 3).reshape(*logits.shape[:2], -1)
        if labels is not None:
            return ops.linear_cross_entropy(h, w, labels)
        return ops.linear(h, w)

    @classmethod
    def from_model_args(cls, model_args: ModelArgs) -> "Transformer":
        return cls(model_args)
