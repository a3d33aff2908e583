"""DeepSeek V2/V3: multi-head latent attention (MLA) + token-choice MoE.

Reference: maester/models/deepseek/model.py.  Kept: optional q-LoRA (``wq_a → RMSNorm → wq_b``),
``wkv_a`` split into (kv_lora_rank, rope_dim) → ``kv_norm`` → ``wkv_b``; q/k = concat(nope, rope),
RoPE on interleaved pairs of the rope slice with the shared ``k_pe`` expanded over heads (:135-236);
YaRN frequency correction and ``mscale²`` on the softmax scale when ``max_seq_len >
original_seq_len`` (:19-115, :169-173); layer-wise init std ``0.02 / sqrt(2 (l+1))`` (:279); output
trunc-normal std ``dim^-0.5`` (:347-356); first ``first_k_dense_replace`` layers dense.
Differences: ``forward`` honours ``labels`` (returns the fused loss) and ``document_ids`` (the
reference ignores both, :383-395), and attention runs on the native kernel with q/k zero-padded
from 192 to 256 channels and v from 128 to 256 (mathematically identical; a dedicated 192/128
kernel is future work).
"""
from __future__ import annotations

import math
import os

import torch
import torch.nn as nn

from maester_b200 import ops
from maester_b200.models.deepseek.args import DeepSeekModelArgs
from maester_b200.models.layers import Linear
from maester_b200.models.moe import FeedForward, MoE
from maester_b200.models.norms import RMSNorm
from maester_b200.ops import reference as ref


# RoPE + q|k|v packing + head-size padding of latent attention as one native kernel (csrc/mla_pack.cu)
FUSED_MLA_PACK = os.environ.get("MB_MLA_PACK", "1") != "0"


class _MLAPack(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, kvb, kpe, pos, inv_freq, dims):
        from maester_b200.ops import cuda as C
        ctx.save_for_backward(pos, inv_freq)
        ctx.dims = dims
        return C.mla_pack_fwd(q.contiguous(), kvb.contiguous(), kpe, pos, inv_freq, *dims)

    @staticmethod
    def backward(ctx, dout):
        from maester_b200.ops import cuda as C
        pos, inv_freq = ctx.saved_tensors
        dq, dkvb, dkpe = C.mla_pack_bwd(dout.contiguous(), pos, inv_freq, *ctx.dims)
        return dq, dkvb, dkpe, None, None, None


def yarn_inv_freq(args: DeepSeekModelArgs, device=None) -> torch.Tensor:
    """Inverse RoPE frequencies with the YaRN ramp between ``beta_fast`` and ``beta_slow`` rotations."""
    dim, base = args.qk_rope_head_dim, args.rope_theta
    freqs = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
    if args.max_seq_len > args.original_seq_len:
        def corr_dim(rot: float) -> float:
            return dim * math.log(args.original_seq_len / (rot * 2 * math.pi)) / (2 * math.log(base))

        low = max(math.floor(corr_dim(args.beta_fast)), 0)
        high = min(math.ceil(corr_dim(args.beta_slow)), dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(dim // 2, dtype=torch.float32, device=device) - low) / (high - low)).clamp(0, 1)
        smooth = 1 - ramp
        freqs = freqs / args.rope_factor * (1 - smooth) + freqs * smooth
    return freqs


class Attention(nn.Module):
    def __init__(self, a: DeepSeekModelArgs):
        super().__init__()
        self.dim, self.n_heads = a.dim, a.n_heads
        self.q_lora_rank, self.kv_lora_rank = a.q_lora_rank, a.kv_lora_rank
        self.qk_nope_head_dim, self.qk_rope_head_dim = a.qk_nope_head_dim, a.qk_rope_head_dim
        self.qk_head_dim = a.qk_nope_head_dim + a.qk_rope_head_dim
        self.v_head_dim = a.v_head_dim
        if self.q_lora_rank == 0:
            self.wq = Linear(self.dim, self.n_heads * self.qk_head_dim)
        else:
            self.wq_a = Linear(self.dim, self.q_lora_rank)
            self.q_norm = RMSNorm(self.q_lora_rank, eps=a.norm_eps)
            self.wq_b = Linear(self.q_lora_rank, self.n_heads * self.qk_head_dim)
        self.wkv_a = Linear(self.dim, self.kv_lora_rank + self.qk_rope_head_dim)
        self.kv_norm = RMSNorm(self.kv_lora_rank, eps=a.norm_eps)
        self.wkv_b = Linear(self.kv_lora_rank, self.n_heads * (self.qk_nope_head_dim + self.v_head_dim))
        self.wo = Linear(self.n_heads * self.v_head_dim, self.dim)
        self.softmax_scale = self.qk_head_dim ** -0.5
        if a.max_seq_len > a.original_seq_len:
            mscale = 0.1 * a.mscale * math.log(a.rope_factor) + 1.0
            self.softmax_scale *= mscale * mscale
        self.pad_dim = 256 if self.qk_head_dim > 128 else (128 if self.qk_head_dim > 64 else 64)

    def forward(self, x, position_ids, inv_freq, document_ids, residual=None):
        B, S, _ = x.shape
        H = self.n_heads
        q = self.wq(x) if self.q_lora_rank == 0 else self.wq_b(self.q_norm(self.wq_a(x)))
        P = self.pad_dim
        if (FUSED_MLA_PACK and ops.use_native(x) and position_ids is not None
                and not (self.qk_nope_head_dim | self.qk_rope_head_dim | self.v_head_dim) & 7):
            # RoPE, the shared k_pe broadcast, q|k|v packing and head-size padding in one kernel
            kv_a = self.wkv_a(x)
            kv_lat, k_pe = kv_a.split([self.kv_lora_rank, self.qk_rope_head_dim], dim=-1)
            kvb = self.wkv_b(self.kv_norm(kv_lat))
            dims = (H, self.qk_nope_head_dim, self.qk_rope_head_dim, self.v_head_dim, P)
            qkv = _MLAPack.apply(q.reshape(B * S, -1), kvb.reshape(B * S, -1), k_pe.reshape(B * S, -1),
                                 position_ids.reshape(-1).to(torch.int64), inv_freq.float().contiguous(), dims)
            out = ops.attention_block(qkv.view(B, S, 3 * H * P), None, None, None, None, None, document_ids, H, H, P,
                                      scale=self.softmax_scale, causal=True, window=None)
            out = out.view(B, S, H, P)[..., : self.v_head_dim].reshape(B, S, H * self.v_head_dim)
            return self.wo(out, residual=residual)
        q = q.view(B, S, H, self.qk_head_dim)
        q_nope, q_pe = q.split([self.qk_nope_head_dim, self.qk_rope_head_dim], dim=-1)
        q_pe = ref.apply_rope(q_pe, position_ids, inv_freq, "interleaved")
        kv = self.wkv_a(x)
        kv, k_pe = kv.split([self.kv_lora_rank, self.qk_rope_head_dim], dim=-1)
        k_pe = ref.apply_rope(k_pe.unsqueeze(2), position_ids, inv_freq, "interleaved")
        kv = self.wkv_b(self.kv_norm(kv)).view(B, S, H, self.qk_nope_head_dim + self.v_head_dim)
        k_nope, v = kv.split([self.qk_nope_head_dim, self.v_head_dim], dim=-1)
        P = self.pad_dim
        zq = x.new_zeros(B, S, H, P - self.qk_head_dim)
        zv = x.new_zeros(B, S, H, P - self.v_head_dim)
        qp = torch.cat([q_nope, q_pe, zq], dim=-1)
        kp = torch.cat([k_nope, k_pe.expand(-1, -1, H, -1), zq], dim=-1)
        vp = torch.cat([v, zv], dim=-1)
        qkv = torch.cat([qp.reshape(B, S, H * P), kp.reshape(B, S, H * P), vp.reshape(B, S, H * P)], dim=-1)
        out = ops.attention_block(qkv, None, None, None, None, None, document_ids, H, H, P,
                                  scale=self.softmax_scale, causal=True, window=None)
        out = out.view(B, S, H, P)[..., : self.v_head_dim].reshape(B, S, H * self.v_head_dim)
        return self.wo(out, residual=residual)

    def init_weights(self, init_std: float) -> None:
        lins = [self.wkv_a, self.wkv_b] + ([self.wq] if self.q_lora_rank == 0 else [self.wq_a, self.wq_b])
        for lin in lins:
            nn.init.trunc_normal_(lin.weight, mean=0.0, std=0.02)
        nn.init.trunc_normal_(self.wo.weight, mean=0.0, std=init_std)
        self.kv_norm.reset_parameters()
        if self.q_lora_rank > 0:
            self.q_norm.reset_parameters()


class TransformerBlock(nn.Module):
    def __init__(self, layer_id: int, a: DeepSeekModelArgs):
        super().__init__()
        self.attention = Attention(a)
        self.attention_norm = RMSNorm(a.dim, eps=a.norm_eps)
        self.ffn_norm = RMSNorm(a.dim, eps=a.norm_eps)
        self.moe_enabled = layer_id >= a.first_k_dense_replace
        if self.moe_enabled:
            self.moe = MoE(a.moe_args, dim=a.dim, hidden_dim=a.moe_intermediate_size)
        else:
            self.feed_forward = FeedForward(a.dim, a.inter_dim)
        self.weight_init_std = 0.02 / (2 * (layer_id + 1)) ** 0.5
        self.layer_id = layer_id
        self.selective_recompute = a.selective_recompute

    def forward(self, x, position_ids, inv_freq, document_ids):
        rc = self.selective_recompute
        x = self.attention(self.attention_norm(x), position_ids, inv_freq, document_ids,
                           residual=x)
        h = self.ffn_norm(x)
        if self.moe_enabled:
            return x + self.moe(h)
        return self.feed_forward(h, residual=x)

    def init_weights(self, buffer_device=None) -> None:
        for n in (self.attention_norm, self.ffn_norm):
            n.reset_parameters()
        self.attention.init_weights(self.weight_init_std)
        if self.moe_enabled:
            self.moe.init_weights(self.weight_init_std, buffer_device)
        else:
            self.feed_forward.init_weights(self.weight_init_std)


class DeepSeekModel(nn.Module):
    def __init__(self, model_args: DeepSeekModelArgs):
        super().__init__()
        self.model_args = model_args
        self.max_seq_len = model_args.max_seq_len
        self.tok_embeddings = nn.Embedding(model_args.vocab_size, model_args.dim)
        self.register_buffer("inv_freq", yarn_inv_freq(model_args), persistent=False)
        self.layers = nn.ModuleDict({str(i): TransformerBlock(i, model_args) for i in range(model_args.n_layers)})
        self.norm = RMSNorm(model_args.dim)
        self.output = Linear(model_args.dim, model_args.vocab_size)
        if self.tok_embeddings.weight.device.type != "meta":
            self.init_weights()

    def init_weights(self, buffer_device: torch.device | None = None) -> None:
        dev = buffer_device or self.tok_embeddings.weight.device
        if dev.type != "meta":
            self.inv_freq = yarn_inv_freq(self.model_args, device=dev)
        nn.init.normal_(self.tok_embeddings.weight)
        for layer in self.layers.values():
            layer.init_weights(buffer_device=dev)
        self.norm.reset_parameters()
        std = self.model_args.dim ** -0.5
        nn.init.trunc_normal_(self.output.weight, mean=0.0, std=std, a=-3 * std, b=3 * std)

    def moe_layers(self):
        return [l.moe for l in self.layers.values() if l.moe_enabled]

    def forward(self, tokens, labels=None, position_ids=None, document_ids=None, eos_id=None, input_batch=None):
        B, S = tokens.shape
        if document_ids is None and eos_id is not None and self.model_args.attn_mask_type == "block_causal":
            src = input_batch if input_batch is not None else tokens
            eos = (src == eos_id)
            document_ids = (eos.cumsum(dim=1) - eos.to(torch.int64)).to(torch.int32)  # EOS closes its document
        h = ops.embedding(tokens, self.tok_embeddings.weight)
        if position_ids is None:
            position_ids = torch.arange(S, device=tokens.device, dtype=torch.int32)[None].expand(B, S)
        if tokens.is_cuda:  # the packing kernel wants one int64 position per token: convert once, not per layer
            position_ids = position_ids.to(torch.int64).contiguous()
        for layer in self.layers.values():
            h = layer(h, position_ids, self.inv_freq, document_ids)
        h = self.norm(h)
        if labels is not None:
            loss = ops.linear_cross_entropy(h, self.output.weight, labels)
            aux = [m.aux_loss for m in self.moe_layers() if m.aux_loss is not None]
            return loss + sum(aux) if aux else loss
        return self.output(h)

    @classmethod
    def from_model_args(cls, model_args: DeepSeekModelArgs) -> "DeepSeekModel":
        return cls(model_args)
