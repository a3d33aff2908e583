"""Context parallelism: the sequence is split over the ``cp`` mesh dimension.

The reference reserves mesh names for context parallelism but implements none
(maester/parallelisms/parallel_dims.py:15, :87-89).  Here every rank of a CP group holds a contiguous
``S / cp`` slice of each sequence for everything that is token-local (embedding, norms, MLP, loss);
around attention the layout is switched from sequence-sharded to head-sharded with one all-to-all
(each rank then sees the full sequence for ``H / cp`` query heads and ``KV / cp`` key/value heads,
GQA groups stay together), the unchanged attention kernel runs with global positions and document
ids, and a second all-to-all restores the sequence sharding.  Causal work is balanced by
construction, and any mask the kernel supports works unchanged.  Parameters are replicated over
``cp`` and sharded over ``dp_shard x cp``; gradients are averaged over that product.

``mode="ring"`` (``context_parallel_mode``) selects the zig-zag ring form of ``ring_attention.py`` instead: every
rank keeps its (zig-zag) slice of the sequence for attention too and pulls the peers' K / V chunks over NVLink; it
works for any head count but supports plain causal attention only.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from maester_b200 import ops


@dataclass
class CPInfo:
    group: object
    size: int
    rank: int
    mode: str = "alltoall"      # "alltoall" (sequence <-> heads) or "ring" (zig-zag, K / V pulled from the peers)
    ring_state: object = None


def _a2a(x: torch.Tensor, cp: CPInfo) -> torch.Tensor:
    out = torch.empty_like(x)
    dist.all_to_all_single(out.view(-1), x.contiguous().view(-1), group=cp.group)
    return out


def _seq_to_heads(x: torch.Tensor, parts: list[int], hd: int, cp: CPInfo) -> torch.Tensor:
    """[B, s, sum(parts)*hd] sequence-sharded → [B, s*cp, sum(parts)/cp*hd] head-sharded.
    ``parts`` are head counts of consecutive tensors (q, k, v): each is split over ranks separately."""
    B, s, _ = x.shape
    pieces, o = [], 0
    for n in parts:
        pieces.append(x[..., o * hd:(o + n) * hd].reshape(B, s, cp.size, (n // cp.size) * hd))
        o += n
    send = torch.cat(pieces, dim=-1).permute(2, 0, 1, 3).contiguous()  # [dst, B, s, local heads*hd]
    recv = _a2a(send, cp)                                              # [src, B, s, ...]
    return recv.permute(1, 0, 2, 3).reshape(B, cp.size * s, -1)


def _heads_to_seq(x: torch.Tensor, parts: list[int], hd: int, cp: CPInfo) -> torch.Tensor:
    """Inverse of ``_seq_to_heads``."""
    B, S, _ = x.shape
    s = S // cp.size
    send = x.reshape(B, cp.size, s, -1).permute(1, 0, 2, 3).contiguous()  # [dst(seq chunk), B, s, local]
    recv = _a2a(send, cp)                                                 # [src(head group), B, s, local]
    outs, o = [], 0
    for n in parts:
        w = (n // cp.size) * hd
        outs.append(recv[..., o:o + w].permute(1, 2, 0, 3).reshape(B, s, n * hd))
        o += w
    return torch.cat(outs, dim=-1)


class _SeqToHeads(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, parts, hd, cp):
        ctx.args = (parts, hd, cp)
        return _seq_to_heads(x, parts, hd, cp)

    @staticmethod
    def backward(ctx, g):
        parts, hd, cp = ctx.args
        return _heads_to_seq(g, parts, hd, cp), None, None, None


class _HeadsToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, parts, hd, cp):
        ctx.args = (parts, hd, cp)
        return _heads_to_seq(x, parts, hd, cp)

    @staticmethod
    def backward(ctx, g):
        parts, hd, cp = ctx.args
        return _seq_to_heads(g, parts, hd, cp), None, None, None


def cp_attention_block(qkv, q_norm_w, k_norm_w, pos_full, inv_freq, rope_cs, doc_full, n_heads, n_kv_heads,
                       head_dim, cp: CPInfo, **kw):
    """``ops.attention_block`` for a sequence-sharded ``qkv`` [B, S/cp, (H+2KV)*hd].

    ``pos_full`` / ``doc_full`` are the position and document ids of the WHOLE sequence [B, S]."""
    assert n_heads % cp.size == 0 and n_kv_heads % cp.size == 0, "head counts must divide by the CP degree"
    x = _SeqToHeads.apply(qkv, [n_heads, n_kv_heads, n_kv_heads], head_dim, cp)
    out = ops.attention_block(x, q_norm_w, k_norm_w, pos_full, inv_freq, rope_cs, doc_full,
                              n_heads // cp.size, n_kv_heads // cp.size, head_dim, **kw)
    return _HeadsToSeq.apply(out, [n_heads], head_dim, cp)


def attention(module, qkv, q_norm_w, k_norm_w, pos, inv_freq, rope_cs, doc, n_heads, n_kv_heads, head_dim, **kw):
    """Attention entry point used by the models: context-parallel if ``module.cp`` is set."""
    cp = getattr(module, "cp", None)
    if cp is None or cp.size == 1:
        return ops.attention_block(qkv, q_norm_w, k_norm_w, pos, inv_freq, rope_cs, doc, n_heads, n_kv_heads,
                                   head_dim, recompute_qk=getattr(module, "recompute_qk", False), **kw)
    if cp.mode == "ring":
        from maester_b200.parallel.ring_attention import ring_attention_block
        return ring_attention_block(qkv, q_norm_w, k_norm_w, pos, inv_freq, rope_cs, n_heads, n_kv_heads, head_dim, cp,
                                    doc_ids=doc, **kw)
    return cp_attention_block(qkv, q_norm_w, k_norm_w, pos, inv_freq, rope_cs, doc, n_heads, n_kv_heads, head_dim,
                              cp, **kw)


def apply_cp(model: torch.nn.Module, parallel_dims, mode: str = "alltoall") -> CPInfo:
    """Mark every attention module (anything with an ``attn``-like forward that calls
    ``context_parallel.attention``) with the CP group."""
    group = parallel_dims.mesh_group("cp")
    cp = CPInfo(group, dist.get_world_size(group), dist.get_rank(group), mode=mode)
    for m in model.modules():
        if hasattr(m, "cp_capable"):
            m.cp = cp
    model.cp = cp
    return cp


def shard_batch_for_cp(batch: dict, cp: CPInfo | None) -> dict:
    """Token-local tensors keep this rank's sequence slice; ids needed by attention stay whole."""
    if cp is None or cp.size == 1:
        return batch
    out = dict(batch)
    S = batch["input_ids"].shape[1]
    if cp.mode == "ring":
        # zig-zag: chunk r and chunk 2 cp - 1 - r; positions are those of the local tokens; documents are not
        # supported (the caller checks that a batch has a single document per row)
        from maester_b200.parallel.ring_attention import zigzag_index
        idx = zigzag_index(S, cp.size, cp.rank, device=batch["input_ids"].device)
        out["input_ids"] = batch["input_ids"].index_select(1, idx)
        out["labels"] = batch["labels"].index_select(1, idx)
        pos = batch.get("position_ids")
        if pos is None:
            B = batch["input_ids"].shape[0]
            out["position_ids"] = idx.to(torch.int32)[None].expand(B, idx.numel()).contiguous()
        else:
            out["position_ids"] = pos.index_select(1, idx)
        out.pop("document_ids", None)
        return out
    assert S % cp.size == 0
    s = S // cp.size
    sl = slice(cp.rank * s, (cp.rank + 1) * s)
    out["input_ids"] = batch["input_ids"][:, sl]
    out["labels"] = batch["labels"][:, sl]
    if batch.get("position_ids") is None:
        B = batch["input_ids"].shape[0]
        out["position_ids"] = torch.arange(S, device=batch["input_ids"].device, dtype=torch.int32)[None].expand(B, S)
    return out
