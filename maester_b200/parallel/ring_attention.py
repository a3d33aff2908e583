"""Ring (zig-zag) context parallelism: every rank keeps its slice of the sequence for attention too.

The reference has no context parallelism (maester/parallelisms/parallel_dims.py:15, :87-89); the all-to-all form
in ``context_parallel.py`` needs the head counts to divide by the CP degree.  This form does not.

Layout.  The sequence is cut into ``2 * cp`` chunks of ``c`` tokens; rank r holds chunks ``r`` and ``2 cp - 1 - r``
(zig-zag), concatenated, so every rank has the same amount of causal work.  A query chunk a attends to a key/value
chunk b iff ``b <= a``: causally if ``b == a``, completely if ``b < a``.  For rank r with chunks ``(a1, a2)``:

* its own keys/values: one causal attention over the local ``[a1 | a2]`` sequence (local order = global order);
* a peer s < r (chunks ``b1 = s``, ``b2``): both query chunks attend completely to ``b1``;
* a peer s > r: query chunk ``a2`` attends completely to ``b1`` and ``b2``.

Every remote piece is a ``c x c`` attention without a mask, so the unchanged attention kernels serve all of them and
the partial results are merged by their log-sum-exp.

Data movement (CUDA).  Each rank publishes its K and V (after norm / RoPE) in a symmetric buffer.  The chunks a rank
needs from a peer are pulled over NVLink ONCE into local memory by this library's copy kernel (plain peer loads, no
multicast) on a side stream while the local causal attention runs, and the attention kernel then reads them from local
memory with TMA: a remote tile read by every query block through NVLink would cross the link ~100 times.  In the
backward pass the dK / dV contributions a rank computes for a peer's chunks are written to an outbox in symmetric
memory; after a barrier each owner adds what the others left for it (``peer_add``).  All barriers are the bounded
barrier kernel of ``SymmBuffer``.

CPU / gloo (tests): the same sharding with an all-gather of K, V and positions and a dense position mask.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from maester_b200.ops import functional as F
from maester_b200.ops import reference as ref


def zigzag_index(S: int, cp_size: int, cp_rank: int, device=None) -> torch.Tensor:
    """Global token indices held by ``cp_rank``: chunk r followed by chunk 2 cp - 1 - r."""
    assert S % (2 * cp_size) == 0, "sequence length must divide by twice the context-parallel degree"
    c = S // (2 * cp_size)
    a = torch.arange(cp_rank * c, (cp_rank + 1) * c, device=device)
    b = torch.arange((2 * cp_size - 1 - cp_rank) * c, (2 * cp_size - cp_rank) * c, device=device)
    return torch.cat([a, b])


# ----------------------------------------------------------------------------- CPU / reference path
class _AllGatherSeq(torch.autograd.Function):
    """[B, s, ...] -> [cp, B, s, ...]; the gradient of a rank's slice is the sum of what every rank sends back."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = dist.get_world_size(group)
        out = torch.empty(n, *x.shape, device=x.device, dtype=x.dtype)
        dist.all_gather_into_tensor(out.view(-1), x.contiguous().view(-1), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g[dist.get_rank(ctx.group)], None


def _ring_reference(qkv, q_norm_w, k_norm_w, pos, inv_freq, H, KV, hd, layout, eps, unit_offset, scale, cp):
    B, s, _ = qkv.shape
    q, k, v = qkv.split([H * hd, KV * hd, KV * hd], dim=-1)
    q, k, v = q.reshape(B, s, H, hd), k.reshape(B, s, KV, hd), v.reshape(B, s, KV, hd)
    q, k = ref.qk_norm_rope(q, k, q_norm_w, k_norm_w, pos, inv_freq, layout, eps, unit_offset)
    kg = _AllGatherSeq.apply(k, cp.group).permute(1, 0, 2, 3, 4).reshape(B, cp.size * s, KV, hd)
    vg = _AllGatherSeq.apply(v, cp.group).permute(1, 0, 2, 3, 4).reshape(B, cp.size * s, KV, hd)
    pg = torch.empty(cp.size, B, s, device=pos.device, dtype=pos.dtype)
    dist.all_gather_into_tensor(pg.view(-1), pos.contiguous().view(-1), group=cp.group)
    pg = pg.permute(1, 0, 2).reshape(B, cp.size * s)
    g = H // KV
    qf = q.float().permute(0, 2, 1, 3)
    kf = kg.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = vg.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    scores = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    mask = (pg[:, None, :] <= pos[:, :, None])[:, None]      # [B, 1, s, cp*s]: key position <= query position
    scores = scores.masked_fill(~mask, float("-inf"))
    out = torch.matmul(torch.softmax(scores, dim=-1), vf).permute(0, 2, 1, 3)
    return out.to(qkv.dtype).reshape(B, s, H * hd)


# ----------------------------------------------------------------------------- CUDA path
class RingState:
    """Symmetric buffers and the side stream of one context-parallel group (shared by every layer)."""

    def __init__(self, cp):
        self.cp = cp
        self.kv = None        # this rank's published K and V: [2, B, s, KV, hd]
        self.outbox = None    # [cp, 2, B, s, KV, hd]: dK / dV contributions computed here for each peer's chunks
        self.side = None
        self.numel = 0

    def ensure(self, numel: int, device) -> None:
        """(Collective) allocate for ``numel`` = 2 * B * s * KV * hd elements per rank."""
        if numel <= self.numel:
            return
        assert self.numel == 0, "the per-rank K/V size must not grow between calls"
        from maester_b200.parallel.symm import SymmBuffer
        self.kv = SymmBuffer(numel, torch.bfloat16, device, self.cp.group)
        self.outbox = SymmBuffer(numel * self.cp.size, torch.bfloat16, device, self.cp.group)
        self.side = torch.cuda.Stream(device)
        self.numel = numel


def _chunk(t: torch.Tensor, lo: int, hi: int) -> torch.Tensor:
    """Rows ``lo:hi`` of ``[B, s, heads, hd]`` with the batch stride the kernels expect (a view when B == 1)."""
    if t.shape[0] == 1:
        return t[0, lo:hi].unsqueeze(0)   # (unsqueeze gives the new batch dimension the stride of the chunk itself)
    return t[:, lo:hi].contiguous()


class _RingAttnBlock(torch.autograd.Function):
    """Packed qkv of this rank's tokens -> [QK-norm] -> RoPE -> zig-zag ring attention, one autograd node."""

    @staticmethod
    def forward(ctx, qkv, qw, kw, pos, cs, H, KV, hd, layout, eps, unit_offset, scale, state):
        from maester_b200.ops import cuda as C
        cp = state.cp
        B, s, _ = qkv.shape
        c = s // 2
        qkv2 = qkv.reshape(B * s, -1)
        pos32 = pos.reshape(-1).to(torch.int32).contiguous()
        need_qk = (qw is not None) or (cs is not None)
        qk = C.qknorm_rope_fwd(qkv2, qw, kw, pos32, cs, H, KV, hd, layout, eps, unit_offset) if need_qk else qkv2
        q = qk[:, : H * hd].view(B, s, H, hd)
        k = qk[:, H * hd:(H + KV) * hd].view(B, s, KV, hd)
        v = qkv2[:, (H + KV) * hd:].view(B, s, KV, hd)
        peer_kv, events = _publish_and_pull(state, k, v)
        out_loc, lse = C.attn_fwd(q, k, v, scale, True, None, None)       # own keys: causal over [a1 | a2]
        acc = torch.empty(B, s, H, hd, device=qkv.device, dtype=torch.float32)
        C.attn_merge(acc, lse, out_loc, lse, 0, True)
        for p, (qi, ki) in _remote_pairs(cp):
            torch.cuda.current_stream().wait_event(events[p])
            kc, vc = _chunk(peer_kv[p][0], ki * c, (ki + 1) * c), _chunk(peer_kv[p][1], ki * c, (ki + 1) * c)
            o, l = C.attn_fwd(_chunk(q, qi * c, (qi + 1) * c), kc, vc, scale, False, None, None)
            C.attn_merge(acc, lse, o, l, qi * c, False)
        out = torch.empty(B, s, H, hd, device=qkv.device, dtype=qkv.dtype)
        C.cast_f32_bf16(acc, out)
        ctx.save_for_backward(qkv2, qk if need_qk else None, qw, kw, pos32, cs, out, lse)
        ctx.cfg = (B, s, H, KV, hd, layout, eps, unit_offset, scale, need_qk)
        ctx.state = state
        return out.view(B, s, H * hd)

    @staticmethod
    def backward(ctx, dout):
        from maester_b200.ops import cuda as C
        qkv2, qk, qw, kw, pos32, cs, out, lse = ctx.saved_tensors
        B, s, H, KV, hd, layout, eps, unit_offset, scale, need_qk = ctx.cfg
        state = ctx.state
        cp = state.cp
        c = s // 2
        if qk is None:
            qk = qkv2
        q = qk[:, : H * hd].view(B, s, H, hd)
        k = qk[:, H * hd:(H + KV) * hd].view(B, s, KV, hd)
        v = qkv2[:, (H + KV) * hd:].view(B, s, KV, hd)
        dout4 = dout.reshape(B, s, H, hd).contiguous()
        peer_kv, events = _publish_and_pull(state, k, v)
        W = (H + 2 * KV) * hd
        dqkv = torch.empty(B * s, W, device=dout.device, dtype=dout.dtype)
        C.attn_bwd(q, k, v, out, dout4, lse, dqkv, scale, True, None, None)
        dq = dqkv[:, : H * hd].view(B, s, H, hd)
        # contributions for the peers' chunks go to this rank's outbox: [peer, k|v, B, s, KV, hd]
        box = state.outbox.tensor[: cp.size * 2 * B * s * KV * hd].view(cp.size, 2, B, s, KV, hd)
        written: dict = {}
        for p, (qi, ki) in _remote_pairs(cp):
            torch.cuda.current_stream().wait_event(events[p])
            rows = slice(qi * c, (qi + 1) * c)
            kc, vc = _chunk(peer_kv[p][0], ki * c, (ki + 1) * c), _chunk(peer_kv[p][1], ki * c, (ki + 1) * c)
            part = torch.empty(B * c, W, device=dout.device, dtype=dout.dtype)
            C.attn_bwd(_chunk(q, rows.start, rows.stop), kc, vc, out[:, rows].contiguous(), dout4[:, rows].contiguous(),
                       lse[:, :, rows].contiguous(), part, scale, False, None, None)
            dq[:, rows] += part[:, : H * hd].view(B, c, H, hd)
            dk_p = part[:, H * hd:(H + KV) * hd].view(B, c, KV, hd)
            dv_p = part[:, (H + KV) * hd:].view(B, c, KV, hd)
            dst_k, dst_v = box[p, 0, :, ki * c:(ki + 1) * c], box[p, 1, :, ki * c:(ki + 1) * c]
            if (p, ki) in written:   # the second query chunk attending to the same remote chunk
                dst_k += dk_p
                dst_v += dv_p
            else:
                dst_k.copy_(dk_p)
                dst_v.copy_(dv_p)
                written[(p, ki)] = True
        # every rank's outbox is complete -> each owner adds what the others left for its chunks
        state.outbox.barrier()
        dkv = torch.empty(2, B, s, KV, hd, device=dout.device, dtype=dout.dtype)
        dkv[0].copy_(dqkv[:, H * hd:(H + KV) * hd].view(B, s, KV, hd))
        dkv[1].copy_(dqkv[:, (H + KV) * hd:].view(B, s, KV, hd))
        per = B * s * KV * hd
        esz = 2
        for p in range(cp.size):
            if p == cp.rank:
                continue
            base = state.outbox.peer_ptrs[p] + (cp.rank * 2 * per) * esz   # rank p's outbox slot for me
            halves = (0,) if p > cp.rank else (0, 1)    # ranks after me used my first chunk only, ranks before me both
            for which in (0, 1):
                for b in range(B):
                    for hf in halves:
                        off = (which * per + b * s * KV * hd + hf * c * KV * hd)
                        C.peer_add_bf16(dkv[which, b, hf * c:(hf + 1) * c], base + off * esz, c * KV * hd)
        dqkv[:, H * hd:(H + KV) * hd].view(B, s, KV, hd).copy_(dkv[0])
        dqkv[:, (H + KV) * hd:].view(B, s, KV, hd).copy_(dkv[1])
        dqw = dkw = None
        if need_qk:
            mq = getattr(qw, "main_grad", None) if qw is not None else None
            mk = getattr(kw, "main_grad", None) if kw is not None else None
            bq = mq if mq is not None else (torch.zeros(hd, device=dout.device) if qw is not None else None)
            bk = mk if mk is not None else (torch.zeros(hd, device=dout.device) if kw is not None else None)
            C.qknorm_rope_bwd(dqkv, qkv2, qw, kw, pos32, cs, bq, bk, H, KV, hd, layout, eps, unit_offset)
            dqw = None if (mq is not None or qw is None) else bq.to(qw.dtype)
            dkw = None if (mk is not None or kw is None) else bk.to(kw.dtype)
        return (dqkv.view(B, s, -1), dqw, dkw) + (None,) * 10


def _remote_pairs(cp):
    """(peer, (query chunk, peer chunk)) attention pieces of this rank beyond its own keys, in ring order."""
    out = []
    for d in range(1, cp.size):
        p = (cp.rank + d) % cp.size
        if p < cp.rank:
            out += [(p, (0, 0)), (p, (1, 0))]
        else:
            out += [(p, (1, 0)), (p, (1, 1))]
    return out


def _publish_and_pull(state: RingState, k: torch.Tensor, v: torch.Tensor):
    """Publish this rank's K / V and pull the chunks needed from every peer into local memory (side stream).
    Returns ``({peer: [2, B, s, KV, hd] local tensor (rows of unused chunks undefined)}, {peer: event})``."""
    from maester_b200.ops import cuda as C
    cp = state.cp
    B, s, KV, hd = k.shape
    c = s // 2
    per = B * s * KV * hd
    state.ensure(2 * per, k.device)
    state.kv.barrier()                       # nobody still reads what this buffer held
    pub = state.kv.tensor[: 2 * per].view(2, B, s, KV, hd)
    pub[0].copy_(k)
    pub[1].copy_(v)
    state.kv.barrier()                       # every rank's K / V is published
    cur = torch.cuda.current_stream()
    state.side.wait_stream(cur)
    peer_kv, events = {}, {}
    with torch.cuda.stream(state.side):
        for d in range(1, cp.size):
            p = (cp.rank + d) % cp.size
            dst = torch.empty(2, B, s, KV, hd, device=k.device, dtype=k.dtype)
            dst.record_stream(cur)
            src = state.kv.peer_ptrs[p]
            if p > cp.rank:                  # both chunks of that rank
                C.peer_copy(dst, src, 2 * per * 2)
            else:                            # its first chunk only
                for which in (0, 1):
                    for b in range(B):
                        off = which * per + b * s * KV * hd
                        C.peer_copy(dst[which, b, :c], src + off * 2, c * KV * hd * 2)
            ev = torch.cuda.Event()
            ev.record(state.side)
            peer_kv[p], events[p] = dst, ev
    return peer_kv, events


def ring_attention_block(qkv, q_norm_w, k_norm_w, pos, inv_freq, rope_cs, n_heads, n_kv_heads, head_dim, cp, *,
                         layout: str = "half", eps: float = 1e-6, unit_offset: bool = False, scale=None,
                         causal: bool = True, window=None, doc_ids=None):
    """Attention of a zig-zag sequence shard ``qkv`` [B, S / cp, (H + 2 KV) hd]; ``pos`` are the global positions of
    the local tokens.  Plain causal attention only (no window, no document mask)."""
    if not causal or (window is not None and window > 0) or doc_ids is not None:
        raise NotImplementedError("ring context parallelism supports plain causal attention; use "
                                  "context_parallel_mode='alltoall' for windows or document masks")
    H, KV, hd = n_heads, n_kv_heads, head_dim
    scale = hd ** -0.5 if scale is None else scale
    if F.use_native(qkv) and hd in (64, 128, 256):
        if getattr(cp, "ring_state", None) is None:
            cp.ring_state = RingState(cp)
        return _RingAttnBlock.apply(qkv, q_norm_w, k_norm_w, pos, rope_cs, H, KV, hd, 0 if layout == "half" else 1,
                                    eps, unit_offset, scale, cp.ring_state)
    return _ring_reference(qkv, q_norm_w, k_norm_w, pos, inv_freq, H, KV, hd, layout, eps, unit_offset, scale, cp)
