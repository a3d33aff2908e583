"""Public op API used by the models: each op runs the native sm_100a kernel for bf16 CUDA tensors
and the plain-PyTorch definition (``reference.py``) otherwise (CPU runs, fp32 oracles).

Weight gradients: if a parameter carries a ``main_grad`` attribute (an fp32 accumulation buffer set
up by the sharding runtime) the backward accumulates into it in place and returns no autograd
gradient for that parameter; otherwise the gradient is returned normally.
"""
from __future__ import annotations

import contextlib
import os

import torch
from torch.autograd import Function

from maester_b200.ops import reference as ref

_ACT = {"gelu_tanh": 0, "silu": 1}


def use_native(*tensors: torch.Tensor) -> bool:
    t = tensors[0]
    return t.is_cuda and t.dtype == torch.bfloat16


def _C():
    from maester_b200.ops import cuda
    return cuda


def _acc_or_return(param: torch.Tensor, make_grad_into):
    """Accumulate into ``param.main_grad`` if present (returns None) else materialise a gradient."""
    mg = getattr(param, "main_grad", None)
    if mg is not None:
        make_grad_into(mg, True)
        return None
    g = torch.zeros(param.shape, device=param.device, dtype=torch.float32)
    make_grad_into(g, True)
    return g.to(param.dtype)


# --------------------------------------------------------------------------- linear
class _Linear(Function):
    @staticmethod
    def forward(ctx, x, w, residual):
        C = _C()
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        if x2.stride(1) != 1:
            x2 = x2.contiguous()
        ctx.save_for_backward(x2, w)
        ctx.x_shape = x.shape
        ctx.has_res = residual is not None
        if residual is None:
            y = C.gemm(x2, w)
        else:
            y = C.gemm(x2, w, epi=C.EPI_BF16_ADD, aux=residual.reshape(-1, w.shape[0]))
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        C = _C()
        x2, w = ctx.saved_tensors
        N = w.shape[0]
        dy2 = dy.reshape(-1, N)
        if dy2.stride(1) != 1:
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = C.gemm(dy2, w, b_mn=True).view(ctx.x_shape)  # [M,N] @ [N,K]
        dw = None
        if ctx.needs_input_grad[1]:
            dw = _acc_or_return(w, lambda buf, acc: C.gemm(dy2, x2, a_mn=True, b_mn=True, out=buf,
                                                          epi=C.EPI_F32_ACC if acc else C.EPI_F32))
        return dx, dw, (dy if ctx.has_res else None)


def linear(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ w.T (+ residual)``; w is [out, in]."""
    if use_native(x, w):
        return _Linear.apply(x, w, residual)
    y = ref.linear(x, w)
    return y if residual is None else y + residual


# --------------------------------------------------------------------------- rmsnorm
class _RMSNorm(Function):
    @staticmethod
    def forward(ctx, x, w, eps, unit_offset, residual):
        y, rstd = _C().rmsnorm_fwd(x, w, eps, unit_offset, residual)
        ctx.save_for_backward(x, w, rstd)
        ctx.unit_offset = unit_offset
        ctx.has_res = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        C = _C()
        x, w, rstd = ctx.saved_tensors
        dy = dy.contiguous()
        dw = None
        if w is not None and ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)
            buf = mg if mg is not None else torch.zeros(w.shape, device=w.device, dtype=torch.float32)
            dx = C.rmsnorm_bwd(dy, x, w, rstd, ctx.unit_offset, buf)
            dw = None if mg is not None else buf.to(w.dtype)
        else:
            dx = C.rmsnorm_bwd(dy, x, w, rstd, ctx.unit_offset, None)
        return dx, dw, None, None, (dy if ctx.has_res else None)


class _RMSNormFork(Function):
    """``x -> (rmsnorm(x), x)``: the start of a pre-norm residual branch.  Autograd hands both gradients to ONE
    backward, so the gradient that arrives over the skip connection is added inside the norm's backward kernel
    (``dres_add``) instead of by a separate pass over the activations."""

    @staticmethod
    def forward(ctx, x, w, eps, unit_offset):
        y, rstd = _C().rmsnorm_fwd(x, w, eps, unit_offset, None)
        ctx.save_for_backward(x, w, rstd)
        ctx.unit_offset = unit_offset
        return y, x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dskip):
        C = _C()
        x, w, rstd = ctx.saved_tensors
        if dy is None:
            return dskip, None, None, None
        add = None if dskip is None else dskip.contiguous()
        mg = getattr(w, "main_grad", None) if w is not None else None
        buf = None
        if w is not None and ctx.needs_input_grad[1]:
            buf = mg if mg is not None else torch.zeros(w.shape, device=w.device, dtype=torch.float32)
        dx = C.rmsnorm_bwd(dy.contiguous(), x, w, rstd, ctx.unit_offset, buf, dres_add=add)
        dw = None if (buf is None or mg is not None) else buf.to(w.dtype)
        return dx, dw, None, None


def rmsnorm_fork(x: torch.Tensor, w: torch.Tensor | None, eps: float, unit_offset: bool = False):
    """``(rmsnorm(x) * (w | 1+w), x)``: use the second value as the residual of the branch that the first one
    enters; the two gradients are then merged inside the norm's backward kernel."""
    if use_native(x) and x.shape[-1] % 8 == 0 and torch.is_grad_enabled() and x.requires_grad:
        return _RMSNormFork.apply(x.contiguous(), w, eps, unit_offset)
    return rmsnorm(x, w, eps, unit_offset), x


def rmsnorm(x: torch.Tensor, w: torch.Tensor | None, eps: float, unit_offset: bool = False,
            residual: torch.Tensor | None = None) -> torch.Tensor:
    """``[residual +] rmsnorm(x) * (w | 1+w)``."""
    if use_native(x) and x.shape[-1] % 8 == 0:
        return _RMSNorm.apply(x.contiguous(), w, eps, unit_offset,
                              None if residual is None else residual.contiguous())
    return ref.rmsnorm(x, w, eps, unit_offset, residual)


# --------------------------------------------------------------------------- GLU
class _GLU(Function):
    @staticmethod
    def forward(ctx, gate_up, act):
        ctx.save_for_backward(gate_up)
        ctx.act = act
        return _C().glu_fwd(gate_up, act)

    @staticmethod
    def backward(ctx, dout):
        (gate_up,) = ctx.saved_tensors
        return _C().glu_bwd(gate_up, dout.contiguous(), ctx.act), None


def glu(gate_up: torch.Tensor, activation: str) -> torch.Tensor:
    """``act(gate) * up`` for ``gate_up = [gate | up]`` on the last dim."""
    if use_native(gate_up) and (gate_up.shape[-1] // 2) % 8 == 0:
        return _GLU.apply(gate_up, _ACT[activation])
    return ref.geglu(gate_up) if activation == "gelu_tanh" else ref.swiglu(gate_up)


class _GluMLP(Function):
    """``down(act(x w_gate^T) * (x w_up^T)) [+ residual]`` with the gated activation fused into the GEMM epilogues.

    Forward: the gate|up projection is one GEMM over the fused weight whose epilogue holds ``gate_j`` and ``up_j`` of
    the same unit in one accumulator row and writes both ``[gate | up]`` (kept for the backward pass) and the
    activation.  Backward: the input-gradient GEMM of the down projection produces ``d(act)`` in tensor memory and its
    epilogue applies the activation's derivative, so ``d(act)`` never exists in global memory and no stand-alone
    element-wise pass runs in either direction."""

    @staticmethod
    def forward(ctx, x, w_gu, w_down, residual, act, save_act):
        C = _C()
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        if x2.stride(1) != 1:
            x2 = x2.contiguous()
        gate_up, a = C.gemm_glu_fwd(x2, w_gu, act)
        D = w_down.shape[0]
        if residual is None:
            y = C.gemm(a, w_down)
        else:
            y = C.gemm(a, w_down, epi=C.EPI_BF16_ADD, aux=residual.reshape(-1, D))
        ctx.save_for_backward(x2, w_gu, w_down, gate_up, a if save_act else None)
        ctx.act, ctx.x_shape, ctx.has_res = act, x.shape, residual is not None
        return y.view(*x.shape[:-1], D)

    @staticmethod
    def backward(ctx, dy):
        C = _C()
        x2, w_gu, w_down, gate_up, a = ctx.saved_tensors
        D = w_down.shape[0]
        dy2 = dy.reshape(-1, D)
        if dy2.stride(1) != 1:
            dy2 = dy2.contiguous()
        if a is None:
            a = C.glu_fwd(gate_up, ctx.act)
        d_gu = C.gemm_glu_bwd(dy2, w_down, gate_up, ctx.act)
        dw_down = None
        if ctx.needs_input_grad[2]:
            dw_down = _acc_or_return(w_down, lambda buf, acc: C.gemm(dy2, a, a_mn=True, b_mn=True, out=buf,
                                                                      epi=C.EPI_F32_ACC if acc else C.EPI_F32))
        del a
        dx = C.gemm(d_gu, w_gu, b_mn=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        dw_gu = None
        if ctx.needs_input_grad[1]:
            dw_gu = _acc_or_return(w_gu, lambda buf, acc: C.gemm(d_gu, x2, a_mn=True, b_mn=True, out=buf,
                                                                  epi=C.EPI_F32_ACC if acc else C.EPI_F32))
        return dx, dw_gu, dw_down, (dy if ctx.has_res else None), None, None


def glu_mlp(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, activation: str,
            residual: torch.Tensor | None = None, save_act: bool = True) -> torch.Tensor:
    """Gated MLP ``down(act(gate) * up) [+ residual]`` with ``w_gate_up = [w_gate; w_up]`` ([2F, K]) and
    ``w_down`` [D, F].  ``save_act=False`` recomputes the activation in the backward pass instead of keeping it."""
    F2 = w_gate_up.shape[0]
    if use_native(x, w_gate_up) and (F2 // 2) % 128 == 0 and w_gate_up.is_contiguous() and w_down.is_contiguous() \
            and x.shape[-1] % 8 == 0 and _C().GEMM_TWO_CTA:
        return _GluMLP.apply(x, w_gate_up, w_down, residual, _ACT[activation], save_act)
    act = glu(linear(x, w_gate_up), activation)
    return linear(act, w_down, residual)


# --------------------------------------------------------------------------- embedding
class _Embedding(Function):
    @staticmethod
    def forward(ctx, tokens, w, scale):
        ctx.save_for_backward(tokens, w)
        ctx.scale = scale
        return _C().embedding_fwd(tokens, w, scale)

    @staticmethod
    def backward(ctx, dout):
        tokens, w = ctx.saved_tensors
        C = _C()
        dout = dout.contiguous()
        dw = _acc_or_return(w, lambda buf, acc: C.embedding_bwd(tokens, dout, buf, ctx.scale))
        return None, dw, None


def embedding(tokens: torch.Tensor, w: torch.Tensor, scale: float | None = None) -> torch.Tensor:
    if use_native(w) and w.shape[1] % 8 == 0:
        return _Embedding.apply(tokens, w, scale)
    return ref.embedding(tokens, w, scale)


# --------------------------------------------------------------------------- attention
def _run_starts(doc: torch.Tensor) -> torch.Tensor:
    """[B, S] int32: index of the first token of the contiguous run of equal ids that contains each token."""
    S = doc.shape[1]
    idx = torch.arange(S, device=doc.device, dtype=torch.int32)
    change = torch.ones_like(doc, dtype=torch.bool)
    change[:, 1:] = doc[:, 1:] != doc[:, :-1]
    return torch.where(change, idx[None], torch.zeros_like(doc)).cummax(dim=1).values.to(torch.int32)


def _run_ends(doc: torch.Tensor) -> torch.Tensor:
    """[B, S] int32: one past the last token of the run that contains each token."""
    S = doc.shape[1]
    idx = torch.arange(S, device=doc.device, dtype=torch.int32)
    change = torch.zeros_like(doc, dtype=torch.bool)
    change[:, 1:] = doc[:, 1:] != doc[:, :-1]
    nxt = torch.where(change, idx[None], torch.full_like(doc, S))
    suffix = nxt.flip(1).cummin(dim=1).values.flip(1)      # smallest run start at or after each position
    return torch.cat([suffix[:, 1:], torch.full_like(suffix[:, :1], S)], dim=1).to(torch.int32)


def kv_block_lower_bounds(S: int, block_q: int, window: int | None, doc: torch.Tensor | None, device,
                          batch: int = 1) -> torch.Tensor | None:
    """Per (batch, query block) lowest kv index any row of the block may attend to.

    Document ids must form contiguous runs (packed sequences); the bound for a row is
    ``max(start of its document, q - window)`` and the block takes the minimum over its rows.
    No host synchronisation.
    """
    plan = attention_plan(S, window, doc, device, batch=batch, block=block_q)
    return plan.lo_blk


def q_block_upper_bounds(S: int, block_kv: int, window: int | None, doc: torch.Tensor | None, device,
                         batch: int = 1) -> torch.Tensor | None:
    """Per (batch, kv block) exclusive upper bound on the query index that may attend to the block:
    ``min(end of the kv row's document, kv + window + 1)`` maximised over the block's rows."""
    plan = attention_plan(S, window, doc, device, batch=batch, block=block_kv)
    return plan.hi_blk


class AttnPlan:
    """Mask description for the attention kernels, built once per (document ids, window) and shared by every
    layer of a step.  With causal attention over packed documents (contiguous runs of equal ids) the mask
    ``kv <= q  and  q - kv <= window  and  doc[q] == doc[kv]`` is one interval per row:

    * ``kv_start[b, q]``: lowest admissible kv index of query row q = max(start of its document, q - window);
    * ``q_end[b, kv]``: one past the highest query row that may attend to kv = min(end of its document,
      kv + window + 1);
    * ``lo_blk`` / ``hi_blk``: the same bounds per block of 128 rows (minimum / maximum over the block), used to
      skip whole kv / query blocks.

    ``doc`` is kept only for non-causal attention, where the kernels compare ids element by element.
    All fields are None when there is neither a window nor document ids."""

    __slots__ = ("kv_start", "q_end", "lo_blk", "hi_blk", "doc")

    def __init__(self, kv_start=None, q_end=None, lo_blk=None, hi_blk=None, doc=None):
        self.kv_start, self.q_end, self.lo_blk, self.hi_blk, self.doc = kv_start, q_end, lo_blk, hi_blk, doc


def attention_plan(S: int, window: int | None, doc: torch.Tensor | None, device, batch: int = 1,
                   causal: bool = True, block: int = 128) -> AttnPlan:
    """Build the mask arrays on the device (a dozen small kernels, no host synchronisation)."""
    has_window = window is not None and window > 0
    if doc is None and not has_window:
        return AttnPlan()
    idx = torch.arange(S, device=device, dtype=torch.int32)
    if doc is not None:
        d = doc.to(device=device, dtype=torch.int32)
        start, end = _run_starts(d), _run_ends(d)
    else:
        start = torch.zeros(batch, S, device=device, dtype=torch.int32)
        end = torch.full((batch, S), S, device=device, dtype=torch.int32)
    if has_window:
        start = torch.maximum(start, (idx - window).clamp_min(0)[None].expand_as(start))
        end = torch.minimum(end, (idx + window + 1).clamp_max(S)[None].expand_as(end))
    nb = (S + block - 1) // block
    pad = nb * block - S
    sp = torch.nn.functional.pad(start, (0, pad), value=S) if pad else start
    ep = torch.nn.functional.pad(end, (0, pad), value=0) if pad else end
    lo = sp.view(sp.shape[0], nb, block).amin(dim=2).to(torch.int32).contiguous()
    hi = ep.view(ep.shape[0], nb, block).amax(dim=2).to(torch.int32).contiguous()
    if causal:
        return AttnPlan(start.contiguous(), end.contiguous(), lo, hi, None)
    # without the causal bound a row may also look ahead inside its document: the interval arrays above do not
    # describe that, so the kernels fall back to comparing ids (block bounds stay valid as lower / upper bounds
    # only for the causal part, so they are dropped too)
    return AttnPlan(None, None, None, None, None if doc is None else doc.to(device=device, dtype=torch.int32).contiguous())


_PLAN_CACHE: dict = {}


def cached_attention_plan(S: int, window: int | None, doc: torch.Tensor | None, device, batch: int,
                          causal: bool) -> AttnPlan:
    """``attention_plan`` memoised on the identity and version of the document-id tensor: all layers of a step
    (and the backward pass) share two plans, one for the windowed and one for the global layers."""
    key = (None if doc is None else (doc.data_ptr(), doc._version, tuple(doc.shape)), S, window if window else 0,
           batch, bool(causal), str(device))
    hit = _PLAN_CACHE.get(key)
    if hit is not None and (doc is None or hit[0] is doc):
        return hit[1]
    plan = attention_plan(S, window, doc, device, batch=batch, causal=causal)
    if len(_PLAN_CACHE) >= 8:
        _PLAN_CACHE.pop(next(iter(_PLAN_CACHE)))
    _PLAN_CACHE[key] = (doc, plan)  # holding ``doc`` keeps its address from being reused by another tensor
    return plan


def rope_table(inv_freq: torch.Tensor, max_pos: int, attn_factor: float = 1.0) -> torch.Tensor:
    """[max_pos, rot/2, 2] fp32 (cos, sin) table gathered by position id inside the kernels."""
    ang = torch.arange(max_pos, device=inv_freq.device, dtype=torch.float32)[:, None] * inv_freq.float()[None]
    return torch.stack([ang.cos() * attn_factor, ang.sin() * attn_factor], dim=-1).contiguous()


class _AttnBlock(Function):
    """qkv (packed) -> [QK-norm] -> RoPE -> masked GQA attention, one autograd node."""

    @staticmethod
    def forward(ctx, qkv, qw, kw, pos, cs, doc, H, KV, hd, layout, eps, unit_offset, scale, causal, window,
                recompute_qk):
        C = _C()
        B, S, _ = qkv.shape
        qkv2 = qkv.reshape(B * S, -1)
        pos32 = pos.reshape(-1).to(torch.int32).contiguous() if pos is not None else None
        need_qk = (qw is not None) or (cs is not None)
        if need_qk:
            qk = C.qknorm_rope_fwd(qkv2, qw, kw, pos32, cs, H, KV, hd, layout, eps, unit_offset)
        else:
            qk = qkv2
        q = qk[:, : H * hd].view(B, S, H, hd)
        k = qk[:, H * hd:(H + KV) * hd].view(B, S, KV, hd)
        v = qkv2[:, (H + KV) * hd:].view(B, S, KV, hd)
        plan = cached_attention_plan(S, window, doc, qkv.device, B, causal)
        out, lse = C.attn_fwd(q, k, v, scale, causal, window, plan)
        # per-op recomputation: the normalised and rotated q / k are rebuilt from the packed projection in backward
        # (one pass of the QK-norm + RoPE kernel) instead of being kept
        ctx.save_for_backward(qkv2, qk if (need_qk and not recompute_qk) else None, qw, kw, pos32, cs, out, lse)
        ctx.plan = plan
        ctx.cfg = (B, S, H, KV, hd, layout, eps, unit_offset, scale, causal, window, need_qk)
        return out.view(B, S, H * hd)

    @staticmethod
    def backward(ctx, dout):
        C = _C()
        qkv2, qk, qw, kw, pos32, cs, out, lse = ctx.saved_tensors
        B, S, H, KV, hd, layout, eps, unit_offset, scale, causal, window, need_qk = ctx.cfg
        if qk is None:
            qk = C.qknorm_rope_fwd(qkv2, qw, kw, pos32, cs, H, KV, hd, layout, eps, unit_offset) if need_qk else qkv2
        q = qk[:, : H * hd].view(B, S, H, hd)
        k = qk[:, H * hd:(H + KV) * hd].view(B, S, KV, hd)
        v = qkv2[:, (H + KV) * hd:].view(B, S, KV, hd)
        dqkv = torch.empty(B * S, (H + 2 * KV) * hd, device=dout.device, dtype=dout.dtype)
        C.attn_bwd(q, k, v, out, dout.reshape(B, S, H, hd).contiguous(), lse, dqkv, scale, causal, window, ctx.plan)
        dqw = dkw = None
        if need_qk:
            mq = getattr(qw, "main_grad", None) if qw is not None else None
            mk = getattr(kw, "main_grad", None) if kw is not None else None
            bq = mq if mq is not None else (torch.zeros(hd, device=dout.device) if qw is not None else None)
            bk = mk if mk is not None else (torch.zeros(hd, device=dout.device) if kw is not None else None)
            C.qknorm_rope_bwd(dqkv, qkv2, qw, kw, pos32, cs, bq, bk, H, KV, hd, layout, eps, unit_offset)
            dqw = None if (mq is not None or qw is None) else bq.to(qw.dtype)
            dkw = None if (mk is not None or kw is None) else bk.to(kw.dtype)
        return (dqkv.view(B, S, -1), dqw, dkw) + (None,) * 13


def attention_block(qkv: torch.Tensor, q_norm_w, k_norm_w, pos: torch.Tensor | None,
                    inv_freq: torch.Tensor | None, rope_cs: torch.Tensor | None, doc_ids: torch.Tensor | None,
                    n_heads: int, n_kv_heads: int, head_dim: int, *, layout: str = "half", eps: float = 1e-6,
                    unit_offset: bool = False, scale: float | None = None, causal: bool = True,
                    window: int | None = None, recompute_qk: bool = False) -> torch.Tensor:
    """Packed ``qkv`` [B,S,(H+2KV)*hd] → attention output [B,S,H*hd].

    Optional per-head RMSNorm on q and k, RoPE (``inv_freq`` for the reference path, ``rope_cs``
    table for the native path), then softmax attention with causal / inclusive sliding-window /
    same-document masking and GQA.  ``recompute_qk``: rebuild the normalised, rotated q / k in backward instead
    of keeping them (the per-op activation-recomputation policy).
    """
    B, S, _ = qkv.shape
    H, KV, hd = n_heads, n_kv_heads, head_dim
    scale = hd ** -0.5 if scale is None else scale
    if use_native(qkv) and hd in (64, 128, 256):
        if pos is None and rope_cs is not None:
            pos = torch.arange(S, device=qkv.device, dtype=torch.int32)[None].expand(B, S)
        return _AttnBlock.apply(qkv, q_norm_w, k_norm_w, pos, rope_cs, doc_ids, H, KV, hd,
                                0 if layout == "half" else 1, eps, unit_offset, scale, causal, window, recompute_qk)
    q, k, v = qkv.split([H * hd, KV * hd, KV * hd], dim=-1)
    q = q.reshape(B, S, H, hd)
    k = k.reshape(B, S, KV, hd)
    v = v.reshape(B, S, KV, hd)
    if pos is None:
        pos = torch.arange(S, device=qkv.device)[None].expand(B, S)
    q, k = ref.qk_norm_rope(q, k, q_norm_w, k_norm_w, pos, inv_freq, layout, eps, unit_offset)
    out = ref.attention(q, k, v, scale, causal, window, doc_ids)
    return out.reshape(B, S, H * hd)


# --------------------------------------------------------------------------- linear + cross-entropy
CE_CHUNK_ROWS = int(os.environ.get("MB_CE_CHUNK_ROWS", "4096"))   # rows of logits held at a time
CE_STORE_LIMIT_BYTES = 12 << 30
_BACKWARD_SCALE: float | None = None


@contextlib.contextmanager
def loss_backward_scale(scale: float | None):
    """Promise that ``backward`` will reach every loss computed inside this block with the output gradient
    ``scale`` (1 / gradient-accumulation steps in the trainer).  ``linear_cross_entropy`` then produces dH and dW
    chunk by chunk while the logits chunk is still at hand, so no logits or logit gradients outlive the forward
    pass; its backward checks the promise on the device and records a status error if it was broken."""
    global _BACKWARD_SCALE
    if os.environ.get("MB_CE_AHEAD", "1") == "0":   # keep the gradient chunks until backward instead (tuning runs)
        scale = None
    old, _BACKWARD_SCALE = _BACKWARD_SCALE, scale
    try:
        yield
    finally:
        _BACKWARD_SCALE = old


class _LinearCE(Function):
    """mean CE(h·Wᵀ, labels) over labels != -100 without holding all logits at once.

    Forward walks row chunks.  The logits GEMM's epilogue leaves per-tile (max, sum-exp) records and the target logit
    (online log-sum-exp: no separate pass over the logits); one kernel merges them per row, one pass turns the chunk
    into d(loss)/d(logits) in place.  With a promised output gradient (``loss_backward_scale``) the chunk is consumed
    at once by the dH and dW GEMMs and its buffer is reused by the next chunk; otherwise the gradient chunks are kept
    (or recomputed if they would exceed ``CE_STORE_LIMIT_BYTES``) and backward runs the two GEMMs per chunk.  dW
    accumulates in fp32 (directly into ``main_grad`` of a tied embedding).
    """

    @staticmethod
    def _chunk(C, h, w, labels, r0, r1, logit_scale, rec, loss_sum, gsl, buf, write_grad):
        logits, stats, tgt = C.gemm_ce(h[r0:r1], w, labels[r0:r1], 0, logit_scale,
                                       logits=None if buf is None else buf[: r1 - r0], store_logits=write_grad)
        C.ce_merge(stats, tgt, rec[r0:r1])
        C.ce_grad(logits, labels[r0:r1], [rec[r0:r1].data_ptr()], loss_sum, gsl, 0, write_grad, rows=r1 - r0)
        return logits

    @staticmethod
    def forward(ctx, h, w, labels, logit_scale, ahead, nvalid):
        C = _C()
        M, D = h.shape
        V = w.shape[0]
        labels = labels.reshape(-1).to(torch.int64).contiguous()
        if nvalid is None:
            nvalid = (labels != ref.IGNORE_INDEX).sum()
        nvalid = nvalid.detach().clamp_min(1).to(torch.float32)
        gs = (1.0 / nvalid).reshape(1)
        loss_sum = torch.zeros(1, device=h.device, dtype=torch.float32)
        rec = torch.empty(M, 4, device=h.device, dtype=torch.float32)
        need = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
        ahead = ahead if need else None
        store = need and ahead is None and (M * V * 2 <= CE_STORE_LIMIT_BYTES)
        gsl = gs * (logit_scale * (ahead if ahead is not None else 1.0))
        chunks, dh, dw_buf, buf = [], None, None, None
        mg = getattr(w, "main_grad", None)
        if ahead is not None:
            # dH of a chunk has few output tiles and a very long contraction (the vocabulary): accumulating in fp32
            # lets the GEMM cut the contraction into several work units per tile and fill its waves
            dh = torch.zeros(M, D, device=h.device, dtype=torch.float32)
            dw_buf = mg if mg is not None else torch.zeros(w.shape, device=w.device, dtype=torch.float32)
            buf = torch.empty(min(M, CE_CHUNK_ROWS), V, device=h.device, dtype=torch.bfloat16)
        for r0 in range(0, M, CE_CHUNK_ROWS):
            r1 = min(M, r0 + CE_CHUNK_ROWS)
            dl = _LinearCE._chunk(C, h, w, labels, r0, r1, logit_scale, rec, loss_sum, gsl, buf,
                                  store or ahead is not None)
            if ahead is not None:
                C.gemm(dl, w, b_mn=True, out=dh[r0:r1], epi=C.EPI_F32_ACC)                # [R,V] @ [V,D]
                C.gemm(dl, h[r0:r1], a_mn=True, b_mn=True, out=dw_buf, epi=C.EPI_F32_ACC)
            elif store:
                chunks.append(dl)
        ctx.ahead, ctx.store, ctx.logit_scale, ctx.has_mg = ahead, store, logit_scale, mg is not None
        if ahead is not None:
            ctx.save_for_backward(dh.to(h.dtype), *(() if mg is not None else (dw_buf,)))
        else:
            ctx.save_for_backward(h, w, labels, gsl, rec, *chunks)
        return (loss_sum * gs).reshape(())

    @staticmethod
    def backward(ctx, gout):
        C = _C()
        if ctx.ahead is not None:
            dh, *rest = ctx.saved_tensors
            C.expect_scalar(gout.detach().reshape(1).to(torch.float32).contiguous(), ctx.ahead)
            return dh, (None if ctx.has_mg else rest[0].to(dh.dtype)), None, None, None, None
        h, w, labels, gsl, rec, *chunks = ctx.saved_tensors
        M, D = h.shape
        g = gout.reshape(1).to(torch.float32).contiguous()
        dh = torch.zeros(M, D, device=h.device, dtype=torch.float32)
        mg = getattr(w, "main_grad", None)
        dw_buf = mg if mg is not None else torch.zeros(w.shape, device=w.device, dtype=torch.float32)
        for i, r0 in enumerate(range(0, M, CE_CHUNK_ROWS)):
            r1 = min(M, r0 + CE_CHUNK_ROWS)
            if ctx.store:
                dl = chunks[i]
            else:  # the row records are kept: only the logits are recomputed
                dl = C.gemm(h[r0:r1], w, alpha=ctx.logit_scale)
                C.ce_grad(dl, labels[r0:r1], [rec[r0:r1].data_ptr()], None, gsl, 0, True)
            C.gemm(dl, w, b_mn=True, out=dh[r0:r1], epi=C.EPI_F32_ACC, alpha_dev=g)   # [R,V] @ [V,D]
            C.gemm(dl, h[r0:r1], a_mn=True, b_mn=True, out=dw_buf, epi=C.EPI_F32_ACC, alpha_dev=g)
        dw = None if mg is not None else dw_buf.to(w.dtype)
        return dh.to(h.dtype), dw, None, None, None, None


def linear_cross_entropy(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor,
                         logit_scale: float = 1.0, nvalid: torch.Tensor | None = None) -> torch.Tensor:
    """Mean cross-entropy of ``h @ w.T * logit_scale`` against ``labels`` (ignore_index = -100).

    ``nvalid`` (0-d tensor) replaces the count of valid labels as the divisor: a rank that holds a slice of the
    tokens passes the count over all slices, and the sum of the ranks' results is the mean over all tokens."""
    h2 = h.reshape(-1, h.shape[-1])
    if use_native(h2, w) and w.shape[0] % 8 == 0:
        return _LinearCE.apply(h2.contiguous(), w, labels, logit_scale, _BACKWARD_SCALE, nvalid)
    if nvalid is None:
        return ref.linear_cross_entropy(h2, w, labels.reshape(-1), logit_scale)
    total = ref.linear_cross_entropy(h2, w, labels.reshape(-1), logit_scale, reduction="sum")
    return total / nvalid.detach().clamp_min(1).to(total.dtype)


# --------------------------------------------------------------------------- grouped (expert) linear
GROUP_ALIGN = 128  # row groups are padded to the GEMM tile height


def padded_group_offsets(counts: torch.Tensor, align: int = GROUP_ALIGN) -> torch.Tensor:
    """int32 [E+1] start offsets of groups whose sizes are rounded up to ``align`` (no host sync)."""
    padded = (counts.to(torch.int64) + align - 1) // align * align
    offs = torch.zeros(counts.numel() + 1, dtype=torch.int64, device=counts.device)
    offs[1:] = padded.cumsum(0)
    return offs.to(torch.int32)


class _GroupedLinear(Function):
    @staticmethod
    def forward(ctx, x, w, offs):
        C = _C()
        ctx.save_for_backward(x, w, offs)
        return C.gemm_grouped_rows(x, w, offs, b_mn=True)

    @staticmethod
    def backward(ctx, dy):
        C = _C()
        x, w, offs = ctx.saved_tensors
        dy = dy.contiguous()
        dx = C.gemm_grouped_rows(dy, w, offs, b_mn=False) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)
            buf = mg if mg is not None else torch.zeros(w.shape, device=w.device, dtype=torch.float32)
            C.gemm_grouped_contr(x, dy, offs, buf)
            dw = None if mg is not None else buf.to(w.dtype)
        return dx, dw, None


class _GroupedSwiGLU(Function):
    """Whole expert FFN ``(silu(x w1) * (x w3)) w2`` over padded row groups.  Gate and up projections write the
    two halves of one ``[rows, 2*hidden]`` buffer (no concatenation); the activation is recomputed in the
    backward pass instead of being saved."""

    @staticmethod
    def forward(ctx, x, w1, w3, w2, offs, out_box=None):
        # out_box: optional one-element list holding a preallocated [rows, dim] output (e.g. a peer-visible buffer)
        C = _C()
        H = w1.shape[2]
        h13 = torch.empty(x.shape[0], 2 * H, device=x.device, dtype=x.dtype)
        C.gemm_grouped_rows(x, w1, offs, b_mn=True, out=h13[:, :H])
        C.gemm_grouped_rows(x, w3, offs, b_mn=True, out=h13[:, H:])
        ctx.save_for_backward(x, w1, w3, w2, offs, h13)
        out = out_box[0] if out_box else None
        return C.gemm_grouped_rows(C.glu_fwd(h13, _ACT["silu"]), w2, offs, b_mn=True, out=out)

    @staticmethod
    def backward(ctx, dy):
        C = _C()
        x, w1, w3, w2, offs, h13 = ctx.saved_tensors
        H = w1.shape[2]
        dy = dy.contiguous()
        act = C.glu_fwd(h13, _ACT["silu"])
        dact = C.gemm_grouped_rows(dy, w2, offs, b_mn=False)
        d13 = C.glu_bwd(h13, dact, _ACT["silu"])
        del dact
        grads = []
        for w, a, b in ((w1, x, d13[:, :H]), (w3, x, d13[:, H:]), (w2, act, dy)):
            mg = getattr(w, "main_grad", None)
            buf = mg if mg is not None else torch.zeros(w.shape, device=w.device, dtype=torch.float32)
            C.gemm_grouped_contr(a, b, offs, buf)
            grads.append(None if mg is not None else buf.to(w.dtype))
        dx = None
        if ctx.needs_input_grad[0]:
            dx = C.gemm_grouped_rows(d13[:, :H], w1, offs, b_mn=False)
            dx.add_(C.gemm_grouped_rows(d13[:, H:], w3, offs, b_mn=False))
        return dx, grads[0], grads[1], grads[2], None, None


def grouped_swiglu(x: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor, w2: torch.Tensor, offs: torch.Tensor,
                   out: torch.Tensor | None = None):
    """Expert FFN over padded row groups: ``w1, w3: [E, dim, hidden]``, ``w2: [E, hidden, dim]``.  ``out`` (optional,
    [rows, dim], contiguous) receives the result on the native path; the returned tensor is the result either way."""
    H = w1.shape[2]
    if (use_native(x, w1) and x.shape[0] % GROUP_ALIGN == 0 and w1.shape[1] % 64 == 0 and H % 64 == 0
            and x.is_contiguous()):
        return _GroupedSwiGLU.apply(x, w1, w3, w2, offs, [out] if out is not None else None)
    h1 = grouped_linear(x, w1, offs)
    h3 = grouped_linear(x, w3, offs)
    return grouped_linear(glu(torch.cat([h1, h3], dim=-1), "silu"), w2, offs)


def grouped_linear(x: torch.Tensor, w: torch.Tensor, offs: torch.Tensor, counts: torch.Tensor | None = None):
    """``y[rows of group e] = x[rows of group e] @ w[e]`` with w: [E, in, out].

    ``offs`` are the padded int32 offsets of the groups inside ``x`` (see ``padded_group_offsets``); rows
    between a group's real size and its padded size must be zero.
    """
    if use_native(x, w) and x.shape[0] % GROUP_ALIGN == 0 and w.shape[1] % 64 == 0 and w.shape[2] % 8 == 0:
        return _GroupedLinear.apply(x, w, offs)
    out = x.new_zeros(x.shape[0], w.shape[2])
    bounds = offs.tolist()
    for e in range(w.shape[0]):
        lo, hi = bounds[e], bounds[e + 1]
        if hi > lo:
            out[lo:hi] = x[lo:hi] @ w[e]
    return out
