"""Plain-PyTorch definitions of every hot op: the CPU execution path and the numerics oracle.

Every function here is differentiable through ordinary autograd and computes in fp32 internally.
The CUDA kernels in ``maester_b200/csrc`` are tested against these.  Semantics follow the
reference models: Gemma RMSNorm ``x̂·(1+w)`` in fp32 (maester/models/gemma/model.py:155-175),
half-split and interleaved RoPE (gemma/model.py:97-106, llama/model.py:133-168), inclusive sliding
window ``0 <= q-kv <= W`` AND same-document (gemma/model.py:203-256), tanh-GELU GeGLU
(gemma/model.py:189-195), SwiGLU (llama/model.py:308-309), mean cross-entropy with
``ignore_index=-100``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

IGNORE_INDEX = -100


def rmsnorm(x: torch.Tensor, w: torch.Tensor | None, eps: float, unit_offset: bool = False,
            residual: torch.Tensor | None = None) -> torch.Tensor:
    """``residual + x * rsqrt(mean(x², -1) + eps) * (w or 1+w)``; fp32 math, result in x.dtype."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if w is not None:
        y = y * ((1.0 + w.float()) if unit_offset else w.float())
    y = y.to(x.dtype)
    if residual is not None:
        y = residual + y
    return y


def layernorm(x, w, b, eps):
    return F.layer_norm(x.float(), (x.shape[-1],), None if w is None else w.float(),
                        None if b is None else b.float(), eps).to(x.dtype)


def rope_inv_freq(rot_dim: int, theta: float, scaling_factor: float = 1.0, device=None) -> torch.Tensor:
    """``theta^(-2i/rot_dim) / scaling_factor`` for i in [0, rot_dim/2), fp32."""
    idx = torch.arange(0, rot_dim, 2, device=device)[: rot_dim // 2].float()
    return (1.0 / (theta ** (idx / rot_dim))) / scaling_factor


def apply_rope(x: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, layout: str,
               attn_factor: float = 1.0) -> torch.Tensor:
    """Rotate the first ``2*len(inv_freq)`` channels of every head.

    x: [B, S, H, hd]; pos: [B, S] integer positions; layout "half" pairs channel i with i+rot/2,
    "interleaved" pairs 2i with 2i+1.  Channels beyond the rotary width pass through.
    """
    rot = inv_freq.numel() * 2
    ang = pos.to(torch.float32)[..., None] * inv_freq.to(torch.float32)  # [B,S,rot/2]
    cos = (ang.cos() * attn_factor)[:, :, None, :]
    sin = (ang.sin() * attn_factor)[:, :, None, :]
    xr = x[..., :rot].float()
    if layout == "half":
        a, b = xr[..., : rot // 2], xr[..., rot // 2:]
        out = torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)
    elif layout == "interleaved":
        a, b = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).flatten(-2)
    else:
        raise ValueError(f"unknown rope layout {layout}")
    out = out.to(x.dtype)
    if rot < x.shape[-1]:
        out = torch.cat([out, x[..., rot:]], dim=-1)
    return out


def qk_norm_rope(q, k, q_w, k_w, pos, inv_freq, layout, eps, unit_offset):
    """Optional per-head RMSNorm of q and k (weights of size head_dim) followed by RoPE."""
    if q_w is not None:
        q = rmsnorm(q, q_w, eps, unit_offset)
    if k_w is not None:
        k = rmsnorm(k, k_w, eps, unit_offset)
    if inv_freq is not None:
        q = apply_rope(q, pos, inv_freq, layout)
        k = apply_rope(k, pos, inv_freq, layout)
    return q, k


def attention_mask(seq_q: int, seq_kv: int, causal: bool, window: int | None,
                   doc_ids: torch.Tensor | None, device=None, q_offset: int = 0) -> torch.Tensor:
    """Dense boolean mask [B or 1, 1, Sq, Skv]; True = attend."""
    q = torch.arange(seq_q, device=device)[:, None] + q_offset
    kv = torch.arange(seq_kv, device=device)[None, :]
    m = torch.ones(seq_q, seq_kv, dtype=torch.bool, device=device)
    if causal:
        m = m & (q >= kv)
    if window is not None and window > 0:
        m = m & (q - kv <= window)
    m = m[None, None]
    if doc_ids is not None:
        d = doc_ids.to(device)
        same = d[:, q_offset:q_offset + seq_q, None] == d[:, None, :seq_kv]
        m = m & same[:, None]
    return m


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, causal: bool = True,
              window: int | None = None, doc_ids: torch.Tensor | None = None,
              return_lse: bool = False):
    """Masked softmax attention with GQA.  q: [B,S,H,hd], k/v: [B,S,KV,hd(v)] → [B,S,H,hd_v]."""
    B, S, H, _ = q.shape
    KV = k.shape[2]
    g = H // KV
    qf = q.float().permute(0, 2, 1, 3)  # B,H,S,hd
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    scores = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    mask = attention_mask(S, k.shape[1], causal, window, doc_ids, device=q.device)
    scores = scores.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(scores, dim=-1)
    p = torch.exp(scores - lse[..., None])
    p = torch.where(mask, p, torch.zeros_like(p))
    out = torch.matmul(p, vf).permute(0, 2, 1, 3).to(q.dtype)
    if return_lse:
        return out, lse
    return out


def geglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``gelu_tanh(gate) * up`` for gate_up = [gate | up] concatenated on the last dim."""
    g, u = gate_up.float().chunk(2, dim=-1)
    return (F.gelu(g, approximate="tanh") * u).to(gate_up.dtype)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    g, u = gate_up.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gate_up.dtype)


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return F.linear(x, w)


def embedding(tokens: torch.Tensor, w: torch.Tensor, scale: float | None = None) -> torch.Tensor:
    h = F.embedding(tokens, w)
    if scale is not None:
        h = h * torch.tensor(scale, dtype=h.dtype, device=h.device)
    return h


def linear_cross_entropy(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor,
                         logit_scale: float = 1.0, reduction: str = "mean") -> torch.Tensor:
    """CE(h·Wᵀ·logit_scale, labels) with ignore_index=-100; softmax in fp32."""
    logits = F.linear(h, w).float() * logit_scale
    return F.cross_entropy(logits, labels, ignore_index=IGNORE_INDEX, reduction=reduction)


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    return F.cross_entropy(logits.float().flatten(0, -2), labels.flatten(), ignore_index=IGNORE_INDEX)


def adamw_step(p32, g32, m, v, step: int, lr: float, beta1: float, beta2: float, eps: float,
               wd: float, grad_scale: float = 1.0, out_lp: torch.Tensor | None = None) -> None:
    """Decoupled AdamW on fp32 tensors in place; optionally emits a low-precision copy of p."""
    g = g32 * grad_scale
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p32.mul_(1 - lr * wd).addcdiv_(m, denom, value=-lr / bc1)
    if out_lp is not None:
        out_lp.copy_(p32)


def newton_schulz(g: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """Quintic Newton–Schulz orthogonalisation in bf16 (maester/optimizers/muon.py:22-49)."""
    a, b, c = 3.4445, -4.7750, 2.0315
    x = g.to(torch.bfloat16)
    transposed = x.shape[-2] > x.shape[-1]
    if transposed:
        x = x.mT
    x = x / (x.norm(dim=(-2, -1), keepdim=True) + eps)
    for _ in range(steps):
        A = x @ x.mT
        Bm = b * A + (c * A) @ A   # the scaled matrix is the left factor, as in the reference: same bf16 roundings
        x = a * x + Bm @ x
    if transposed:
        x = x.mT
    return x
