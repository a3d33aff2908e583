"""Optimizers for MoE models with the auxiliary-loss-free load-balancing hook.

A step pre-hook on the optimizer container (reference: maester/models/deepseek/optimizer.py:14-222)
visits every MoE layer: sums ``tokens_per_expert`` over the data-parallel group, updates
``expert_bias += coeff * sign(mean - tokens)`` (then re-centres the bias to zero mean) and zeroes the
counter.  Balance statistics — max violation, coefficient of variation, fraction of "dead" experts
(load below 5 % of the ideal) for the batch and as running totals — are published in
``optimizers._hook_stats`` for the metric logger.

All layers are processed with one stacked all-reduce and one device-to-host transfer per step (the
reference issues one of each per layer).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from maester_b200.optimizers.container import OptimizersContainer, build_optimizers

_DEAD_THRESHOLD_FRACTION = 0.05


class _MoEBalanceTracker:
    """Running per-layer totals of tokens per expert."""

    def __init__(self):
        self.totals: torch.Tensor | None = None  # [layers, experts] on CPU
        self.batches = 0

    def update(self, tokens: torch.Tensor) -> dict[str, torch.Tensor]:
        self.totals = tokens.clone() if self.totals is None else self.totals + tokens
        self.batches += 1
        return _balance_stats(self.totals)


def _balance_stats(tokens: torch.Tensor) -> dict[str, torch.Tensor]:
    """tokens: [layers, experts] → per-layer maxvio / cv / dead fraction."""
    expected = tokens.sum(dim=1, keepdim=True) / tokens.shape[1]
    safe = expected.clamp_min(1e-12)
    maxvio = (tokens.max(dim=1, keepdim=True).values - expected) / safe
    cv = tokens.std(dim=1, unbiased=False, keepdim=True) / safe
    dead = (tokens <= expected * _DEAD_THRESHOLD_FRACTION).float().mean(dim=1, keepdim=True)
    zero = expected <= 0
    return {"maxvio": torch.where(zero, torch.zeros_like(maxvio), maxvio).squeeze(1),
            "cv": torch.where(zero, torch.zeros_like(cv), cv).squeeze(1),
            "dead_frac": torch.where(zero, torch.zeros_like(dead), dead).squeeze(1)}


def _moe_modules(model: nn.Module) -> list[nn.Module]:
    layers = getattr(model, "layers", None)
    if layers is None:
        return []
    vals = layers.values() if isinstance(layers, nn.ModuleDict) else layers
    return [l.moe for l in vals if getattr(l, "moe_enabled", False) and hasattr(l.moe, "tokens_per_expert")]


def build_deepseek_optimizers(model: nn.Module, cfg, parallel_dims) -> OptimizersContainer:
    optimizers = build_optimizers(model, cfg, parallel_dims)
    optimizers._hook_stats = {}
    tracker = _MoEBalanceTracker()
    optimizers._moe_balance_tracker = tracker

    def update_expert_bias(*_args, **_kw) -> None:
        moes = _moe_modules(model)
        optimizers._hook_stats.clear()
        if not moes:
            return
        with torch.no_grad():
            tokens = torch.stack([m.tokens_per_expert for m in moes])  # [L, E]
            if parallel_dims is not None and parallel_dims.dp_enabled and dist.is_initialized():
                group = parallel_dims.mesh_group("dp")
                dist.all_reduce(tokens, op=dist.ReduceOp.SUM, group=group)
            for i, m in enumerate(moes):
                if m.load_balance_coeff is not None and m.expert_bias is not None:
                    t = tokens[i]
                    delta = m.load_balance_coeff * torch.sign(t.mean() - t)
                    m.expert_bias.add_(delta - delta.mean())
                m.tokens_per_expert.zero_()
            tokens_cpu = tokens.float().cpu()  # the only host transfer of the hook
        batch = _balance_stats(tokens_cpu)
        running = tracker.update(tokens_cpu)
        st = optimizers._hook_stats
        for key, vals in (("batch", batch), ("global", running)):
            st[f"expert_balance/{key}_maxvio_mean"] = vals["maxvio"].mean().item()
            st[f"expert_balance/{key}_maxvio_max"] = vals["maxvio"].max().item()
            st[f"expert_balance/{key}_cv_mean"] = vals["cv"].mean().item()
            st[f"expert_balance/{key}_dead_frac_mean"] = vals["dead_frac"].mean().item()
        st["expert_balance/batches"] = tracker.batches
        if cfg.enable_wandb:
            try:
                import wandb
                for i, m in enumerate(moes):
                    if m.expert_bias is not None:
                        st[f"expert_balance/bias_hist_layer{i}"] = wandb.Histogram(m.expert_bias.float().cpu().numpy())
            except ImportError:
                pass

    optimizers.register_step_pre_hook(update_expert_bias)
    return optimizers
