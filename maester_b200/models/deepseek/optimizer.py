"""Optimizers for MoE models with the auxiliary-loss-free load-balancing hook.

A step pre-hook on the optimizer container (reference: maester/models/deepseek/optimizer.py:14-222)
visits every MoE layer: sums ``tokens_per_expert`` over the data-parallel group, updates
``expert_bias += coeff * sign(mean - tokens)`` (then re-centres the bias to zero mean) and zeroes the
counter.  Balance statistics — max violation, coefficient of variation, fraction of "dead" experts
(load below 5 % of the ideal) for the batch and as running totals — are published in
``optimizers._hook_stats`` for the metric logger.

All layers are processed with one stacked all-reduce per step (the reference issues one per layer).  The
statistics stay on the device: ``optimizers._hook_stats`` is a mapping that computes its values, with ONE
device-to-host transfer, the first time it is read after a step (the metric logger reads it on log steps only), so
the optimizer step itself never waits for the GPU.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from maester_b200.optimizers.container import OptimizersContainer, build_optimizers

_DEAD_THRESHOLD_FRACTION = 0.05


class _MoEBalanceTracker:
    """Running per-layer totals of tokens per expert (kept where the counters live)."""

    def __init__(self):
        self.totals: torch.Tensor | None = None  # [layers, experts]
        self.batches = 0

    def update(self, tokens: torch.Tensor) -> None:
        self.totals = tokens.clone() if self.totals is None else self.totals + tokens
        self.batches += 1


class _LazyStats(dict):
    """Mapping of balance statistics that is filled in on first read (one host transfer of two small tensors)."""

    def __init__(self):
        super().__init__()
        self._pending = None   # (batch tokens, running totals, batches, extra) still on the device

    def defer(self, batch: torch.Tensor, totals: torch.Tensor, batches: int, extra) -> None:
        super().clear()
        self._pending = (batch, totals, batches, extra)

    def clear(self) -> None:
        super().clear()
        self._pending = None

    def _fill(self) -> None:
        if self._pending is None:
            return
        batch, totals, batches, extra = self._pending
        self._pending = None
        both = torch.stack([batch.float(), totals.float()]).cpu()   # the only host transfer
        # the reference's metric names (maester/models/deepseek/optimizer.py:181-203): average, maximum and minimum
        # over the MoE layers of each statistic, for this step's batch and for the running totals
        for kind, vals in (("batch", _balance_stats(both[0])), ("global", _balance_stats(both[1]))):
            for stat in ("maxvio", "dead_frac", "cv"):
                v = vals[stat]
                super().__setitem__(f"expert_balance/{stat}_{kind}_avg", v.mean().item())
                super().__setitem__(f"expert_balance/{stat}_{kind}_max", v.max().item())
                super().__setitem__(f"expert_balance/{stat}_{kind}_min", v.min().item())
        super().__setitem__("expert_balance/batches", batches)
        if extra is not None:
            for k, v in extra().items():
                super().__setitem__(k, v)

    def __getitem__(self, k):
        self._fill()
        return super().__getitem__(k)

    def __contains__(self, k):
        self._fill()
        return super().__contains__(k)

    def __iter__(self):
        self._fill()
        return super().__iter__()

    def __len__(self):
        self._fill()
        return super().__len__()

    def __bool__(self):
        return self._pending is not None or super().__len__() > 0

    def keys(self):
        self._fill()
        return super().keys()

    def items(self):
        self._fill()
        return super().items()

    def values(self):
        self._fill()
        return super().values()

    def get(self, k, default=None):
        self._fill()
        return super().get(k, default)


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


def _moe_modules(model: nn.Module, with_names: bool = False) -> list:
    layers = getattr(model, "layers", None)
    if layers is None:
        return []
    named = layers.items() if isinstance(layers, nn.ModuleDict) else ((str(i), l) for i, l in enumerate(layers))
    found = [(n, l.moe) for n, l in named if getattr(l, "moe_enabled", False) and hasattr(l.moe, "tokens_per_expert")]
    return found if with_names else [m for _, m in found]


def build_deepseek_optimizers(model: nn.Module, cfg, parallel_dims) -> OptimizersContainer:
    optimizers = build_optimizers(model, cfg, parallel_dims)
    optimizers._hook_stats = _LazyStats()
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
            tracker.update(tokens)

        def histograms() -> dict:
            out = {}
            if cfg.enable_wandb:
                try:
                    import wandb
                    for name, m in _moe_modules(model, with_names=True):   # keyed by the layer's name in the model
                        if m.expert_bias is not None:
                            out[f"expert_balance_bias/layer{name}"] = wandb.Histogram(m.expert_bias.float().cpu().tolist())
                except ImportError:
                    pass
            return out

        optimizers._hook_stats.defer(tokens, tracker.totals.clone(), tracker.batches, histograms)

    optimizers.register_step_pre_hook(update_expert_bias)
    return optimizers
