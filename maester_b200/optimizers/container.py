"""Several optimizers behind one ``Optimizer`` facade, and the builders that assign parameters.

Reference behaviour (maester/optimizers/container.py:16-239): the container exposes the
concatenated ``param_groups`` so that one LR scheduler drives every optimizer, supports step
pre/post hooks, and prefixes state-dict keys with ``opt{i}_`` when it holds more than one
optimizer.  ``build_optimizers`` implements the two assignment schemes: the muP three-group rule
and first-match-wins ``optimizer_groups`` (``min_dim``, ``exclude_names``, import-string class).

Parameters come from the sharding runtime when the model has one (fp32 master shards whose
``.grad`` are views of the reduced gradient shard); the names used for matching and for
state-dict keys are the model's fully-qualified parameter names either way.
"""
from __future__ import annotations

import importlib
import os
from typing import Any

import torch
from torch.distributed.checkpoint.stateful import Stateful
from torch.optim import Optimizer

from maester_b200.log_utils import logger
from maester_b200.optimizers.adamw import FusedAdamW

# peer-memory sharding runtime: update each unit under the backward pass ("0": one kernel for all units in step())
EAGER_UNIT_UPDATES = os.environ.get("MB_FSDP_EAGER", "1") != "0"


def _named_trainable(model: torch.nn.Module) -> list[tuple[str, torch.nn.Parameter]]:
    sharded = getattr(model, "_sharded", None)
    if sharded is not None:
        return [(n, p) for n, p in sharded.named_master_parameters() if p.requires_grad]
    return [(n, p) for n, p in model.named_parameters() if p.requires_grad]


def _import(path: str):
    """Class by dotted path.  Paths into the reference's package (``maester.optimizers.Muon``, the default of its
    ``optimizer_groups``, maester/config.py:132-157) name this package's class of the same name, so a job directory
    written by the reference's tooling runs unchanged."""
    if path.startswith("maester."):
        path = "maester_b200." + path[len("maester."):]
    mod, _, name = path.rpartition(".")
    return getattr(importlib.import_module(mod), name)


class OptimizersContainer(Optimizer, Stateful):
    def __init__(self, model: torch.nn.Module, optimizers: list[Optimizer], names: dict[int, str] | None = None):
        self.model = model
        self.optimizers = optimizers
        all_params = [p for opt in optimizers for g in opt.param_groups for p in g["params"]]
        Optimizer.__init__(self, all_params, defaults={})
        # share the group dicts: a scheduler that rewrites group["lr"] reaches the real optimizers
        self.param_groups = [g for opt in optimizers for g in opt.param_groups]
        self._names = names or {}
        self._hook_stats: dict[str, Any] = {}

    # -- stepping
    def announce_step(self) -> bool:
        """Call before the backward pass whose gradients the next ``step()`` consumes (the last micro-batch), when
        nothing has to look at the complete gradient first (no clipping by the global norm).  With the peer-memory
        sharding runtime every unit is then reduced, updated and re-gathered by its own kernel launch as soon as
        its gradients are complete, under the backward pass of the earlier blocks, instead of all at once in
        ``step()``.  Returns whether that mode is on for this step."""
        sharded = getattr(self.model, "_sharded", None)
        if sharded is None or not sharded.fused or not EAGER_UNIT_UPDATES:
            return False
        if not all(isinstance(o, FusedAdamW) and o._flat is not None for o in self.optimizers):
            return False
        if not all(o.eager_begin() for o in self.optimizers):
            return False
        sharded.eager_active = True
        return True

    def step(self, closure=None):  # hooks registered on the container wrap this method
        loss = None
        sharded = getattr(self.model, "_sharded", None)
        if sharded is not None and sharded.fused:
            if not all(isinstance(o, FusedAdamW) and o._flat is not None for o in self.optimizers):
                raise RuntimeError("fused_collectives=True needs every optimizer group to be AdamW; "
                                   "set fused_collectives=False to use other optimizers")
            sharded.pre_optimizer_step()
        for opt in self.optimizers:
            out = opt.step(closure) if closure is not None else opt.step()
            loss = out if out is not None else loss
        if sharded is not None:
            if sharded.eager_active:
                sharded.eager_active = False
                for u in sharded.units:
                    u.eager_done = False
            sharded.lowp_fresh = sharded.device.type == "cuda" and all(
                isinstance(o, FusedAdamW) and o._flat is not None for o in self.optimizers)
            # every parameter's gradient was consumed and cleared by a kernel that owns it: zero_grad() may skip
            if sharded.grad_cleared_by_optimizer is not None:
                sharded.grad_cleared_by_optimizer = all(getattr(o, "cleared_grad", False) for o in self.optimizers)
            for o in self.optimizers:
                if hasattr(o, "cleared_grad"):
                    o.cleared_grad = False
            sharded.gather_params()
        return loss

    def zero_grad(self, set_to_none: bool = True) -> None:
        sharded = getattr(self.model, "_sharded", None)
        if sharded is not None:
            sharded.zero_grad()  # gradients are views of flat buffers: zero in place, never drop them
            return
        for opt in self.optimizers:
            opt.zero_grad(set_to_none=set_to_none)

    def train(self) -> None:
        for opt in self.optimizers:
            if hasattr(opt, "train"):
                opt.train()

    # -- state
    def _opt_state(self, opt: Optimizer) -> dict[str, Any]:
        """State dict keyed by parameter FQN (flat ``state.<fqn>.<key>`` entries plus param_groups)."""
        out: dict[str, Any] = {}
        for g in opt.param_groups:
            for p in g["params"]:
                fqn = self._names.get(id(p), str(id(p)))
                for k, v in opt.state.get(p, {}).items():
                    out[f"state.{fqn}.{k}"] = v
        groups = []
        for g in opt.param_groups:
            gg = {k: v for k, v in g.items() if k != "params"}
            gg["params"] = [self._names.get(id(p), str(id(p))) for p in g["params"]]
            groups.append(gg)
        out["param_groups"] = groups
        return out

    def _load_opt_state(self, opt: Optimizer, sd: dict[str, Any]) -> None:
        by_name = {self._names.get(id(p), str(id(p))): p for g in opt.param_groups for p in g["params"]}
        for key, val in sd.items():
            if not key.startswith("state."):
                continue
            fqn, _, k = key[len("state."):].rpartition(".")
            p = by_name.get(fqn)
            if p is None:
                continue
            st = opt.state.setdefault(p, {})
            if torch.is_tensor(st.get(k)) and torch.is_tensor(val) and st[k].shape == val.shape:
                st[k].copy_(val)  # keep views into flat optimizer buffers intact
            else:
                st[k] = val
        for g, saved in zip(opt.param_groups, sd.get("param_groups", [])):
            for k, v in saved.items():
                if k != "params":
                    g[k] = v

    def state_dict(self) -> dict[str, Any]:
        if len(self.optimizers) == 1:
            return self._opt_state(self.optimizers[0])
        out: dict[str, Any] = {}
        for i, opt in enumerate(self.optimizers):
            for k, v in self._opt_state(opt).items():
                out[f"opt{i}_{k}"] = v
        return out

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        if len(self.optimizers) == 1:
            self._load_opt_state(self.optimizers[0], state_dict)
            return
        for i, opt in enumerate(self.optimizers):
            pre = f"opt{i}_"
            self._load_opt_state(opt, {k[len(pre):]: v for k, v in state_dict.items() if k.startswith(pre)})


def _make_optimizer(opt_class, params_or_groups, opt_cfg: dict, model) -> Optimizer:
    cfg = dict(opt_cfg)
    sharded = getattr(model, "_sharded", None)
    if opt_class is torch.optim.AdamW and sharded is not None:
        opt_class = FusedAdamW  # same arithmetic, one launch over the flat shard
    if opt_class is FusedAdamW:
        cfg.pop("fused", None)
    elif opt_class is torch.optim.AdamW and not torch.cuda.is_available():
        cfg.pop("fused", None)
    if "betas" in cfg:
        cfg["betas"] = tuple(cfg["betas"])
    opt = opt_class(params_or_groups, **cfg)
    if sharded is not None and hasattr(opt, "attach_sharding"):
        opt.attach_sharding(sharded)
    if isinstance(opt, FusedAdamW) and sharded is not None:
        seg = sharded.flat_segments()
        mine = {p: seg[p] for g in opt.param_groups for p in g["params"]}
        if not hasattr(sharded, "adam_m"):  # one pair of state buffers shared by every FusedAdamW
            sharded.adam_m = torch.zeros_like(sharded.master)
            sharded.adam_v = torch.zeros_like(sharded.master)
        opt.attach_flat(sharded.master, sharded.shard_grad, sharded.shard_lp, mine, sharded.adam_m, sharded.adam_v)
        opt._flat["sharded"] = sharded
    return opt


def build_optimizers(model: torch.nn.Module, cfg, parallel_dims=None) -> OptimizersContainer:
    named = _named_trainable(model)
    names = {id(p): n for n, p in named}
    if cfg.enable_mup:
        # muP: hidden matrices get lr / width_mult, everything 2-D decays, vectors do not
        g0 = cfg.optimizer_groups[0]
        opt_class = _import(g0["opt_class"]) if isinstance(g0["opt_class"], str) else g0["opt_class"]
        opt_cfg = dict(g0.get("opt_cfg", {}))
        lr = opt_cfg.pop("lr")
        wd = opt_cfg.pop("weight_decay", opt_cfg.pop("wd", 0.0))
        width_mul = cfg.model_width / cfg.base_model_width
        hidden, other, vecs = [], [], []
        for n, p in named:
            if p.dim() >= 2 and ("attention" in n or "feed_forward" in n):
                hidden.append(p)
            elif p.dim() >= 2:
                other.append(p)
            else:
                vecs.append(p)
        groups = [
            {"params": hidden, "lr": lr / width_mul, "weight_decay": wd},
            {"params": other, "lr": lr, "weight_decay": wd},
            {"params": vecs, "lr": lr, "weight_decay": 0.0},
        ]
        groups = [g for g in groups if g["params"]]
        logger.info(f"muP optimizer groups: hidden={len(hidden)} other={len(other)} vectors={len(vecs)}")
        return OptimizersContainer(model, [_make_optimizer(opt_class, groups, opt_cfg, model)], names)

    buckets: list[list] = [[] for _ in cfg.optimizer_groups]
    for n, p in named:
        for gi, g in enumerate(cfg.optimizer_groups):
            if p.dim() < g.get("min_dim", 0):
                continue
            if any(ex in n for ex in g.get("exclude_names", [])):
                continue
            buckets[gi].append(p)
            logger.debug(f"param {n} -> optimizer group {gi}")
            break
        else:
            raise ValueError(f"Parameter {n} was not assigned to any optimizer group")
    opts = []
    for g, params in zip(cfg.optimizer_groups, buckets):
        if not params:
            continue
        oc = g["opt_class"]
        opt_class = _import(oc) if isinstance(oc, str) else oc
        opts.append(_make_optimizer(opt_class, params, g.get("opt_cfg", {}), model))
        logger.info(f"optimizer {opt_class.__name__}: {len(params)} tensors, {sum(p.numel() for p in params):,} elements")
    return OptimizersContainer(model, opts, names)
