"""Metrics: GPU memory monitor, TensorBoard / W&B loggers, per-parameter weight-RMS monitor and
logit statistics hooks (reference: maester/metrics.py:48-338).

The weight monitor computes every parameter's RMS with one batched ``_foreach_norm`` and a single
device-to-host transfer per logging step instead of one ``.item()`` per parameter.
"""
from __future__ import annotations

import math
import os
from collections import defaultdict, namedtuple
from datetime import datetime
from typing import Any

import torch
import torch.distributed as dist

from maester_b200.log_utils import logger
from maester_b200.utils import clean_param_name

GPUMemStats = namedtuple(
    "GPUMemStats",
    ["max_active_gib", "max_active_pct", "max_reserved_gib", "max_reserved_pct", "num_alloc_retries", "num_ooms"],
)
_GIB = 1024 ** 3


class GPUMemoryMonitor:
    def __init__(self, device: str = "cuda"):
        self.enabled = torch.cuda.is_available()
        if not self.enabled:
            self.device_name, self.device_index, self.device_capacity = "cpu", 0, 1
            self.device_capacity_gib = 0.0
            return
        self.device = torch.device(device)
        self.device_name = torch.cuda.get_device_name(self.device)
        self.device_index = torch.cuda.current_device()
        self.device_capacity = torch.cuda.get_device_properties(self.device).total_memory
        self.device_capacity_gib = self.device_capacity / _GIB
        torch.cuda.reset_peak_memory_stats()
        torch.cuda.empty_cache()

    def get_peak_stats(self) -> GPUMemStats:
        if not self.enabled:
            return GPUMemStats(0.0, 0.0, 0.0, 0.0, 0, 0)
        info = torch.cuda.memory_stats(self.device)
        active, reserved = info["active_bytes.all.peak"], info["reserved_bytes.all.peak"]
        retries, ooms = info["num_alloc_retries"], info["num_ooms"]
        if retries > 0:
            logger.warning(f"{retries} CUDA memory allocation retries.")
        if ooms > 0:
            logger.warning(f"{ooms} CUDA OOM errors thrown.")
        cap = self.device_capacity
        return GPUMemStats(active / _GIB, 100 * active / cap, reserved / _GIB, 100 * reserved / cap, retries, ooms)

    def reset_peak_stats(self) -> None:
        if self.enabled:
            torch.cuda.reset_peak_memory_stats()
            torch.cuda.reset_accumulated_memory_stats()


def build_gpu_memory_monitor() -> GPUMemoryMonitor:
    mon = GPUMemoryMonitor("cuda")
    logger.info(f"GPU capacity: {mon.device_name} ({mon.device_index}) with {mon.device_capacity_gib:.2f}GiB memory")
    return mon


class NullMetricLogger:
    def log(self, metrics: dict[str, Any], step: int) -> None:
        pass

    def close(self) -> None:
        pass


class TBMetricLogger:
    def __init__(self, log_dir: str, tag: str | None):
        from torch.utils.tensorboard import SummaryWriter

        self.tag = tag
        self.writer = SummaryWriter(log_dir, max_queue=1000)

    def log(self, metrics: dict[str, Any], step: int) -> None:
        for k, v in metrics.items():
            self.writer.add_scalar(k if self.tag is None else f"{self.tag}/{k}", v, step)

    def close(self) -> None:
        self.writer.close()


class WandbMetricLogger:
    def __init__(self, cfg):
        import wandb

        self.wandb = wandb
        wandb.init(project=cfg.wandb_project, entity=cfg.wandb_entity, name=cfg.job_name,
                   config=cfg.model_dump(mode="json"), resume="allow")

    def log(self, metrics: dict[str, Any], step: int) -> None:
        self.wandb.log(metrics, step=step)

    def close(self) -> None:
        self.wandb.finish()


def build_metric_logger(cfg, tag: str | None = None):
    """W&B xor TensorBoard xor nothing; rank filtering follows ``log_rank0_only``."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    if cfg.enable_wandb and (rank == 0 or not cfg.log_rank0_only):
        return WandbMetricLogger(cfg)
    if cfg.enable_tensorboard:
        stamp = datetime.now().strftime("%Y%m%d-%H%M")
        log_dir = os.path.join(cfg.dump_dir, cfg.job_name, cfg.save_tb_folder, stamp)
        if not cfg.log_rank0_only:
            log_dir = os.path.join(log_dir, f"rank_{rank}")
        elif rank != 0:
            return NullMetricLogger()
        logger.info(f"Metrics logging active. Tensorboard logs will be saved at {log_dir}")
        return TBMetricLogger(log_dir, tag)
    return NullMetricLogger()


class WeightScaleMonitor:
    """RMS of every (sharded) parameter, grouped as ``layerN/kind/name/weight_rms``, every log_freq steps."""

    def __init__(self, model: torch.nn.Module, log_freq: int = 100, ignored_substrings: set[str] | None = None):
        self.model, self.log_freq, self.step = model, log_freq, 0
        self.ignored = ignored_substrings or set()
        self.weight_stats: dict[str, list[float]] = defaultdict(list)

    def _named(self):
        sharded = getattr(self.model, "_sharded", None)
        src = sharded.named_master_parameters() if sharded is not None else self.model.named_parameters()
        return [(n, p) for n, p in src if p.requires_grad and not any(s in n for s in self.ignored)]

    def step_monitor(self) -> dict[str, float] | None:
        self.step += 1
        if self.step % self.log_freq != 0:
            return None
        sharded = getattr(self.model, "_sharded", None)
        if sharded is not None:
            # one multi-tensor launch over the flat master shards, then the all-reduces of one small vector
            slots = sharded._slot_list()
            keep = [i for i, sl in enumerate(slots) if sl.master.requires_grad and not any(s in sl.fqn for s in self.ignored)]
            if not keep:
                return {}
            sq = sharded.global_sqnorms("master")
            # expert tensors: this rank's experts only (the norm was summed over the ranks holding the same experts)
            full = torch.tensor([max(1, math.prod(slots[i].global_shape) // (sharded.ep_size if slots[i].dom == 1 else 1))
                                 for i in keep], device=sq.device, dtype=torch.float32)
            rms = (sq[torch.tensor(keep, device=sq.device)] / full).sqrt().tolist()
            stats = {}
            for i, r in zip(keep, rms):
                g = clean_param_name(slots[i].fqn)
                self.weight_stats[g].append(r)
                stats[f"{g}/weight_rms"] = r
            return stats
        named = [(n, p) for n, p in self._named() if p.numel() > 0]
        if not named:
            return {}
        sq = torch.stack([x.float() ** 2 for x in torch._foreach_norm([p.data for _, p in named])])
        numels = torch.tensor([p.numel() for _, p in named], device=sq.device, dtype=torch.float32)
        sharded = getattr(self.model, "_sharded", None)
        if sharded is not None and sharded.world > 1:
            full = torch.tensor([math.prod(sharded.slot_of(p).shape) for _, p in named], device=sq.device,
                                dtype=torch.float32)
            dist.all_reduce(sq, group=sharded.group)
            numels = full
        rms = (sq / numels).sqrt().tolist()  # one transfer for all parameters
        stats = {}
        for (n, _), r in zip(named, rms):
            g = clean_param_name(n)
            self.weight_stats[g].append(r)
            stats[f"{g}/weight_rms"] = r
        return stats


def register_logits_monitoring(model: torch.nn.Module, train_state, log_freq: int, monitor_attention: bool = False):
    """Forward hook on the output projection collecting logit statistics every ``log_freq`` steps.

    Returns ``(get_metrics, cleanup, reinit_storage)`` as the reference does (metrics.py:245-338).
    Models whose loss path never materialises logits only report when called without labels.
    """
    storage: dict[str, torch.Tensor] = {}
    handles = []

    def out_hook(mod, inp, out):
        if train_state.step % log_freq == 0 and torch.is_tensor(out) and out.dim() == 3:
            with torch.no_grad():
                o = out.float()
                storage["logits/mean"] = o.mean()
                storage["logits/std"] = o.std()
                storage["logits/max"] = o.max()
                storage["logits/min"] = o.min()

    target = getattr(model, "output", None)
    if isinstance(target, torch.nn.Module):
        handles.append(target.register_forward_hook(out_hook))

    def get_metrics() -> dict[str, float]:
        return {k: v.item() for k, v in storage.items()}

    def cleanup() -> None:
        for h in handles:
            h.remove()

    def reinit_storage() -> None:
        storage.clear()

    return get_metrics, cleanup, reinit_storage
