"""Distributed bring-up, metric reductions, peak-FLOPs table, gradient clipping, metric-name helper.

Reference behaviour: maester/utils.py:36-43 (dist_mean/dist_max), :52-76 (set_pg_timeouts),
:107-128 (peak FLOPs table), :131-160 (init_distributed), :245-288 (clip_grad_norm),
:290-312 (clean_param_name).
"""
from __future__ import annotations

import os
import re
from datetime import timedelta
from typing import Iterable

import torch
import torch.distributed as dist

from maester_b200.log_utils import logger

# bf16 dense peak per device name fragment; first match wins (order matters: "A100" before "A10").
_PEAK_BF16 = [
    ("A100", 312e12),
    ("B200", 2250e12),
    ("H100 NVL", 1979e12),
    ("H100 PCIe", 756e12),
    ("H100", 989e12),
    ("A10", 125e12),
    ("MI250X", 191.5e12),
]


def get_peak_flops(device_name: str) -> float:
    """bf16 dense peak used as the MFU denominator; unknown devices fall back to the A100 figure."""
    if "H100" in device_name:
        if "NVL" in device_name:
            return 1979e12
        if "PCIe" in device_name:
            return 756e12
        return 989e12
    for frag, flops in _PEAK_BF16:
        if frag in device_name:
            return flops
    logger.warning("Unknown device %r, defaulting to A100 peak flops.", device_name)
    return 312e12


def device_for_training() -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    return torch.device("cpu")


def resolve_backend(cfg=None) -> str:
    want = getattr(cfg, "comm_backend", "auto") if cfg is not None else "auto"
    if want != "auto":
        return want
    return "nccl" if torch.cuda.is_available() else "gloo"


def init_distributed(cfg) -> None:
    """Create the default process group (NCCL on GPUs, gloo on CPU).

    ``TORCH_NCCL_ASYNC_ERROR_HANDLING=3`` keeps the watchdog from tearing the communicator down so
    that the flight recorder can still dump on a timeout.
    """
    if dist.is_initialized():
        return
    backend = resolve_backend(cfg)
    if backend == "nccl":
        if os.environ.get("TORCH_NCCL_ASYNC_ERROR_HANDLING", "3") != "3":
            logger.warning("TORCH_NCCL_ASYNC_ERROR_HANDLING overridden to 3 (skip cleanup)")
        os.environ["TORCH_NCCL_ASYNC_ERROR_HANDLING"] = "3"
        os.environ["TORCH_NCCL_AVOID_RECORD_STREAMS"] = "1"
    kwargs = {}
    if backend == "nccl" and torch.cuda.is_available():
        kwargs["device_id"] = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group(backend, timeout=timedelta(seconds=cfg.init_timeout_seconds), **kwargs)


def set_pg_timeouts(timeout: timedelta, world_mesh=None) -> None:
    """Barrier, then shorten the timeout of every mesh-dim group and the default group.

    The barrier comes first so a slow rank still finishing its start-up under the long timeout
    cannot be hit by peers that already issue collectives under the short one.
    """
    logger.info("Synchronizing and adjusting timeout for all ProcessGroups to %s", timeout)
    dist.barrier()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    groups = [None]
    if world_mesh is not None:
        try:
            groups += list(world_mesh.get_all_groups())
        except Exception:  # older meshes: one group per dimension
            groups += [world_mesh.get_group(d) for d in range(world_mesh.ndim)]
    for g in groups:
        try:
            dist.distributed_c10d._set_pg_timeout(timeout, g)
        except Exception as e:  # gloo groups of old torch builds lack the setter
            logger.debug("could not set timeout on %s: %s", g, e)


def _scalar_reduce(x: float, op, group) -> torch.Tensor:
    dev = "cuda" if (torch.cuda.is_available() and dist.get_backend(group) == "nccl") else "cpu"
    t = torch.tensor(float(x), device=dev, dtype=torch.float32)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=op, group=group)
    return t


def dist_max(x: float, group=None) -> torch.Tensor:
    return _scalar_reduce(x, dist.ReduceOp.MAX, group)


def dist_mean(x: float, group=None) -> torch.Tensor:
    t = _scalar_reduce(x, dist.ReduceOp.SUM, group)
    n = dist.get_world_size(group) if dist.is_initialized() else 1
    return t / n


def get_num_params(model: torch.nn.Module, exclude_embedding: bool = False) -> int:
    total = sum(p.numel() for p in model.parameters())
    if not exclude_embedding:
        return total
    emb = sum(p.numel() for n, p in model.named_parameters() if "tok_embeddings" in n)
    return total - emb


def get_num_flop_per_token(num_params: int, model_config, seq_len: int) -> int:
    """6·N + 12·L·H·(dim/H)·T; causal sparsity is not discounted."""
    l, h = model_config.n_layers, model_config.n_heads
    return 6 * num_params + 12 * l * h * (model_config.dim // h) * seq_len


@torch.no_grad()
def clip_grad_norm(
    parameters: Iterable[torch.Tensor] | torch.Tensor,
    max_norm: float,
    norm_type: float = 2.0,
    group=None,
    error_if_nonfinite: bool = False,
) -> torch.Tensor:
    """Scale ``.grad`` of the given (possibly sharded) parameters so the global norm is ≤ max_norm.

    ``group`` is the process group the shards are spread over; per-shard norms are combined with an
    all-reduce of the p-th powers.  Returns the total norm before clipping.
    """
    if isinstance(parameters, torch.Tensor):
        parameters = [parameters]
    grads = [p.grad for p in parameters if p.grad is not None]
    if not grads:
        return torch.tensor(0.0)
    norm_type = float(norm_type)
    if norm_type == float("inf"):
        local = torch.stack([g.detach().abs().max().float() for g in grads]).max()
        if group is not None or (dist.is_initialized() and dist.get_world_size() > 1 and group is not False):
            dist.all_reduce(local, op=dist.ReduceOp.MAX, group=group or None)
        total = local
    else:
        norms = torch._foreach_norm(grads, norm_type)
        local = torch.stack([n.float() for n in norms]).pow(norm_type).sum()
        if group is not False and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(local, op=dist.ReduceOp.SUM, group=group)
        total = local.pow(1.0 / norm_type)
    if error_if_nonfinite and not torch.isfinite(total):
        raise RuntimeError(f"The total norm of order {norm_type} for gradients is non-finite")
    coef = torch.clamp(max_norm / (total + 1e-6), max=1.0)
    torch._foreach_mul_(grads, coef.to(grads[0].device))
    return total


def clean_param_name(name: str) -> str:
    """Map a parameter FQN to a grouped metric name such as ``layer3/ffn/proj/weight``.  The grouping words are the
    reference's (maester/utils.py:290-311: "attention", then "mlp" / "ffn", else "other"), so that the metric names of
    an existing dashboard stay the same: Llama's ``feed_forward`` and Gemma's ``self_attn`` land in "other" there too."""
    parts = re.split(r"[._]", name)
    tail = "/".join(parts[-2:])
    if "layers" in parts:
        idx = parts[parts.index("layers") + 1]
        if "attention" in name:
            kind = "attention"
        elif any(k in name for k in ("mlp", "ffn")):
            kind = "ffn"
        else:
            kind = "other"
        return f"layer{idx}/{kind}/{tail}"
    for key in ("embedding", "norm", "output"):
        if key in name:
            return f"{key}/{tail}"
    return f"other/{tail}"


def has_cuda_capability(major: int, minor: int) -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability() >= (major, minor)
