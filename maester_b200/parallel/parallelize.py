"""Apply the parallel plan to a model: activation checkpointing, then flat-buffer sharding.

Reference entry points: ``parallelize_llama`` / ``parallelize_gemma`` / ``parallelize_deepseek``
(maester/parallelisms/parallelize_*.py), called as ``parallelize(model, world_mesh, parallel_dims,
cfg)`` before the weights exist.  The order there is TP -> AC -> compile -> FSDP; here there is no
compile step, and sharding also materialises the parameters (the model may arrive on the meta
device).
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from maester_b200.config import TORCH_DTYPE_MAP
from maester_b200.log_utils import logger
from maester_b200.parallel.fsdp import ShardedModel
from maester_b200.utils import device_for_training


def transformer_blocks(model: nn.Module) -> list[tuple[str, nn.Module]]:
    """The per-layer units of a model: ``model.layers`` (Gemma) or ``layers`` (Llama, DeepSeek, GLM4)."""
    inner = getattr(model, "language_model", model)
    holder = inner.model if hasattr(inner, "model") and hasattr(inner.model, "layers") else inner
    layers = holder.layers
    items = layers.items() if isinstance(layers, nn.ModuleDict) else enumerate(layers)
    return [(f"layer{i}", m) for i, m in items]


class CheckpointWrapper(nn.Module):
    """Full activation checkpointing of one block: keep only its inputs, recompute in backward.
    The wrapped module keeps its attribute name, so parameter FQNs do not change."""

    def __init__(self, mod: nn.Module):
        super().__init__()
        self._checkpoint_wrapped_module = mod

    def forward(self, *args, **kwargs):
        if not torch.is_grad_enabled():
            return self._checkpoint_wrapped_module(*args, **kwargs)
        return checkpoint(self._checkpoint_wrapped_module, *args, use_reentrant=False, preserve_rng_state=False,
                          **kwargs)


def apply_ac(model: nn.Module, cfg) -> None:
    """ac_mode: none | full | selective; selective_ac_option: "op" or an integer N (every N-th block).

    "op" is the per-op policy of the reference (save GEMM and attention outputs, recompute the rest,
    parallelize_llama.py:183-250).  With hand-written fused kernels it becomes an explicit plan: the attention
    modules rebuild the normalised, rotated q / k from the packed projection in backward (one QK-norm + RoPE pass,
    (H + KV) * head_dim values per token and block not kept); GEMM, attention and norm outputs are kept, because a
    norm's output is the GEMM operand that the weight gradient needs anyway.  The blocks' ``selective_recompute``
    flag additionally lets a gated MLP rebuild its activation (``glu_mlp(save_act=False)``), which costs a full
    pass over [tokens, ffn] per block and is left off.
    """
    mode = cfg.ac_mode
    if mode == "none":
        return
    blocks = transformer_blocks(model)
    if mode == "selective" and str(cfg.selective_ac_option) == "op":
        for _, b in blocks:
            b.selective_recompute = True
            for m in b.modules():
                if hasattr(m, "cp_capable"):
                    m.recompute_qk = True
        logger.info("Applied selective (per-op) activation recomputation to %d blocks", len(blocks))
        return
    every = 1
    if mode == "selective":
        every = int(cfg.selective_ac_option)
        assert every >= 1
    elif mode != "full":
        raise ValueError(f"Invalid ac_mode {mode}")
    inner = getattr(model, "language_model", model)
    holder = inner.model if hasattr(inner, "model") and hasattr(inner.model, "layers") else inner
    count = 0
    for idx, (name, b) in enumerate(blocks):
        if (idx + 1) % every == 0 or mode == "full":
            key = name[len("layer"):]
            w = _Checkpointed(b)
            if isinstance(holder.layers, nn.ModuleDict):
                holder.layers[key] = w
            else:
                holder.layers[int(key)] = w
            count += 1
    logger.info("Applied %s activation checkpointing to %d of %d blocks", mode, count, len(blocks))


class _Checkpointed(nn.Module):
    """Same as CheckpointWrapper but transparent for FQNs: parameters are reached through the inner
    module registered under the reserved name ``_orig_mod``-free path by overriding ``named_*``."""

    def __init__(self, mod: nn.Module):
        super().__init__()
        object.__setattr__(self, "inner", mod)
        # register children/params of the inner module as our own so FQNs are unchanged
        self._modules = mod._modules
        self._parameters = mod._parameters
        self._buffers = mod._buffers

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(object.__getattribute__(self, "inner"), name)

    def forward(self, *args, **kwargs):
        inner = object.__getattribute__(self, "inner")
        if not torch.is_grad_enabled():
            return inner(*args, **kwargs)
        return checkpoint(inner, *args, use_reentrant=False, preserve_rng_state=False, **kwargs)


def parallelize(model: nn.Module, world_mesh, parallel_dims, cfg) -> nn.Module:
    """Checkpointing plan + sharded flat buffers.  Stores the runtime as ``model._sharded`` and adds
    ``model.set_requires_gradient_sync`` (the hook the training loop uses during accumulation)."""
    from maester_b200.models.moe.moe import MoE
    has_moe = any(isinstance(m, MoE) for m in model.modules())
    ep = None
    if parallel_dims.ep_enabled:
        from maester_b200.parallel.expert_parallel import apply_ep
        assert has_moe, "expert_parallel_degree > 1 needs a mixture-of-experts model"
        ep = apply_ep(model, parallel_dims, use_peer_memory=bool(cfg.ep_peer_dispatch) and device_for_training().type == "cuda",
                      capacity_factor=cfg.ep_capacity_factor)
    if parallel_dims.tp_enabled:
        if has_moe:  # as in the reference, only the MoE parts of DeepSeek / GLM-4.5 have a TP plan
            from maester_b200.parallel.expert_parallel import apply_expert_tp
            apply_expert_tp(model, parallel_dims)
        else:
            from maester_b200.parallel.tensor_parallel import apply_tp
            apply_tp(model, parallel_dims, cfg)
    apply_ac(model, cfg)
    device = device_for_training()
    param_dtype = TORCH_DTYPE_MAP[cfg.mixed_precision_param]
    reduce_dtype = TORCH_DTYPE_MAP[cfg.mixed_precision_reduce]
    if device.type == "cpu":
        param_dtype = torch.float32 if param_dtype == torch.bfloat16 and not getattr(cfg, "cpu_bf16", False) else param_dtype
    shard_group = parallel_dims.mesh_group("dp_shard_cp") if parallel_dims.fsdp_enabled else None
    rep_group = parallel_dims.mesh_group("dp_replicate") if parallel_dims.dp_replicate_enabled else None
    reshard = _reshard_policy(cfg, model, device, parallel_dims)
    sharded = ShardedModel(
        model, transformer_blocks(model), device=device, param_dtype=param_dtype, reduce_dtype=reduce_dtype,
        reshard=reshard, cpu_offload=bool(cfg.enable_cpu_offload),
        shard_group=shard_group, replicate_group=rep_group,
        gradient_divide_factor=float(parallel_dims.fsdp_gradient_divide_factor),
        tp_group=parallel_dims.mesh_group("tp") if parallel_dims.tp_enabled else None,
        # the fused reduce-scatter + AdamW + all-gather kernel only exists for AdamW groups
        fused_comm=bool(cfg.fused_collectives) and device.type == "cuda" and all(
            str(g.get("opt_class", "")).endswith("AdamW") for g in cfg.optimizer_groups),
        expert_group=parallel_dims.mesh_group("dp_shard_mod_ep") if ep is not None else None,
        ep_size=ep.size if ep is not None else 1, ep_rank=ep.rank if ep is not None else 0,
    )
    sharded.device_mesh = world_mesh["dp_shard_cp"] if (shard_group is not None and world_mesh is not None) else None
    sharded.ckpt_meshes = _checkpoint_meshes(world_mesh, parallel_dims, ep is not None)
    sharded.ep_group = ep.group if ep is not None else None
    object.__setattr__(model, "_sharded", sharded)
    model.set_requires_gradient_sync = sharded.set_requires_gradient_sync
    # buffers that are still on the meta device (RoPE tables) are rebuilt by init_weights()
    return model


def _reshard_policy(cfg, model: nn.Module, device, parallel_dims) -> bool:
    """``fsdp_reshard_after_forward``: "always" frees every block's gathered parameters after use (and keeps gradients
    per block), "never" keeps the whole bf16 model and a whole fp32 gradient buffer on every GPU (fastest: one fused
    reduce-scatter + update + all-gather kernel per block), "default" picks "never" when that resident copy
    (6 bytes per parameter) takes less than 45 % of the device memory and "always" otherwise.  CPU offload of the
    optimizer state implies resharding."""
    mode = cfg.fsdp_reshard_after_forward
    if not parallel_dims.fsdp_enabled:
        return False
    if cfg.enable_cpu_offload or mode == "always":
        return True
    if mode == "never":
        return False
    if device.type != "cuda":
        return False
    nparams = sum(p.numel() for p in model.parameters())
    total = torch.cuda.get_device_properties(device).total_memory
    return 6 * nparams > 0.45 * total


def _checkpoint_meshes(world_mesh, parallel_dims, has_ep: bool) -> dict:
    """Sub-meshes over which checkpointed tensors are split (see ``checkpoint._as_dtensor``):
    ``dense``: ``(dp_shard_cp,)``; ``dense_tp``: ``(dp_shard_cp, tp)`` or ``(tp,)``; ``expert``:
    ``(dp_shard_mod_ep, dp_shard_in_ep)`` (the layout FSDP2 on top of expert parallelism produces);
    ``expert_tp``: the same with ``tp`` appended."""
    out: dict = {}
    if world_mesh is None:
        return out
    names = set(world_mesh.mesh_dim_names or ())
    if parallel_dims.fsdp_enabled:
        out["dense"] = world_mesh["dp_shard_cp"]
    if parallel_dims.tp_enabled:
        out["dense_tp"] = world_mesh["dp_shard_cp", "tp"] if parallel_dims.fsdp_enabled else world_mesh["tp"]
    if has_ep:
        in_ep = ("dp_shard_in_ep",) if "dp_shard_in_ep" in names else ()
        if in_ep:
            out["expert"] = world_mesh[("dp_shard_mod_ep",) + in_ep]
            if parallel_dims.tp_enabled:
                out["expert_tp"] = world_mesh[("dp_shard_mod_ep",) + in_ep + ("tp",)]
    return out


def materialize(model: nn.Module) -> None:
    """``to_empty`` + ``init_weights`` of the reference start-up (train.py:189-190) for a sharded
    model: parameters already live in the flat buffers, so only initialise and load the shards."""
    model.init_weights()
    sharded = getattr(model, "_sharded", None)
    if sharded is not None:
        sharded.init_master_from_full()


parallelize_llama = parallelize
parallelize_gemma = parallelize
parallelize_deepseek = parallelize
