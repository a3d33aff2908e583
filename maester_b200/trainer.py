"""Model/optimizer construction and the training step, shared by ``train.py`` and ``bench.py``.

``Trainer(cfg)`` performs the start-up sequence of the reference trainer (train.py:96-251): parallel
dims and mesh, meta-device model build with config overrides (norm type, vocab size, max_seq_len,
muP width), parameter/FLOP count, parallelize, weight init, optimizers and LR scheduler.
``train_step(batches)`` runs one optimizer step over ``gradient_accumulation_steps`` micro-batches
with the reference's loop semantics (train.py:314-390): per-micro-step reseed, loss / accum,
gradient sync only on the last micro-batch unless ``gradient_accumulation_sync_each_step``,
optimizer step then scheduler step.
"""
from __future__ import annotations

import copy
import os
from typing import Any, Iterable

import torch
import torch.distributed as dist

from maester_b200.config import Config
from maester_b200.log_utils import logger
from maester_b200.lr_scheduling import get_lr_scheduler
from maester_b200.models import (
    model_name_to_cls,
    model_name_to_optimizers_builder,
    model_name_to_parallelize,
    models_config,
)
from maester_b200 import ops
from maester_b200.ops import reference as ref
from maester_b200.parallel import ParallelDims, materialize
from maester_b200.utils import clip_grad_norm, device_for_training, get_peak_flops


def build_model_args(cfg: Config, vocab_size: int | None = None):
    """Flavor args with the training-time overrides applied (train.py:136-155)."""
    args = copy.deepcopy(models_config[cfg.model_name][cfg.flavor])
    if hasattr(args, "norm_type"):
        args.norm_type = cfg.norm_type
    if getattr(args, "vocab_size", 0) <= 0:
        if vocab_size is None:
            raise ValueError("flavor has no vocab_size: pass a tokenizer or set synthetic_vocab_size")
        args.vocab_size = vocab_size
    args.max_seq_len = cfg.seq_len
    if cfg.moe_aux_loss_coeff > 0 and hasattr(args, "moe_args"):
        args.moe_args.aux_loss_coeff = cfg.moe_aux_loss_coeff
    if cfg.enable_mup:
        args.enable_mup = True
        args.mup_input_alpha = cfg.mup_input_alpha
        args.mup_output_alpha = cfg.mup_output_alpha
        args.mup_width_mul = cfg.model_width / cfg.base_model_width
        args.dim = cfg.model_width
        head_dim = 128
        args.n_heads = cfg.model_width // head_dim
        if getattr(args, "n_kv_heads", None):
            args.n_kv_heads = min(args.n_kv_heads, args.n_heads)
    return args


class Trainer:
    def __init__(self, cfg: Config, vocab_size: int | None = None):
        self.cfg = cfg
        self.device = device_for_training()
        world_size = int(os.environ.get("WORLD_SIZE", "1")) if dist.is_initialized() else 1
        self.parallel_dims = ParallelDims(
            dp_shard=cfg.data_parallel_shard_degree,
            dp_replicate=cfg.data_parallel_replicate_degree,
            tp=cfg.tensor_parallel_degree,
            ep=cfg.expert_parallel_degree,
            cp=cfg.context_parallel_degree,
            world_size=world_size,
            enable_loss_parallel=cfg.enable_loss_parallel,
        )
        pd = self.parallel_dims
        self.world_mesh = pd.world_mesh if world_size > 1 else None
        if pd.dp_enabled and self.world_mesh is not None:
            dp_mesh = self.world_mesh["dp"]
            self.dp_group, self.dp_degree, self.dp_rank = dp_mesh.get_group(), dp_mesh.size(), dp_mesh.get_local_rank()
        else:
            self.dp_group, self.dp_degree, self.dp_rank = None, 1, 0

        self.model_args = build_model_args(cfg, vocab_size or (cfg.synthetic_vocab_size or None))
        with torch.device("meta"):
            self.model = model_name_to_cls[cfg.model_name].from_model_args(self.model_args)
        self.nparams, self.flops_per_token = self.model_args.get_nparams_and_flops(self.model, cfg.seq_len)
        logger.info(f"Model {cfg.model_name} {cfg.flavor} size: {self.nparams:,} total parameters")
        self.peak_flops = get_peak_flops(torch.cuda.get_device_name(self.device)) if self.device.type == "cuda" else 312e12
        model_name_to_parallelize[cfg.model_name](self.model, self.world_mesh, pd, cfg)
        self.cp = None
        if pd.cp_enabled:
            from maester_b200.parallel.context_parallel import apply_cp
            self.cp = apply_cp(self.model, pd, mode=cfg.context_parallel_mode)
        materialize(self.model)
        self.sharded = getattr(self.model, "_sharded", None)
        self.optimizers = model_name_to_optimizers_builder[cfg.model_name](self.model, cfg, pd)
        self.scheduler = get_lr_scheduler(self.optimizers, cfg)
        self.model.train()
        self.grad_accum = max(1, cfg.gradient_accumulation_steps)
        self.global_micro_step = 0
        self.step = 0
        self.heartbeat = None
        if cfg.step_heartbeat and dist.is_initialized() and world_size > 1:
            from maester_b200.heartbeat import StepHeartbeat
            self.heartbeat = StepHeartbeat()
        self.activation_stats: dict[str, list] = {}
        if cfg.enable_mup and cfg.mup_log_coord_check:
            self._register_coord_check_hooks()

    # ------------------------------------------------------------------ muP coordinate check
    def _register_coord_check_hooks(self) -> None:
        """Forward hooks that record mean |activation| of the embedding, attention / feed-forward projections and the
        output head on log steps (reference train.py:209-235); ``pop_activation_stats`` turns them into
        ``act/<key>_abs_mean`` metrics."""
        def hook(key):
            def fn(mod, inp, out):
                if (self.step + 1) % self.cfg.log_freq == 0 or self.step == 0:
                    self.activation_stats.setdefault(key, []).append(out.detach().abs().float().mean())
            return fn

        n = 0
        for name, mod in self.model.named_modules():
            key = None
            if name == "tok_embeddings":
                key = "tok_embed"
            elif "attention." in name and name.endswith((".wq", ".wk", ".wv", ".wo")):
                key = "attn"
            elif "feed_forward." in name and name.endswith((".w1", ".w2", ".w3")):
                key = "ffn"
            elif name == "output":
                key = "output"
            if key is not None:
                mod.register_forward_hook(hook(key))
                n += 1
        logger.info(f"Activation hooks registered for {n} modules")

    def pop_activation_stats(self) -> dict[str, float]:
        out = {f"act/{k}_abs_mean": float(torch.stack(v).mean().item()) for k, v in self.activation_stats.items() if v}
        self.activation_stats = {}
        return out

    # ------------------------------------------------------------------ health between steps
    def check_device_status(self, sync: bool = False) -> None:
        """Raise if a kernel gave up on a bounded wait since the last check (its output is then garbage).  Call where
        the host has just synchronised (after reading losses) and, with ``sync=True``, before saving a checkpoint."""
        if self.device.type == "cuda":
            from maester_b200.ops import cuda as C
            C.check_status(sync=sync)

    def pop_dropped_rows(self) -> int | None:
        """Rows the peer-memory expert dispatcher dropped over capacity since the last call (None without it)."""
        disp = getattr(getattr(self.model, "ep", None), "peer_dispatcher", None)
        if disp is None:
            return None
        n = int(disp.dropped())
        disp.reset_dropped()
        disp.adapt_capacity()   # collective over the expert-parallel group: every rank reaches this on log steps
        if n:
            logger.warning(f"expert-parallel peer dispatch dropped {n} rows over capacity "
                           f"(ep_capacity_factor={self.cfg.ep_capacity_factor}); the all-to-all dispatcher never drops")
        return n

    # ------------------------------------------------------------------ one optimizer step
    def to_device(self, batch: dict[str, Any]) -> dict[str, Any]:
        out = {}
        for k in ("input_ids", "labels", "position_ids", "document_ids"):
            v = batch.get(k)
            if v is not None:
                out[k] = v.to(self.device, non_blocking=True)
        return out

    def forward_backward(self, batch: dict[str, Any], sync: bool = True) -> torch.Tensor:
        cfg = self.cfg
        if self.sharded is not None and self.grad_accum > 1:
            self.sharded.set_requires_gradient_sync(sync)
        if self.cp is not None and self.cp.mode == "ring":
            d = batch.get("document_ids")  # still on the host here: the check costs no device synchronisation
            if d is not None and not d.is_cuda and bool((d != d[:, :1]).any()):
                raise NotImplementedError("context_parallel_mode='ring' attends causally over the whole sequence; "
                                          "packed documents need context_parallel_mode='alltoall'")
        b = self.to_device(batch)
        if self.cp is not None:
            from maester_b200.parallel.context_parallel import shard_batch_for_cp
            b = shard_batch_for_cp(b, self.cp)
        if cfg.enable_cut_cross_entropy:
            # the loss below reaches backward() with exactly this output gradient: the loss layer may produce its
            # gradients chunk by chunk during forward and keep no logits
            with ops.loss_backward_scale(1.0 / self.grad_accum):
                loss = self.model(b["input_ids"], b["labels"], position_ids=b.get("position_ids"),
                                  document_ids=b.get("document_ids"))
        else:
            pred = self.model(b["input_ids"], position_ids=b.get("position_ids"), document_ids=b.get("document_ids"))
            loss = ref.cross_entropy(pred, b["labels"])
            del pred
        (loss / self.grad_accum).backward()
        if self.sharded is not None:
            self.sharded.finish_backward()
            if self.grad_accum > 1:
                self.sharded.set_requires_gradient_sync(True)
        return loss.detach()

    def train_step(self, batches: Iterable[dict[str, Any]] | dict[str, Any]) -> torch.Tensor:
        """One optimizer step; ``batches`` is one micro-batch dict or ``gradient_accumulation_steps`` of them.
        Returns the mean micro-batch loss as a 0-d tensor on the training device."""
        if isinstance(batches, dict):
            batches = [batches]
        self.optimizers.zero_grad(set_to_none=True)
        skip_sync = self.grad_accum > 1 and not self.cfg.gradient_accumulation_sync_each_step
        losses = []
        batches = list(batches)
        clip = bool(self.cfg.clip_gradients and self.cfg.max_grad_norm and self.cfg.max_grad_norm > 0)
        if self.heartbeat is not None:  # nobody launches kernels towards a peer that is gone
            self.heartbeat.beat(self.step + 1)
            self.heartbeat.check(self.step + 1, timeout_s=self.cfg.heartbeat_timeout_seconds)
        for i, batch in enumerate(batches):
            self.global_micro_step += 1
            torch.manual_seed(self.global_micro_step + self.dp_rank)
            sync = (i == len(batches) - 1) if skip_sync else True
            if i == len(batches) - 1 and not clip and hasattr(self.optimizers, "announce_step"):
                self.optimizers.announce_step()  # units may be updated as soon as their gradients are complete
            losses.append(self.forward_backward(batch, sync))
        if clip:
            if self.sharded is not None:
                self.last_grad_norm = self.sharded.clip_grad_norm(self.cfg.max_grad_norm)
            else:
                params = [p for g in self.optimizers.param_groups for p in g["params"]]
                self.last_grad_norm = clip_grad_norm(params, self.cfg.max_grad_norm, group=False)
        self.optimizers.step()
        self.scheduler.step()
        self.step += 1
        return torch.stack(losses).mean() if len(losses) > 1 else losses[0]

    # ------------------------------------------------------------------ metrics helpers
    def mfu(self, tokens_per_second_per_gpu: float) -> float:
        return 100.0 * self.flops_per_token * tokens_per_second_per_gpu / self.peak_flops
