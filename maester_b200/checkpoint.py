"""Checkpoint manager on top of ``torch.distributed.checkpoint`` (DCP).

Same contract as the reference (maester/checkpoint.py:95-255): states ``train_state``, ``model``,
``optimizer``, ``lr_scheduler`` saved under ``<dump_dir>/<job_name>/<checkpoint_folder>/step-<N>``
every ``checkpoint_interval`` steps; the forced save at the last step keeps only
``{"model": {fqn: tensor.to(export_dtype)}}`` when ``model_weights_only``; ``load`` prefers
``forced_load_path`` (model only), else the highest ``step-*`` folder, and loads only the model for
step 0 (seed checkpoint) or ``model_only=True``.

Sharded tensors are published as ``DTensor`` with ``Shard(0)`` placement built over this rank's rows
of the flat fp32 master / optimizer-state buffers, so DCP writes the same per-rank shard files as for
an FSDP2 model and can reshard on load.  Keys are the model's parameter FQNs.
"""
from __future__ import annotations

import enum
import os
import re
import time
from typing import Any

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
import torch.nn as nn
from torch.distributed.checkpoint.stateful import Stateful

from maester_b200.config import TORCH_DTYPE_MAP
from maester_b200.log_utils import logger


def _check_device_status() -> None:
    """A kernel whose bounded wait ran out leaves garbage behind: refuse to write it to disk."""
    if torch.cuda.is_available():
        from maester_b200.ops import cuda as C
        C.check_status(sync=True)


class IntervalType(enum.Enum):
    SECONDS = enum.auto()
    STEPS = enum.auto()


def _as_dtensor(local: torch.Tensor, slot, sharded) -> torch.Tensor:
    """Present this rank's piece of a parameter (or of its optimizer state) as a DTensor over the mesh dimensions
    that split it, so that DCP writes whole tensors and can reshard on load.  A plain tensor is returned only when
    nothing splits the parameter (one process, or a data-parallel group of one without tensor parallelism).

    Splits, outermost first: experts over ``dp_shard_in_ep`` (expert parallelism) and each rank's experts over
    ``dp_shard_mod_ep`` (the ranks holding the same experts): a strided shard plus a shard on dim 0; dense parameters
    over ``dp_shard_cp`` on dim 0; on top of either, the tensor-parallel slice along ``slot.tp_dim`` over ``tp`` (a
    slice of dim 0 makes the data-parallel shard of dim 0 strided).  Parameters that are replicated over ``tp`` are
    published over the data-parallel mesh only; DCP keeps one copy of identical pieces."""
    from torch.distributed.tensor import DTensor, Shard
    from torch.distributed.tensor.placement_types import _StridedShard

    if sharded is None:
        return local
    if getattr(slot, "tp_segments", None) is not None:
        return _as_row_pieces(local, slot, sharded)
    meshes = getattr(sharded, "ckpt_meshes", None) or {}
    tp = slot.tp_dim >= 0
    if slot.dom == 1:
        mesh = meshes.get("expert_tp" if tp else "expert")
        if mesh is None:
            raise NotImplementedError(f"no checkpoint mesh for the expert parameter {slot.fqn}")
        placements = [_StridedShard(0, split_factor=mesh.size(1)), Shard(0)]
        if tp:
            assert slot.tp_dim > 0, "expert tensors are tensor-parallel along their hidden dimension"
            placements.append(Shard(slot.tp_dim))
    elif tp:
        mesh = meshes.get("dense_tp")
        if mesh is None:
            raise NotImplementedError(f"no checkpoint mesh for the tensor-parallel parameter {slot.fqn}")
        if mesh.ndim == 1:
            placements = [Shard(slot.tp_dim)]
        elif slot.tp_dim == 0:
            placements = [_StridedShard(0, split_factor=mesh.size(1)), Shard(0)]
        else:
            placements = [Shard(0), Shard(slot.tp_dim)]
    else:
        mesh = meshes.get("dense")
        if mesh is None or sharded.world == 1:
            return local
        placements = [Shard(0)]
    shape = slot.global_shape
    stride = torch.empty(shape, device="meta").stride()
    return DTensor.from_local(local, mesh, placements, run_check=False, shape=shape, stride=stride)


def row_pieces(slot, own_lo: int, own_hi: int) -> list[tuple[int, int, int]]:
    """For a parameter whose tensor-parallel slice consists of several row ranges of the whole tensor
    (``slot.tp_segments``): the pieces of this rank's rows ``[own_lo, own_hi)`` of the LOCAL slice as
    ``(first local row relative to own_lo, first global row, rows)``."""
    out, start = [], 0
    for g0, n in slot.tp_segments:
        lo, hi = max(own_lo, start), min(own_hi, start + n)
        if hi > lo:
            out.append((lo - own_lo, g0 + (lo - start), hi - lo))
        start += n
    return out


def _as_row_pieces(local: torch.Tensor, slot, sharded) -> torch.Tensor:
    """This rank's rows of a head-group-split projection as a checkpointable object with SEVERAL chunks, each at its
    place in the whole tensor (the reference's row order), so that the checkpoint holds the tensor exactly as an
    unsharded model has it and any other layout can load it.  DTensor cannot describe this (one contiguous range per
    rank), so the tensor carries DCP's checkpointable hooks itself: one write / read item per piece."""
    from torch.distributed.checkpoint.metadata import ChunkStorageMetadata, MetadataIndex, TensorProperties
    from torch.distributed.checkpoint.planner import TensorWriteData, WriteItem, WriteItemType

    lo, hi = sharded._own_rows(slot)
    cols = tuple(slot.shape[1:])
    rows2d = local.reshape(-1, *cols)[: hi - lo] if hi > lo else local.reshape(-1, *cols)[:0]
    pieces = row_pieces(slot, lo, hi)
    size = slot.global_shape
    zeros = (0,) * len(cols)
    t = rows2d.view(rows2d.shape)          # a fresh tensor object over the same memory to carry the hooks
    chunks = [ChunkStorageMetadata(offsets=torch.Size((g0, *zeros)), sizes=torch.Size((n, *cols))) for _, g0, n in pieces]
    views = {c.offsets: rows2d[l0: l0 + n] for c, (l0, _, n) in zip(chunks, pieces)}

    def create_write_items(fqn, obj):
        return [WriteItem(index=MetadataIndex(fqn, c.offsets), type=WriteItemType.SHARD,
                          tensor_data=TensorWriteData(chunk=c, properties=TensorProperties.create_from_tensor(rows2d),
                                                      size=size)) for c in chunks]

    def get_tensor_shard(index):
        return views[torch.Size(index.offset)]

    t.__create_write_items__ = create_write_items
    t.__create_chunk_list__ = lambda: list(chunks)
    t.__get_tensor_shard__ = get_tensor_shard
    # the load planner compares ``obj.size()`` with the stored (whole) size before it asks for the chunk list
    t.size = lambda *dim: size if not dim else size[dim[0]]
    t._mb_rewrap = lambda new_local: _as_row_pieces(new_local, slot, sharded)   # after a dtype conversion
    return t


class ModelWrapper(Stateful):
    """fp32 master weights (sharded) plus persistent buffers, keyed by FQN."""

    def __init__(self, model: nn.Module):
        self.model = model

    def state_dict(self) -> dict[str, Any]:
        sharded = getattr(self.model, "_sharded", None)
        out: dict[str, Any] = {}
        if sharded is None:
            out.update({k: v for k, v in self.model.state_dict().items()})
            return out
        for u in sharded.units:
            for sl in u.slots:
                out[sl.fqn] = _as_dtensor(sl.master.data, sl, sharded)
        for name, buf in self.model.named_buffers():
            mod_name, _, leaf = name.rpartition(".")
            owner = self.model.get_submodule(mod_name) if mod_name else self.model
            if leaf not in owner._non_persistent_buffers_set:
                out[name] = buf
        return out

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        sharded = getattr(self.model, "_sharded", None)
        if sharded is None:
            self.model.load_state_dict(state_dict, strict=False)
            return
        # DCP loaded in place into the master shards; refresh the compute-dtype copy
        sharded.lowp_fresh = False
        sharded.gather_params()


class OptimizerWrapper(Stateful):
    def __init__(self, model: nn.Module, optimizer):
        self.model, self.optimizer = model, optimizer

    def _merged(self) -> dict[str, Any]:
        """One ``state.<fqn>.<key>`` namespace and one ``param_groups`` list over ALL optimizers of the container, in
        their order: what ``get_optimizer_state_dict(model, [opt0, opt1, ...])`` gives the reference's wrapper
        (maester/checkpoint.py:54-70), so the default Muon + AdamW job has the same keys on disk on both sides.  (The
        container's own ``state_dict`` prefixes ``opt{i}_``; like the reference's, it is not what checkpoints use.)"""
        opts = getattr(self.optimizer, "optimizers", None)
        if opts is None or len(opts) == 1:
            return self.optimizer.state_dict()
        out: dict[str, Any] = {}
        groups: list = []
        for opt in opts:
            sd = self.optimizer._opt_state(opt)
            groups += sd.pop("param_groups")
            out.update(sd)
        out["param_groups"] = groups
        return out

    def state_dict(self) -> dict[str, Any]:
        sharded = getattr(self.model, "_sharded", None)
        flat = self._merged()
        if sharded is None:
            return flat
        slots = {sl.fqn: sl for u in sharded.units for sl in u.slots}
        out: dict[str, Any] = {}
        for k, v in flat.items():
            if torch.is_tensor(v) and v.dim() > 0 and ".state." in f".{k}":
                fqn = k.split("state.", 1)[1].rsplit(".", 1)[0]
                if fqn in slots and v.shape[1:] == slots[fqn].shape[1:]:
                    v = _as_dtensor(v, slots[fqn], sharded)
            out[k] = v
        return out

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        plain = {}
        for k, v in state_dict.items():
            if hasattr(v, "to_local"):
                v = v.to_local()
            plain[k] = v
        opts = getattr(self.optimizer, "optimizers", None)
        if opts is None or len(opts) == 1:
            self.optimizer.load_state_dict(plain)
            return
        first = 0
        for opt in opts:   # every optimizer takes the entries of its own parameters and its run of the group list
            names = {self.optimizer._names.get(id(p), str(id(p))) for g in opt.param_groups for p in g["params"]}
            sub = {k: v for k, v in plain.items()
                   if k.startswith("state.") and k[len("state."):].rpartition(".")[0] in names}
            sub["param_groups"] = plain.get("param_groups", [])[first:first + len(opt.param_groups)]
            first += len(opt.param_groups)
            self.optimizer._load_opt_state(opt, sub)


def resume_step(cfg) -> int:
    """The optimizer step of the checkpoint that ``CheckpointManager.load()`` will resume from with this configuration
    (0: none, or a model-only load from ``forced_load_path``).  The data pipeline is built before the manager exists and
    needs the step to load the loader state that belongs to it."""
    if not cfg.enable_checkpoint or cfg.forced_load_path:
        return 0
    folder = os.path.join(cfg.dump_dir, cfg.job_name, cfg.checkpoint_folder)
    if not os.path.isdir(folder):
        return 0
    steps = [int(m.group(1)) for f in os.listdir(folder) if (m := re.fullmatch(r"step-(\d+)", f))]
    return max(steps) if steps else 0


class CheckpointManager:
    def __init__(self, model: nn.Module, optimizer, lr_scheduler, dataloader, states: dict[str, Any], cfg) -> None:
        self.enable_checkpoint: bool = cfg.enable_checkpoint
        self.forced_load_path: str | None = cfg.forced_load_path
        if not self.enable_checkpoint:
            return
        self.states = states
        self.states.update({
            "model": ModelWrapper(model),
            "optimizer": OptimizerWrapper(model, optimizer),
            "lr_scheduler": lr_scheduler,
        })
        self.dataloader = dataloader
        self.folder = os.path.join(cfg.dump_dir, cfg.job_name, cfg.checkpoint_folder)
        self.interval_type = IntervalType.STEPS
        self.interval = cfg.checkpoint_interval
        self.model_weights_only = cfg.model_weights_only
        self.export_dtype = TORCH_DTYPE_MAP[cfg.export_dtype]
        self.begin = 0.0
        # CPU-side coordination group, as in the reference (time-based interval agreement)
        self.pg = dist.new_group(backend="gloo") if dist.is_initialized() else None
        logger.info(f"Checkpointing active. Checkpoints will be loaded from and saved to {self.folder}")

    def reset(self) -> None:
        self.begin = time.monotonic()

    def _stateful_loader(self):
        """What carries the position of the data stream in THIS process: a loader with its own ``state_dict``, or the
        dataset of a loader without worker processes (the packed SFT reader: its epoch and index advance as batches
        are taken, nothing is prefetched).  Pipelines that run inside a worker process save themselves from there
        (``Checkpoint_Dataset``); the copy of the dataset in this process never moves and is not saved."""
        dl = self.dataloader
        if dl is None:
            return None
        if hasattr(dl, "state_dict") and hasattr(dl, "load_state_dict"):
            return dl
        ds = getattr(dl, "dataset", None)
        if getattr(dl, "num_workers", 1) == 0 and hasattr(ds, "state_dict") and hasattr(ds, "load_state_dict"):
            return ds
        return None

    def _checkpoint_id(self, step: int) -> str:
        return os.path.join(self.folder, f"step-{step}")

    def _no_dist(self) -> bool:
        return not dist.is_initialized()

    def will_save(self, curr_step: int, force: bool = False) -> bool:
        return bool(self.enable_checkpoint and (force or curr_step % self.interval == 0))

    def save(self, curr_step: int, force: bool = False) -> None:
        if not self.will_save(curr_step, force):
            return
        _check_device_status()  # raises before anything is written
        states: dict[str, Any] = self.states
        if force and self.model_weights_only:
            sd = self.states["model"].state_dict()
            if self.export_dtype != torch.float32:
                sd = {k: (v._mb_rewrap(v.to(self.export_dtype)) if hasattr(v, "_mb_rewrap") else v.to(self.export_dtype))
                      for k, v in sd.items()}
            states = {"model": sd}
            logger.info(f"Saving a model weights only checkpoint in {self.export_dtype} at step {curr_step}")
        else:
            logger.info(f"Saving a full checkpoint at step {curr_step}")
        begin = time.monotonic()
        dcp.save(states, checkpoint_id=self._checkpoint_id(curr_step), no_dist=self._no_dist())
        stateful = self._stateful_loader()
        if stateful is not None:
            rank = dist.get_rank() if dist.is_initialized() else 0
            d = os.path.join(self.folder, "dataloader", f"step-{curr_step}")
            os.makedirs(d, exist_ok=True)
            torch.save(stateful.state_dict(), os.path.join(d, f"loader_state_{rank}.pth"))
        self.reset()
        logger.info(f"Finished saving the checkpoint in {time.monotonic() - begin:.2f} seconds")

    def latest_step(self) -> int | None:
        if not os.path.isdir(self.folder):
            return None
        steps = [int(m.group(1)) for f in os.listdir(self.folder) if (m := re.fullmatch(r"step-(\d+)", f))]
        return max(steps) if steps else None

    def load(self, step: int = -1, model_only: bool = False) -> bool:
        if not self.enable_checkpoint:
            return False
        if self.forced_load_path:
            if not os.path.isdir(self.forced_load_path):
                raise ValueError(f"Checkpoint folder {self.forced_load_path} does not exist")
            logger.info(f"Forcing load from {self.forced_load_path}")
            self._load({"model": self.states["model"]}, self.forced_load_path)
            return True
        if step == -1:
            found = self.latest_step()
            if found is None:
                return False
            step = found
        elif not os.path.isdir(self._checkpoint_id(step)):
            return False
        states = self.states
        if step == 0 or model_only:
            states = {"model": self.states["model"]}
        logger.info(f"Loading the checkpoint at step {step}, containing keys {list(states.keys())}")
        begin = time.monotonic()
        self._load(states, self._checkpoint_id(step))
        stateful = self._stateful_loader()
        if states is self.states and stateful is not None:
            rank = dist.get_rank() if dist.is_initialized() else 0
            f = os.path.join(self.folder, "dataloader", f"step-{step}", f"loader_state_{rank}.pth")
            if os.path.exists(f):
                stateful.load_state_dict(torch.load(f, weights_only=False))
        logger.info(f"Finished loading the checkpoint in {time.monotonic() - begin:.2f} seconds")
        return True

    def _load(self, states: dict[str, Any], path: str) -> None:
        from torch.distributed.checkpoint.api import CheckpointException
        try:
            renamed = _stored_names(path)
            if renamed:
                self._load_renamed(states, path, renamed)
            else:
                dcp.load(states, checkpoint_id=path, no_dist=self._no_dist())
        except CheckpointException as e:  # derives from BaseException: turn it into an ordinary error
            raise RuntimeError(f"checkpoint {path} is unreadable or does not match the model: {e}") from e

    def _load_renamed(self, states: dict[str, Any], path: str, stored: dict[str, str]) -> None:
        """Load a checkpoint whose keys carry ``_orig_mod`` components (it was written from modules wrapped by
        ``torch.compile``): every flat state dict is read under the stored names and handed back under ours."""
        logger.info(f"{path}: {len(stored)} keys were written through a torch.compile wrapper; mapping them")
        plain: dict[str, Any] = {}
        for top, obj in states.items():
            sd = obj.state_dict() if isinstance(obj, Stateful) else obj
            if not (isinstance(sd, dict) and all(isinstance(k, str) for k in sd)):
                plain[top] = obj
                continue
            there = {stored.get(f"{top}.{k}", f"{top}.{k}")[len(top) + 1:]: v for k, v in sd.items()}
            dcp.load({top: there}, checkpoint_id=path, no_dist=self._no_dist())
            back = {k: there[stored.get(f"{top}.{k}", f"{top}.{k}")[len(top) + 1:]] for k in sd}
            if isinstance(obj, Stateful):
                obj.load_state_dict(back)
            else:
                obj.update(back)
        if plain:
            dcp.load(plain, checkpoint_id=path, no_dist=self._no_dist())


def _stored_names(path: str) -> dict[str, str]:
    """{name without ``_orig_mod`` components: name as stored} for the keys of a checkpoint that have such components
    (empty for an ordinary checkpoint, or when the metadata cannot be read: the load itself then reports why)."""
    try:
        meta = dcp.FileSystemReader(path).read_metadata()
    except Exception:
        return {}
    out = {}
    for k in meta.state_dict_metadata:
        clean = ".".join(part for part in k.split(".") if part != "_orig_mod")
        if clean != k:
            out[clean] = k
    return out
