"""Reading and writing the two on-disk formats of the converters.

* Hugging Face side: a directory with ``config.json`` and either ``model.safetensors`` or shards listed
  in ``model.safetensors.index.json``.
* Native side: a ``torch.distributed.checkpoint`` directory whose ``model`` entry maps parameter FQNs
  to tensors (what the trainer writes, and what ``to_dcp`` scripts write as ``{"model": flat_dict}``,
  reference: scripts/convert/gemma/to_dcp.py:85-89).  A DCP checkpoint is read WITHOUT building the
  model or a process group: the metadata is walked and every ``model.*`` tensor is materialised on
  the CPU (the reference does the same through ``_EmptyStateDictLoadPlanner``,
  scripts/convert/gemma/from_dcp.py:44-70).
"""
from __future__ import annotations

import json
import os
from pathlib import Path

import torch


# ----------------------------------------------------------------------------------------- safetensors
def read_hf_dir(path: str | os.PathLike) -> tuple[dict[str, torch.Tensor], dict]:
    """(state dict, config dict) of an HF checkpoint directory."""
    from safetensors import safe_open

    path = Path(path)
    index = path / "model.safetensors.index.json"
    if index.is_file():
        with open(index) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
    else:
        files = sorted(p.name for p in path.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors files in {path}")
    sd: dict[str, torch.Tensor] = {}
    for name in files:
        with safe_open(str(path / name), framework="pt", device="cpu") as f:
            for k in f.keys():
                sd[k] = f.get_tensor(k)
    cfg_path = path / "config.json"
    cfg = json.loads(cfg_path.read_text()) if cfg_path.is_file() else {}
    return sd, cfg


def write_hf_dir(path: str | os.PathLike, sd: dict[str, torch.Tensor], config: dict | None = None,
                 max_shard_bytes: int = 5 * 2**30, dtype: torch.dtype | None = torch.bfloat16) -> list[str]:
    """Write ``sd`` as (sharded) safetensors with an index; returns the file names."""
    from safetensors.torch import save_file

    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    shards: list[dict[str, torch.Tensor]] = [{}]
    size = 0
    for k in sorted(sd):
        t = sd[k].detach()
        if dtype is not None and t.is_floating_point():
            t = t.to(dtype)
        t = t.contiguous().cpu()
        nbytes = t.numel() * t.element_size()
        if size + nbytes > max_shard_bytes and shards[-1]:
            shards.append({})
            size = 0
        shards[-1][k] = t
        size += nbytes
    names, weight_map, total = [], {}, 0
    for i, shard in enumerate(shards):
        name = "model.safetensors" if len(shards) == 1 else f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(shard, str(path / name), metadata={"format": "pt"})
        names.append(name)
        for k, t in shard.items():
            weight_map[k] = name
            total += t.numel() * t.element_size()
    if len(shards) > 1:
        (path / "model.safetensors.index.json").write_text(
            json.dumps({"metadata": {"total_size": total}, "weight_map": weight_map}, indent=2))
    if config is not None:
        (path / "config.json").write_text(json.dumps(config, indent=2))
    return names


# ----------------------------------------------------------------------------------------- DCP
def write_dcp(path: str | os.PathLike, model_sd: dict[str, torch.Tensor]) -> None:
    """Write ``{"model": model_sd}`` as a single-process DCP checkpoint."""
    import torch.distributed.checkpoint as dcp

    Path(path).mkdir(parents=True, exist_ok=True)
    dcp.save({"model": {k: v.contiguous() for k, v in model_sd.items()}}, checkpoint_id=str(path), no_dist=True)


def read_dcp_model(path: str | os.PathLike, prefix: str = "model.") -> dict[str, torch.Tensor]:
    """All tensors stored under ``model`` in a DCP checkpoint, on the CPU, keyed by FQN."""
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint.metadata import TensorStorageMetadata

    reader = dcp.FileSystemReader(str(path))
    meta = reader.read_metadata()
    target: dict[str, torch.Tensor] = {}
    for key, m in meta.state_dict_metadata.items():
        if key.startswith(prefix) and isinstance(m, TensorStorageMetadata):
            target[key] = torch.empty(m.size, dtype=m.properties.dtype)
    if not target:
        raise KeyError(f"{path}: no tensors under '{prefix}'")
    nested: dict = {}
    for key, t in target.items():  # DCP flattens nested dicts with '.', so "model" -> {fqn: tensor} is one level
        nested.setdefault(prefix.rstrip("."), {})[key[len(prefix):]] = t
    dcp.load(nested, checkpoint_id=str(path), no_dist=True)
    return nested[prefix.rstrip(".")]


def find_job_config(checkpoint_dir: str | os.PathLike) -> dict | None:
    """``config.json`` of the job that wrote a checkpoint (``<job>/checkpoints/step-N`` -> ``<job>/config.json``)."""
    p = Path(checkpoint_dir).resolve()
    for parent in [p, *p.parents][:4]:
        f = parent / "config.json"
        if f.is_file():
            try:
                d = json.loads(f.read_text())
            except json.JSONDecodeError:
                continue
            if "model_name" in d and "flavor" in d:
                return d
    return None
