"""Parallel degrees and the device mesh (reference: maester/parallelisms/parallel_dims.py:10-213).

Mesh dimension names and the flattened aliases (``dp``, ``dp_shard_cp``, ``dp_cp``, ``ep``) match the
reference.  Context parallelism, which the reference only reserves names for, is a real degree
here: ``dp_shard_cp`` is the product of ``dp_shard`` and ``cp`` and is the group parameters are
sharded over.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch.distributed.device_mesh import DeviceMesh, init_device_mesh

from maester_b200.log_utils import logger


@dataclass
class ParallelDims:
    dp_replicate: int
    dp_shard: int
    tp: int
    ep: int
    world_size: int
    enable_loss_parallel: bool
    cp: int = 1
    _world_mesh: DeviceMesh | None = None

    def __post_init__(self):
        self._validate()

    def _validate(self) -> None:
        for d in (self.dp_replicate, self.tp, self.ep, self.cp):
            assert d >= 1, "Parallelism degree should be >= 1, except for dp_shard"
        assert self.dp_shard == -1 or self.dp_shard >= 1, "dp_shard must be -1 or >= 1"
        if self.dp_shard < 0:
            self.dp_shard = self.world_size // (self.dp_replicate * self.tp * self.cp)
        assert self.dp_shard >= 1
        prod = self.dp_replicate * self.dp_shard * self.cp * self.tp
        assert prod == self.world_size, (
            f"Invalid parallel dims: dp_replicate({self.dp_replicate}) * dp_shard({self.dp_shard}) * "
            f"cp({self.cp}) * tp({self.tp}) != WORLD_SIZE({self.world_size})"
        )
        if self.ep > 1:
            assert self.ep % self.tp == 0 and (self.dp_shard * self.cp * self.tp) % self.ep == 0

    # ------------------------------------------------------------------ mesh
    def _dims(self) -> tuple[list[int], list[str]]:
        if self.ep > 1:
            mod_ep = self.dp_shard * self.cp * self.tp // self.ep
            in_ep = self.ep // self.tp
            cand = [(self.dp_replicate, "dp_replicate"), (mod_ep, "dp_shard_mod_ep"), (in_ep, "dp_shard_in_ep"),
                    (self.tp, "tp")]
            keep = [(d, n) for d, n in cand if d > 1 or n == "dp_shard_mod_ep"]
        else:
            cand = [(self.dp_replicate, "dp_replicate"), (self.dp_shard, "dp_shard"), (self.cp, "cp"), (self.tp, "tp")]
            keep = [(d, n) for d, n in cand if d > 1]
            if not keep:
                keep = [(1, "dp_shard")]
        return [d for d, _ in keep], [n for _, n in keep]

    def build_mesh(self, device_type: str | None = None) -> DeviceMesh:
        device_type = device_type or ("cuda" if torch.cuda.is_available() else "cpu")
        dims, names = self._dims()
        logger.info(f"Building {len(dims)}-D device mesh with {names}, {dims}")
        mesh = init_device_mesh(device_type, dims, mesh_dim_names=tuple(names))
        have = set(names)

        def flat(parts: list[str], alias: str) -> None:
            parts = [p for p in parts if p in have]
            if not parts:
                return
            if len(parts) == 1 and parts[0] == alias:
                return
            mesh[tuple(parts)]._flatten(mesh_dim_name=alias)

        if self.ep > 1:
            shard = ["dp_shard_mod_ep", "dp_shard_in_ep"]
            flat(["dp_replicate"] + shard, "dp")
            flat(shard, "dp_shard_cp")
            flat(["dp_replicate"] + shard, "dp_cp")
            flat(["dp_shard_in_ep"], "ep")  # experts are split over ep/tp ranks and, inside, by tp
        else:
            flat(["dp_replicate", "dp_shard"], "dp")
            flat(["dp_shard", "cp"], "dp_shard_cp")
            flat(["dp_replicate", "dp_shard", "cp"], "dp_cp")
        return mesh

    @property
    def world_mesh(self) -> DeviceMesh:
        if self._world_mesh is None:
            self._world_mesh = self.build_mesh()
        return self._world_mesh

    # ------------------------------------------------------------------ predicates
    @property
    def dp_enabled(self) -> bool:
        return self.dp_replicate > 1 or self.dp_shard > 1

    @property
    def dp_replicate_enabled(self) -> bool:
        return self.dp_replicate > 1

    @property
    def dp_shard_enabled(self) -> bool:
        return self.dp_shard > 1

    @property
    def cp_enabled(self) -> bool:
        return self.cp > 1

    @property
    def tp_enabled(self) -> bool:
        return self.tp > 1

    @property
    def ep_enabled(self) -> bool:
        return self.ep > 1

    @property
    def fsdp_enabled(self) -> bool:
        return self.dp_shard_enabled or self.cp_enabled

    @property
    def loss_parallel_enabled(self) -> bool:
        return self.tp > 1 and self.enable_loss_parallel

    @property
    def fsdp_gradient_divide_factor(self) -> int:
        # matches the reference: expert parameters sharded over a different mesh still divide by
        # the full data-parallel size
        return self.dp_replicate * self.dp_shard * self.cp

    @property
    def non_data_parallel_size(self) -> int:
        return self.cp * self.tp

    @property
    def model_parallel_size(self) -> int:
        return self.tp

    def mesh_group(self, name: str):
        """Process group of a (possibly flattened) mesh dimension, or None if the dimension is absent."""
        try:
            return self.world_mesh[name].get_group()
        except (KeyError, RuntimeError, ValueError):
            return None
