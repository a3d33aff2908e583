"""Sharded data parallelism over flat buffers ("FSDP" of this framework).

The reference wraps every transformer block and the root with PyTorch FSDP2 ``fully_shard``
(maester/parallelisms/parallelize_llama.py:265-286, parallelize_gemma.py:268-289): bf16 parameters
are all-gathered per block, gradients reduce-scattered in fp32 and divided by the data-parallel
size, fp32 master shards feed the optimizer.  This runtime keeps those semantics (dim-0 sharding
per parameter, bf16 compute / fp32 reduce / fp32 master and optimizer state, per-block units,
gradient-sync toggle for accumulation) with a layout chosen for 180 GB GPUs:

* every parameter of the model is a view into one flat ``full`` buffer in the compute dtype; fused
  projections (qkv, gate/up) are single GEMMs over adjacent views;
* weight gradients accumulate in fp32 straight from the GEMM epilogues into ``main_grad`` views of a
  flat gradient buffer, so there is no per-parameter ``.grad`` allocation, cast or copy;
* each rank owns rows ``[r*c, (r+1)*c)`` of every parameter (``c = ceil(dim0 / world)``) in flat fp32
  ``master`` / ``grad`` shards, which is the shard geometry DCP expects for ``Shard(0)`` DTensors;
* the full bf16 model stays resident between steps (it is 2 bytes/param), so a step needs ONE
  all-gather of the updated shards (issued per unit on a side stream right after the optimizer
  step, consumed by forward pre-hooks) and ONE reduce-scatter per unit, launched from backward hooks
  so it overlaps the backward of the preceding unit.

* with peer-mapped (symmetric) buffers the reduce-scatter, the AdamW update and the all-gather of a unit are one
  kernel (``csrc/comm.cu``) that reads the peers' gradient buffers and writes the peers' parameter buffers through
  NVSwitch; it is launched per unit from the same backward hooks once the optimizers have announced the step
  (``_eager_update``), so it runs under the backward pass of the earlier blocks.

With one rank the shard and full buffers coincide and no communication code runs.

Resharding mode (``reshard=True``; the reference's ``fsdp_reshard_after_forward`` / ``CPUOffloadPolicy``,
parallelize_llama.py:265-286, parallelize_deepseek.py:264-300).  For models whose whole bf16 copy plus a whole fp32
gradient buffer (6 bytes per parameter per GPU) would not fit, a block's parameters exist in full only while the block
runs: every rank keeps just its rows (``shard_lp``), the blocks share ``STAGES`` staging buffers of the largest block's
size (block i always uses buffer i % STAGES, so parameter views never move), a block is all-gathered into its buffer on
the side stream while the previous block computes (forward) or while the next block's backward runs (backward), and
its fp32 gradients live in a matching staging buffer that is reduce-scattered into the owner's shard and cleared as
soon as the backward pass has left the block.  Only the root unit (embedding, final norm, head) stays gathered for
the whole step.  Per GPU this needs ``2 bytes x (root + STAGES blocks)`` and ``4 bytes x (root + STAGES blocks)``
instead of ``6 bytes x all parameters``.  Gradient accumulation reduces after every micro-batch in this mode (the
staging buffers are reused), and ``cpu_offload`` keeps the fp32 master weights, gradient shards and optimizer state
in pinned host memory with the optimizer step running there.  Where the peer-memory plane is usable the ranks' rows
live in a symmetric buffer and a block is gathered by ONE launch of the library's table-driven copy kernel
(``csrc/cp_ring.cu::mb_peer_gather``: every (parameter, owner) piece goes from the owner's rows straight to its place
in the staging buffer over NVLink), ordered by one cross-rank barrier per step; otherwise by an all-gather of the
process group plus per-parameter copies.

Gradient clearing.  With one rank the AdamW kernel clears the accumulation buffer as it reads it, so ``zero_grad``
has nothing left to do; with several ranks the buffer is cleared on a side stream while the forward pass (which never
touches it) runs, and the last block's forward pre-hook waits for that before the loss layer or the backward pass can
write a gradient.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field

import torch
import torch.distributed as dist
import torch.nn as nn

from maester_b200.log_utils import logger


@dataclass
class ParamSlot:
    fqn: str
    param: nn.Parameter          # compute-dtype view into `full`
    shape: torch.Size
    rows: int                    # dim 0 (1 for scalars)
    row_numel: int
    chunk_rows: int              # rows owned per rank (ceil)
    full_off: int = 0            # offset into the flat full buffer (padded rows included)
    shard_off: int = 0           # offset into the flat shard buffers
    master: nn.Parameter | None = None  # fp32 shard view given to the optimizer
    dom: int = 0                 # 0: sharded over the data-parallel shard group; 1: expert-parallel local
                                 # slice, sharded over the ranks that hold the same experts
    global_rows: int = 0         # dim 0 of the whole (all experts) tensor
    row_base: int = 0            # first global row of this rank's local slice (expert-parallel offset)
    tp_dim: int = -1             # tensor-parallel slice dimension of this parameter (-1: not tensor-parallel)
    tp_size: int = 1
    # A tensor-parallel slice on dim 0 that is NOT one contiguous row range of the whole tensor (the fused q|k|v
    # projection split by head groups): the local rows are these ranges of the whole tensor, in order:
    # ((first global row, rows), ...).  None: the slice is the contiguous range given by the rank.
    tp_segments: tuple | None = None

    @property
    def padded_numel(self) -> int:
        return self.chunk_rows * self.row_numel

    @property
    def global_shape(self) -> torch.Size:
        if not len(self.shape):
            return self.shape
        dims = [self.global_rows, *self.shape[1:]]
        if self.tp_dim >= 0:
            dims[self.tp_dim] *= self.tp_size
        return torch.Size(dims)


@dataclass
class Domain:
    """A set of ranks that parameters are sharded over (process group, its size, this rank's index)."""
    group: object
    world: int
    rank: int


@dataclass
class Unit:
    name: str
    module: nn.Module
    slots: list[ParamSlot] = field(default_factory=list)
    full_lo: int = 0
    full_hi: int = 0
    shard_lo: int = 0
    shard_mid: int = 0           # dense slots occupy [shard_lo, shard_mid), expert slots [shard_mid, shard_hi)
    shard_hi: int = 0
    gather_event: torch.cuda.Event | None = None
    gathered: bool = True
    grads_pending: bool = False
    eager_done: bool = False     # fused mode: this step's update of the unit already ran under the backward pass


def _ordered_params(module: nn.Module, prefix: str, seen: set, skip_modules: set):
    """(fqn, param) in registration order, except that a module may pin the order of its direct
    children with ``fused_param_order`` so that fused projections are adjacent in memory."""
    out = []
    for n, p in module.named_parameters(recurse=False):
        if p is not None and id(p) not in seen:
            seen.add(id(p))
            out.append((f"{prefix}{n}", p))
    children = dict(module.named_children())
    order = list(getattr(module, "fused_param_order", ())) + [c for c in children if c not in getattr(module, "fused_param_order", ())]
    for cname in order:
        child = children[cname]
        if child in skip_modules:
            continue
        out.extend(_ordered_params(child, f"{prefix}{cname}.", seen, skip_modules))
    return out


class ShardedModel:
    """Owns the flat buffers of ``model`` and the collectives that keep them consistent."""

    def __init__(self, model: nn.Module, unit_modules: list[tuple[str, nn.Module]], *, device: torch.device,
                 param_dtype: torch.dtype = torch.bfloat16, reduce_dtype: torch.dtype = torch.float32,
                 shard_group=None, replicate_group=None, gradient_divide_factor: float | None = None,
                 tp_group=None, fused_comm: bool = False, expert_group=None, ep_size: int = 1, ep_rank: int = 0,
                 reshard: bool = False, cpu_offload: bool = False):
        self.model = model
        self.device = device
        self.param_dtype, self.reduce_dtype = param_dtype, reduce_dtype
        self.group = shard_group
        self.replicate_group = replicate_group
        self.tp_group = tp_group
        self.world = dist.get_world_size(shard_group) if (shard_group is not None and dist.is_initialized()) else 1
        self.rank = dist.get_rank(shard_group) if self.world > 1 else 0
        self.rep_world = dist.get_world_size(replicate_group) if replicate_group is not None else 1
        # expert-parallel parameters (marked ``ep_local`` by apply_ep) hold E/ep experts per rank and are
        # sharded over the ranks with the same experts (reference: parallelize_deepseek.py:315-355)
        e_world = dist.get_world_size(expert_group) if (expert_group is not None and dist.is_initialized()) else 1
        e_rank = dist.get_rank(expert_group) if e_world > 1 else 0
        self.domains = [Domain(shard_group, self.world, self.rank), Domain(expert_group, e_world, e_rank)]
        self.ep_size, self.ep_rank = ep_size, ep_rank
        self.divide = gradient_divide_factor or float(self.world * self.rep_world)
        self.require_sync = True
        self.lowp_fresh = False
        self.grad_cleared_by_optimizer = False   # set by the optimizer container after a step that cleared the gradients
        self._use_cuda = device.type == "cuda"
        self.comm_stream = torch.cuda.Stream(device) if (self._use_cuda and self.world * self.rep_world > 1) else None

        # ---- units: listed blocks first, everything left over forms the root unit
        seen: set = set()
        block_mods = {m for _, m in unit_modules}
        self.units: list[Unit] = []
        prefix_of = {m: n for n, m in model.named_modules()}
        for name, mod in unit_modules:
            u = Unit(name, mod)
            for fqn, p in _ordered_params(mod, prefix_of[mod] + ".", seen, set()):
                u.slots.append(self._slot(fqn, p))
            u.slots.sort(key=lambda sl: sl.dom)  # stable: dense first, fused-projection adjacency kept
            self.units.append(u)
        root = Unit("root", model)
        for fqn, p in _ordered_params(model, "", seen, block_mods):
            root.slots.append(self._slot(fqn, p))
        root.slots.sort(key=lambda sl: sl.dom)
        self.units.append(root)
        self.has_experts = any(sl.dom == 1 for u in self.units for sl in u.slots)
        self.root = root

        # ---- offsets (each parameter start is aligned to 256 elements: 16-byte TMA alignment for
        #      any dtype and whole 1 KiB lines for the optimizer kernel)
        def align(x: int) -> int:
            return (x + 255) // 256 * 256

        f = s = 0
        for u in self.units:
            u.full_lo, u.shard_lo = f, s
            u.shard_mid = -1
            for sl in u.slots:
                if sl.dom == 1 and u.shard_mid < 0:
                    u.shard_mid = s
                sl.full_off, sl.shard_off = f, s
                f = align(f + sl.padded_numel * self.domains[sl.dom].world)
                s = align(s + sl.padded_numel)
            u.full_hi, u.shard_hi = f, s
            if u.shard_mid < 0:
                u.shard_mid = s
        self.full_numel, self.shard_numel = f, s

        # ---- resharding mode (dense data-parallel sharding only)
        self.reshard = bool(reshard) and self.world > 1 and not self.has_experts
        if reshard and not self.reshard and self.world > 1:
            logger.warning("resharding is not available with expert-parallel parameters: keeping the model resident")
        self.cpu_offload = bool(cpu_offload) and self.reshard
        if cpu_offload and not self.cpu_offload:
            logger.warning("enable_cpu_offload needs the resharding mode (fsdp_reshard_after_forward != 'never', "
                           "data-parallel shard degree > 1): ignored")
        self.resharded = False          # becomes True once the weights are initialised and the full buffer is dropped
        self.stage: list[torch.Tensor] = []
        self.gstage: list[torch.Tensor] = []
        self.slot_owner: list[int] = []
        self.gslot_event: list = []
        if self.reshard:
            fused_comm = False          # the per-block gather / reduce-scatter below replace the fused step kernel

        # ---- buffers
        self.fused = False
        self.symm_full = self.symm_grad = None
        self.eager_hooks: list = []   # fused mode: callables(unit) that run the optimizer kernel for one unit
        self.eager_active = False     # set for the backward pass whose gradients the next optimizer step consumes
        if fused_comm and not self.has_experts and self.world > 1 and self.rep_world == 1 and param_dtype == torch.bfloat16 and all(
                sl.padded_numel % 4 == 0 for u in self.units for sl in u.slots):
            from maester_b200.parallel.symm import SymmBuffer, symmetric_memory_available
            if symmetric_memory_available(shard_group):
                try:
                    self.symm_full = SymmBuffer(f, param_dtype, device, shard_group)
                    self.symm_grad = SymmBuffer(f, torch.float32, device, shard_group)
                    self.fused = True
                except Exception as e:  # noqa: BLE001  (no peer access, unsupported driver, ...)
                    logger.warning(f"symmetric memory unavailable, using NCCL collectives: {e}")
                    self.symm_full = self.symm_grad = None
        self.full = self.symm_full.tensor.zero_() if self.fused else torch.zeros(f, dtype=param_dtype, device=device)
        state_dev = torch.device("cpu") if self.cpu_offload else device
        pin = self.cpu_offload and self._use_cuda
        self.master = torch.zeros(s, dtype=torch.float32, device=state_dev, pin_memory=pin)
        self.shard_grad = torch.zeros(s, dtype=torch.float32, device=state_dev, pin_memory=pin)
        if self.reshard:
            # until the weights are initialised the parameters are views of a temporary full buffer; gradients only
            # exist in the staging buffers created by _enter_reshard()
            self.full_grad = None
            self.shard_lp = self._symmetric_rows(s, param_dtype, device, shard_group)
        elif self.world > 1:
            self.full_grad = self.symm_grad.tensor.zero_() if self.fused else \
                torch.zeros(f, dtype=torch.float32, device=device)
            self.shard_lp = torch.zeros(s if not self.fused else 1, dtype=param_dtype, device=device)
        else:
            self.full_grad = self.shard_grad  # identical geometry with one rank
            self.shard_lp = self.full
        self._rebind_parameters()
        self._install_hooks()
        logger.info(
            f"ShardedModel: {sum(len(u.slots) for u in self.units)} params in {len(self.units)} units, "
            f"full={f * self.full.element_size() / 2**30:.2f} GiB {param_dtype}, "
            f"shard={s * 4 / 2**30:.2f} GiB fp32 x3 (master, grad + optimizer state), world={self.world}, "
            f"collectives={'own kernels over ' + ('NVLS multimem' if self.symm_grad.multicast_ptr else 'peer memory') if self.fused else ('nccl/gloo' if self.world * self.rep_world > 1 else 'none')}"
        )

    # ------------------------------------------------------------------ construction helpers
    def _slot(self, fqn: str, p: nn.Parameter) -> ParamSlot:
        shape = p.shape
        rows = shape[0] if p.dim() > 0 else 1
        row_numel = int(math.prod(shape[1:])) if p.dim() > 1 else 1
        dom = 1 if getattr(p, "ep_local", False) else 0
        chunk = (rows + self.domains[dom].world - 1) // self.domains[dom].world
        ep, er = (self.ep_size, self.ep_rank) if dom == 1 else (1, 0)
        tp_dim = int(getattr(p, "tp_dim", -1))
        tp_size = dist.get_world_size(self.tp_group) if (tp_dim >= 0 and self.tp_group is not None) else 1
        seg = getattr(p, "tp_segments", None)
        return ParamSlot(fqn, p, shape, rows, row_numel, chunk, dom=dom, global_rows=rows * ep, row_base=rows * er,
                         tp_dim=tp_dim if tp_size > 1 else -1, tp_size=tp_size,
                         tp_segments=tuple(seg) if (seg is not None and tp_size > 1) else None)

    def _rebind_parameters(self) -> None:
        """Point every model parameter at its view of ``full`` and create the fp32 master shards."""
        for u in self.units:
            for sl in u.slots:
                n = sl.rows * sl.row_numel
                pbuf, gbuf, base = self._unit_buffers(u)
                view = pbuf[sl.full_off - base: sl.full_off - base + n].view(sl.shape)
                new = nn.Parameter(view, requires_grad=sl.param.requires_grad)
                if gbuf is not None:
                    new.main_grad = gbuf[sl.full_off - base: sl.full_off - base + n].view(sl.shape)
                for attr in ("tp_replicated", "ep_local"):
                    if getattr(sl.param, attr, False):
                        setattr(new, attr, True)
                self._replace_param(sl.param, new)
                sl.param = new
                if sl.master is not None:
                    continue  # second binding (entering the resharding mode): the optimizers keep the shards they have
                lo, hi = self._own_rows(sl)
                m = self.master[sl.shard_off: sl.shard_off + (hi - lo) * sl.row_numel]
                g = self.shard_grad[sl.shard_off: sl.shard_off + (hi - lo) * sl.row_numel]
                shard_shape = (hi - lo, *sl.shape[1:]) if len(sl.shape) > 0 else ()
                mp = nn.Parameter(m.view(shard_shape), requires_grad=True)
                mp.grad = g.view(shard_shape)
                mp.fqn = sl.fqn
                sl.master = mp

    def _unit_buffers(self, u: Unit):
        """(parameter buffer, gradient buffer or None, offset of the buffers' element 0 in the flat numbering)."""
        if not self.resharded:
            return self.full, self.full_grad, 0
        if u is self.root:
            return self.root_full, self.root_grad, u.full_lo
        k = self.units.index(u) % self.STAGES
        return self.stage[k], self.gstage[k], u.full_lo

    STAGES = 2

    def _enter_reshard(self) -> None:
        """Drop the full parameter buffer: bind every block to its staging buffers, keep only the root gathered."""
        blocks = self.units[:-1]
        cap = max((u.full_hi - u.full_lo for u in blocks), default=0)
        dev = self.device
        self.stage = [torch.zeros(cap, dtype=self.param_dtype, device=dev) for _ in range(self.STAGES)]
        self.gstage = [torch.zeros(cap, dtype=torch.float32, device=dev) for _ in range(self.STAGES)]
        r = self.root
        self.root_full = self.full[r.full_lo:r.full_hi].clone()
        self.root_grad = torch.zeros(r.full_hi - r.full_lo, dtype=torch.float32, device=dev)
        self.full = None
        self.resharded = True
        self._setup_peer_gather()
        self.slot_owner = [-1] * self.STAGES
        self.gslot_event = [None] * self.STAGES
        self._rebind_parameters()
        if hasattr(self, "_by_master"):
            del self._by_master
        if self._use_cuda:
            torch.cuda.empty_cache()
        logger.info(
            f"ShardedModel: resharding mode, {self.STAGES} staging buffers of {cap * 2 / 2**20:.0f} MiB (+ fp32 gradients), "
            f"root unit resident ({(r.full_hi - r.full_lo) * 2 / 2**30:.2f} GiB), "
            f"optimizer state on {'the host' if self.cpu_offload else 'the device'}"
        )

    peer_gather = False   # blocks are gathered by the library's copy kernel over peer memory instead of NCCL
    symm_lp = None

    def _symmetric_rows(self, s: int, dtype, device, group) -> torch.Tensor:
        """Buffer of this rank's compute-dtype rows (resharding mode).  Where the peer-memory plane is usable it is a
        symmetric allocation, so that the other ranks can read the rows they need for a block directly."""
        usable = (device.type == "cuda" and 1 < self.world <= 8 and not self.has_experts and dtype == torch.bfloat16
                  and os.environ.get("MB_RESHARD_PEER_GATHER", "1") != "0")
        if usable:
            from maester_b200.parallel.symm import SymmBuffer, symmetric_memory_available
            if symmetric_memory_available(group):
                try:
                    self.symm_lp = SymmBuffer(s, dtype, device, group)
                    return self.symm_lp.tensor.zero_()
                except Exception as e:  # noqa: BLE001
                    logger.warning(f"symmetric memory unavailable for the block gathers, using NCCL: {e}")
                    self.symm_lp = None
        return torch.zeros(s, dtype=dtype, device=device)

    def _setup_peer_gather(self) -> None:
        """One copy table per block: entry = (offset in the block's staging buffer, offset in the owner's rows,
        length, owner).  Needs the symmetric row buffer and 16-byte aligned pieces."""
        if self.symm_lp is None:
            return
        blocks = self.units[:-1]
        if any((sl.padded_numel | sl.shard_off | (sl.full_off - u.full_lo)) % 8 for u in blocks for sl in u.slots):
            return
        world = self.domains[0].world
        self._gather_tables = {}
        for i, u in enumerate(blocks):
            self._gather_tables[i] = torch.tensor(gather_table(u, world), dtype=torch.int64, device=self.device)
        self.peer_gather = True
        self.symm_lp.barrier()   # every rank's rows are in place before the first gather

    def _replace_param(self, old: nn.Parameter, new: nn.Parameter) -> None:
        """Swap a Parameter object everywhere it is registered (tied weights appear more than once)."""
        for mod in self.model.modules():
            for k, v in list(mod._parameters.items()):
                if v is old:
                    mod._parameters[k] = new

    def _own_rows(self, sl: ParamSlot) -> tuple[int, int]:
        lo = min(sl.rows, self.domains[sl.dom].rank * sl.chunk_rows)
        hi = min(sl.rows, lo + sl.chunk_rows)
        return lo, hi

    # ------------------------------------------------------------------ views for the optimizer / checkpoint
    def named_master_parameters(self):
        for u in self.units:
            for sl in u.slots:
                yield sl.fqn, sl.master

    def slot_of(self, master: nn.Parameter) -> ParamSlot:
        if not hasattr(self, "_by_master"):
            self._by_master = {id(sl.master): sl for u in self.units for sl in u.slots}
        return self._by_master[id(master)]

    def flat_segments(self):
        """{master parameter: (offset, numel)} into the flat shard buffers (for the fused optimizer)."""
        return {sl.master: (sl.shard_off, sl.master.numel()) for u in self.units for sl in u.slots}

    # ------------------------------------------------------------------ per-tensor norms over the flat shard buffers
    def _slot_list(self) -> list[ParamSlot]:
        return [sl for u in self.units for sl in u.slots]

    def _norm_table(self):
        """Chunk table {offset, length, tensor = slot index} over every slot's shard (cached: geometry only)."""
        if getattr(self, "_norm_tab", None) is None:
            from maester_b200.optimizers.adamw import build_chunk_table
            segs = [(sl.shard_off, sl.master.numel(), 1.0, 0.0) for sl in self._slot_list() if sl.master.numel() > 0]
            idx = [i for i, sl in enumerate(self._slot_list()) if sl.master.numel() > 0]
            chunks, _, n = build_chunk_table(segs, self.device)
            self._norm_tab = (chunks, n, torch.tensor(idx, device=self.device, dtype=torch.long))
        return self._norm_tab

    @torch.no_grad()
    def shard_sqnorms(self, which: str = "grad") -> torch.Tensor:
        """fp32 [n_slots]: sum of squares of this rank's shard of every parameter (``which`` = "grad" | "master").
        One native launch on CUDA (multi-tensor kernel over the flat buffer), a loop of torch reductions on CPU."""
        flat = self.shard_grad if which == "grad" else self.master
        slots = self._slot_list()
        out = torch.zeros(len(slots), device=self.device, dtype=torch.float32)
        if flat.device != self.device:  # optimizer state offloaded to the host: reduce there
            for i, sl in enumerate(slots):
                n = sl.master.numel()
                if n:
                    out[i] = flat[sl.shard_off: sl.shard_off + n].pow(2).sum().to(self.device)
            return out
        if flat.is_cuda and flat.dtype == torch.float32:
            from maester_b200.ops import cuda as C
            chunks, n, idx = self._norm_table()
            if n:
                dense = torch.zeros(idx.numel(), device=self.device, dtype=torch.float32)
                C.multi_sqnorm(flat, chunks, n, dense)
                out[idx] = dense
            return out
        for i, sl in enumerate(slots):
            n = sl.master.numel()
            if n:
                out[i] = flat[sl.shard_off: sl.shard_off + n].float().pow(2).sum()
        return out

    @torch.no_grad()
    def global_sqnorms(self, which: str = "grad") -> torch.Tensor:
        """Per-parameter sums of squares over all ranks that hold a piece of the parameter: data-parallel shards (each
        slot's own sharding domain) and tensor-parallel slices; replicas are counted once."""
        sq = self.shard_sqnorms(which)
        if not dist.is_initialized():
            return sq
        slots = self._slot_list()
        for d, dom in enumerate(self.domains):
            if dom.world > 1:
                mask = torch.tensor([sl.dom == d for sl in slots], device=self.device)
                if bool(mask.any()):
                    part = torch.where(mask, sq, torch.zeros_like(sq))
                    dist.all_reduce(part, group=dom.group)
                    sq = torch.where(mask, part, sq)
        if self.tp_group is not None and dist.get_world_size(self.tp_group) > 1:
            mask = torch.tensor([sl.tp_dim >= 0 for sl in slots], device=self.device)
            if bool(mask.any()):
                part = torch.where(mask, sq, torch.zeros_like(sq))
                dist.all_reduce(part, group=self.tp_group)
                sq = torch.where(mask, part, sq)
        return sq

    @torch.no_grad()
    def clip_grad_norm(self, max_norm: float) -> torch.Tensor:
        """Scale the reduced gradient shards so that the global L2 norm is at most ``max_norm``; returns the norm
        before clipping (the reference's ``clip_grad_norm``, maester/utils.py:245-288, on the flat buffers: one norm
        launch, the all-reduces of a few hundred floats, one scale launch)."""
        sq = self.global_sqnorms("grad")
        if self.ep_size > 1 and dist.is_initialized():
            # expert tensors differ between expert-parallel ranks: add the other ranks' experts
            slots = self._slot_list()
            mask = torch.tensor([sl.dom == 1 for sl in slots], device=self.device)
            if bool(mask.any()) and getattr(self, "ep_group", None) is not None:
                part = torch.where(mask, sq, torch.zeros_like(sq))
                dist.all_reduce(part, group=self.ep_group)
                sq = torch.where(mask, part, sq)
        total = sq.sum().sqrt()
        coef = torch.clamp(max_norm / (total + 1e-6), max=1.0).reshape(1)
        if self.shard_grad.is_cuda and self.shard_grad.dtype == torch.float32:
            from maester_b200.ops import cuda as C
            chunks, n, _ = self._norm_table()
            if n:
                C.multi_sqnorm(self.shard_grad, chunks, n, None, coef)
        else:
            self.shard_grad.mul_(coef.to(self.shard_grad.device))
        return total

    # ------------------------------------------------------------------ initialisation
    @torch.no_grad()
    def init_master_from_full(self) -> None:
        """After ``model.init_weights()`` filled the compute-dtype parameters: broadcast rank 0's
        values (so all ranks agree) and load this rank's rows into the fp32 master shards."""
        # ranks that hold the same (tensor-parallel) slice of the model must start identical
        if not self.has_experts:
            for g in (self.group, self.replicate_group):
                if g is not None and dist.get_world_size(g) > 1:
                    dist.broadcast(self.full, group=g, group_src=0)
        else:  # expert slices differ between expert-parallel ranks: broadcast inside each slot's own domain
            for u in self.units:
                for sl in u.slots:
                    for g in (self.domains[sl.dom].group, self.replicate_group):
                        if g is not None and dist.get_world_size(g) > 1:
                            dist.broadcast(sl.param.data, group=g, group_src=0)
        if self.tp_group is not None and dist.get_world_size(self.tp_group) > 1:
            for u in self.units:
                for sl in u.slots:
                    if getattr(sl.param, "tp_replicated", False):
                        dist.broadcast(sl.param.data, group=self.tp_group, group_src=0)
        for u in self.units:
            for sl in u.slots:
                lo, hi = self._own_rows(sl)
                if hi > lo:
                    src = sl.param.data.reshape(sl.rows, -1)[lo:hi]
                    sl.master.data.view(hi - lo, -1).copy_(src)
        self.lowp_fresh = True
        if self.reshard and not self.resharded:
            self._shards_to_lowp()
            self._enter_reshard()

    @torch.no_grad()
    def _shards_to_lowp(self) -> None:
        """bf16 copy of this rank's master rows (what the per-block all-gathers send)."""
        self.shard_lp.copy_(self.master, non_blocking=True)
        if self.peer_gather:
            self.symm_lp.barrier()   # every rank's new rows are visible before anyone gathers a block from them

    @torch.no_grad()
    def load_full_weights(self, weights: dict[str, torch.Tensor]) -> None:
        """Load unsharded weights (by parameter name; already sliced for this rank's tensor / expert parallel part):
        every rank keeps its rows in the fp32 master shards and refreshes the compute-dtype copies.  Works in both
        modes; in the resharding mode the full model is never materialised."""
        for u in self.units:
            for sl in u.slots:
                w = weights[sl.fqn].to(torch.float32)
                lo, hi = self._own_rows(sl)
                if hi > lo:
                    sl.master.data.view(hi - lo, -1).copy_(w.reshape(sl.rows, -1)[lo:hi])
        self.lowp_fresh = False
        if self.reshard and not self.resharded:
            self._shards_to_lowp()
            self._enter_reshard()
        self.gather_params()

    # ------------------------------------------------------------------ hooks
    def _install_hooks(self) -> None:
        if self.world * self.rep_world == 1:
            return
        for i, u in enumerate(self.units[:-1]):
            u.module.register_forward_pre_hook(lambda m, a, u=u, i=i: self._pre_forward(u, i))
            u.module.register_full_backward_pre_hook(lambda m, g, i=i: self._on_backward_reach(i))
        def root_pre_forward(m, a):  # must return None: a returned value would replace the inputs
            self._wait_gather(self.root)
            self.mark_backward_start()

        self.model.register_forward_pre_hook(root_pre_forward)

    def _wait_gather(self, u: Unit) -> None:
        if u.gather_event is not None:
            torch.cuda.current_stream().wait_event(u.gather_event) if self._use_cuda else None
            u.gather_event = None

    def _pre_forward(self, u: Unit, i: int) -> None:
        if i == len(self.units) - 2:
            self._wait_zeroed()   # gradient buffer cleared (side stream) before anything can write into it
        if not self.resharded:
            self._wait_gather(u)
            return
        # resharding mode (also reached when a checkpointed block is recomputed inside the backward pass)
        self._ensure_block(i)
        if not self._in_backward and i + 1 < len(self.units) - 1:
            self._prefetch_block(i + 1)

    def _on_backward_reach(self, i: int) -> None:
        # backward has reached unit i, so unit i+1 (the one after it in forward order) is complete
        nblocks = len(self.units) - 1
        if self.resharded:
            self._in_backward = True
            self._ensure_block(i)
            k = i % self.STAGES
            if self.gslot_event[k] is not None and self._use_cuda:  # this block's gradient staging buffer is clear again
                torch.cuda.current_stream().wait_event(self.gslot_event[k])
                self.gslot_event[k] = None
        if i + 1 < nblocks:
            self._reduce_unit(self.units[i + 1])
        if self.resharded and i - 1 >= 0:
            self._prefetch_block(i - 1)

    # ------------------------------------------------------------------ resharding mode: per-block all-gather
    _in_backward = False

    @torch.no_grad()
    def _gather_block(self, i: int) -> None:
        """All-gather block i's parameters from the ranks' bf16 shards into its staging buffer (side stream)."""
        u = self.units[i]
        k = i % self.STAGES
        stream = self.comm_stream
        if stream is not None:
            stream.wait_stream(torch.cuda.current_stream())  # the buffer's previous owner has finished computing
        ctx = torch.cuda.stream(stream) if stream is not None else _null()
        buf = self.stage[k]
        with ctx, torch.autograd._unsafe_preserve_version_counter(buf):
            # (tensors saved for the backward pass are views of this buffer: block i always returns to the same
            # addresses, so refilling it must not look like an in-place modification to autograd)
            dom = self.domains[0]
            if self.peer_gather:
                # one launch: every (parameter, owner) piece goes straight from the owner's rows to its place
                from maester_b200.ops import cuda as C
                C.peer_gather(buf, self.symm_lp, self._gather_tables[i])
            else:
                n_shard = u.shard_hi - u.shard_lo
                recv = torch.empty(dom.world * n_shard, dtype=self.param_dtype, device=self.device)
                dist.all_gather_into_tensor(recv, self.shard_lp[u.shard_lo:u.shard_hi], group=dom.group)
                rv = recv.view(dom.world, n_shard)
                for sl in u.slots:
                    o = sl.full_off - u.full_lo
                    buf[o: o + sl.padded_numel * dom.world].view(dom.world, sl.padded_numel).copy_(
                        rv[:, sl.shard_off - u.shard_lo: sl.shard_off - u.shard_lo + sl.padded_numel])
            if stream is not None:
                u.gather_event = torch.cuda.Event()
                u.gather_event.record(stream)
        self.slot_owner[k] = i

    def _prefetch_block(self, i: int) -> None:
        if self.slot_owner[i % self.STAGES] != i:
            self._gather_block(i)

    def _ensure_block(self, i: int) -> None:
        if self.slot_owner[i % self.STAGES] != i:
            self._gather_block(i)
        self._wait_gather(self.units[i])

    # ------------------------------------------------------------------ collectives
    def set_requires_gradient_sync(self, flag: bool) -> None:
        self.require_sync = flag

    def mark_backward_start(self) -> None:
        self._in_backward = False  # called from the root's forward pre-hook: a new forward / backward pair begins
        for u in self.units:
            u.grads_pending = True

    @torch.no_grad()
    def _reduce_unit(self, u: Unit) -> None:
        """Reduce-scatter (and replicate all-reduce) of one unit's accumulated fp32 gradients."""
        if not u.grads_pending or not (self.require_sync or self.resharded):
            return  # (the resharding mode reduces after every micro-batch: its staging buffers are reused)
        u.grads_pending = False
        tp_sync = self.tp_group is not None and dist.get_world_size(self.tp_group) > 1
        for sl in u.slots:  # gradients that ordinary autograd left in .grad (plain-PyTorch op path)
            g = sl.param.grad
            if g is not None:
                sl.param.main_grad.add_(g.to(torch.float32))
                sl.param.grad = None
            if tp_sync and getattr(sl.param, "tp_replicated", False):
                dist.all_reduce(sl.param.main_grad, group=self.tp_group)
        if self.world * self.rep_world == 1 or self.fused:
            # fused mode: the optimizer kernel reduces straight from the peers' gradient buffers, for this unit
            # right away (on the side stream, under the backward pass of the earlier blocks) when the optimizers
            # have announced the step, else for all units at the optimizer step
            if self.fused and self.eager_active and self.eager_hooks:
                self._eager_update(u)
            return
        stream = self.comm_stream
        if stream is not None:
            stream.wait_stream(torch.cuda.current_stream())
        ctx = torch.cuda.stream(stream) if stream is not None else _null()
        with ctx:
            if self.resharded:
                self._reduce_unit_resharded(u)
                return
            shard = self.shard_grad[u.shard_lo:u.shard_hi]
            for dom, lo, hi, slots in self._segments(u):
                seg = self.shard_grad[lo:hi]
                if dom.world == 1:
                    if self.full_grad is not self.shard_grad:  # same geometry: move and clear
                        for sl in slots:
                            src = self.full_grad[sl.full_off: sl.full_off + sl.padded_numel]
                            self.shard_grad[sl.shard_off: sl.shard_off + sl.padded_numel].copy_(src)
                            src.zero_()
                    continue
                # pack rank-major: [rank][slot] so that the scatter leaves each rank its own rows
                n_shard = hi - lo
                send = torch.empty(dom.world * n_shard, dtype=self.reduce_dtype, device=self.device)
                sv = send.view(dom.world, n_shard)
                for sl in slots:
                    src = self.full_grad[sl.full_off: sl.full_off + sl.padded_numel * dom.world]
                    sv[:, sl.shard_off - lo: sl.shard_off - lo + sl.padded_numel].copy_(
                        src.view(dom.world, sl.padded_numel))
                    src.zero_()
                out = seg if self.reduce_dtype == torch.float32 else torch.empty(n_shard, dtype=self.reduce_dtype, device=self.device)
                dist.reduce_scatter_tensor(out, send, op=dist.ReduceOp.SUM, group=dom.group)
                if out is not seg:
                    seg.copy_(out)
            if self.rep_world > 1:
                dist.all_reduce(shard, op=dist.ReduceOp.SUM, group=self.replicate_group)
            shard.mul_(1.0 / self.divide)

    def _reduce_unit_resharded(self, u: Unit) -> None:
        """Resharding mode: reduce-scatter the unit's gradient staging buffer, ADD the result (divided) to this rank's
        gradient shard, clear the staging buffer for the block that uses it next.  Runs on the side stream."""
        _, gbuf, base = self._unit_buffers(u)
        dom = self.domains[0]
        n_shard = u.shard_hi - u.shard_lo
        send = torch.empty(dom.world * n_shard, dtype=self.reduce_dtype, device=self.device)
        sv = send.view(dom.world, n_shard)
        for sl in u.slots:
            o = sl.full_off - base
            src = gbuf[o: o + sl.padded_numel * dom.world]
            sv[:, sl.shard_off - u.shard_lo: sl.shard_off - u.shard_lo + sl.padded_numel].copy_(
                src.view(dom.world, sl.padded_numel))
        gbuf[: u.full_hi - u.full_lo].zero_()
        out = torch.empty(n_shard, dtype=self.reduce_dtype, device=self.device)
        dist.reduce_scatter_tensor(out, send, op=dist.ReduceOp.SUM, group=dom.group)
        if self.rep_world > 1:
            dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.replicate_group)
        seg = self.shard_grad[u.shard_lo:u.shard_hi]
        if seg.device != out.device:   # optimizer state on the host
            seg.add_(out.to(torch.float32).cpu(), alpha=1.0 / self.divide)
        else:
            seg.add_(out.to(torch.float32), alpha=1.0 / self.divide)
        if u is not self.root and self.comm_stream is not None:
            k = self.units.index(u) % self.STAGES
            ev = torch.cuda.Event()
            ev.record(self.comm_stream)
            self.gslot_event[k] = ev

    def _segments(self, u: Unit):
        """(domain, shard range, slots) of a unit: dense parameters first, then expert-parallel ones."""
        if u.shard_mid > u.shard_lo:
            yield self.domains[0], u.shard_lo, u.shard_mid, [sl for sl in u.slots if sl.dom == 0]
        if u.shard_hi > u.shard_mid:
            yield self.domains[1], u.shard_mid, u.shard_hi, [sl for sl in u.slots if sl.dom == 1]

    @torch.no_grad()
    def collect_autograd_grads(self) -> None:
        """Fold gradients that ordinary autograd left in ``param.grad`` (ops running on their
        plain-PyTorch path) into the flat fp32 accumulation buffer, then drop them."""
        for u in self.units:
            for sl in u.slots:
                g = sl.param.grad
                if g is not None:
                    sl.param.main_grad.add_(g.to(torch.float32))
                    sl.param.grad = None

    def finish_backward(self) -> None:
        """Call after ``loss.backward()``: reduces the units whose hooks cannot fire (first block, root)
        and makes the compute stream wait for all reductions.  Without gradient sync (accumulation
        micro-steps) the gradients are only folded into the accumulation buffer."""
        if not self.require_sync:
            self.collect_autograd_grads()
        if self.world * self.rep_world == 1:
            self.mark_backward_start()  # no forward hooks are installed without data parallelism
        for u in self.units:
            self._reduce_unit(u)
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)

    @torch.no_grad()
    def gather_params(self) -> None:
        """After the optimizer step: cast the updated master shards and all-gather them into ``full``,
        one unit at a time on the side stream; forward pre-hooks wait per unit."""
        if self.resharded:
            # every rank refreshes the bf16 copy of its rows; blocks are gathered when they run, the root unit now
            if not self.lowp_fresh or self.cpu_offload:
                self._shards_to_lowp()
            elif self.peer_gather:
                self.symm_lp.barrier()   # (the optimizer kernel wrote the rows) visible before anyone gathers a block
            self.lowp_fresh = False
            self.slot_owner = [-1] * self.STAGES
            stream = self.comm_stream
            if stream is not None:
                stream.wait_stream(torch.cuda.current_stream())
            ctx = torch.cuda.stream(stream) if stream is not None else _null()
            u, dom = self.root, self.domains[0]
            with ctx, torch.autograd._unsafe_preserve_version_counter(self.root_full):
                n_shard = u.shard_hi - u.shard_lo
                recv = torch.empty(dom.world * n_shard, dtype=self.param_dtype, device=self.device)
                dist.all_gather_into_tensor(recv, self.shard_lp[u.shard_lo:u.shard_hi], group=dom.group)
                rv = recv.view(dom.world, n_shard)
                for sl in u.slots:
                    o = sl.full_off - u.full_lo
                    self.root_full[o: o + sl.padded_numel * dom.world].view(dom.world, sl.padded_numel).copy_(
                        rv[:, sl.shard_off - u.shard_lo: sl.shard_off - u.shard_lo + sl.padded_numel])
                if stream is not None:
                    u.gather_event = torch.cuda.Event()
                    u.gather_event.record(stream)
            return
        if self.fused:
            if not self.lowp_fresh:  # no fused optimizer step wrote the parameters: push the shards
                from maester_b200.ops import cuda as C
                chunks, n = self.fused_chunk_table()
                self.symm_full.barrier()
                C.push_shards(self.master, self.symm_full, chunks, n)
            self.lowp_fresh = False
            self.symm_full.barrier()  # every rank's stores have landed before anyone's next forward
            return
        if not self.lowp_fresh:
            self.shard_lp.copy_(self.master) if self.world > 1 else self.full.copy_(self.master)
        self.lowp_fresh = False
        if self.world == 1:
            return
        stream = self.comm_stream
        if stream is not None:
            stream.wait_stream(torch.cuda.current_stream())
        # the root unit is needed first (embedding), then blocks in forward order
        order = [self.root] + self.units[:-1]
        ctx = torch.cuda.stream(stream) if stream is not None else _null()
        with ctx:
            for u in order:
                for dom, lo, hi, slots in self._segments(u):
                    if dom.world == 1:
                        for sl in slots:
                            self.full[sl.full_off: sl.full_off + sl.padded_numel].copy_(
                                self.shard_lp[sl.shard_off: sl.shard_off + sl.padded_numel])
                        continue
                    n_shard = hi - lo
                    recv = torch.empty(dom.world * n_shard, dtype=self.param_dtype, device=self.device)
                    dist.all_gather_into_tensor(recv, self.shard_lp[lo:hi], group=dom.group)
                    rv = recv.view(dom.world, n_shard)
                    for sl in slots:
                        dst = self.full[sl.full_off: sl.full_off + sl.padded_numel * dom.world]
                        dst.view(dom.world, sl.padded_numel).copy_(
                            rv[:, sl.shard_off - lo: sl.shard_off - lo + sl.padded_numel])
                if stream is not None:
                    u.gather_event = torch.cuda.Event()
                    u.gather_event.record(stream)

    # ------------------------------------------------------------------ fused (peer-memory) mode
    def fused_chunk_table(self, params=None, tensor_of=None):
        """Chunk records {shard offset, full offset of this rank's rows, length, tensor index} for the
        fused kernels, for all parameters or for the given master parameters."""
        import numpy as np

        recs = []
        wanted = None if params is None else {id(p) for p in params}
        for u in self.units:
            for sl in u.slots:
                if wanted is not None and id(sl.master) not in wanted:
                    continue
                ti = 0 if tensor_of is None else tensor_of[id(sl.master)]
                full0 = sl.full_off + self.rank * sl.padded_numel
                for c0 in range(0, sl.padded_numel, 32768):
                    recs.append((sl.shard_off + c0, full0 + c0, min(32768, sl.padded_numel - c0), ti))
        arr = np.zeros(len(recs), dtype=np.dtype([("s", "<i8"), ("f", "<i8"), ("len", "<i4"), ("t", "<i4")]))
        for i, r in enumerate(recs):
            arr[i] = r
        return torch.from_numpy(arr.view(np.uint8).copy()).to(self.device), len(recs)

    def _eager_update(self, u: Unit) -> None:
        """Reduce-scatter + optimizer update + all-gather of one unit as soon as its gradients are complete.
        The cross-rank barrier in front says that every rank has finished this unit's backward pass: its gradient
        buffers are final and nobody reads its parameters any more, so the kernel may overwrite them everywhere."""
        stream = self.comm_stream
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            self.symm_grad.barrier()
            for hook in self.eager_hooks:
                hook(u)
        u.eager_done = True

    def pre_optimizer_step(self) -> None:
        """Fused mode: all ranks' gradient buffers must be complete before any rank reduces them."""
        if self.fused:
            self.symm_grad.barrier()

    @torch.no_grad()
    def zero_grad(self) -> None:
        if self.grad_cleared_by_optimizer:   # the optimizer kernel cleared what it read; nothing has been written since
            self.grad_cleared_by_optimizer = False
            return
        # (None switches the optimizer's clearing off for good: tests compare the two ways)
        self.shard_grad.zero_()
        if self.resharded:
            return  # the staging buffers are cleared by the reduce-scatter that empties them
        if self.full_grad is not self.shard_grad:
            if self._use_cuda and self.world * self.rep_world > 1:
                # 4 B/parameter of zeros take milliseconds: written on a side stream under the forward pass, which
                # never touches the gradient buffer; the last block's forward pre-hook waits for the event, before
                # the loss layer or the backward pass can write a gradient
                if self._zero_stream is None:
                    self._zero_stream = torch.cuda.Stream(self.device)
                self._zero_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self._zero_stream):
                    self.full_grad.zero_()
                self._zero_event = torch.cuda.Event()
                self._zero_event.record(self._zero_stream)
            else:
                self.full_grad.zero_()

    _zero_stream = None
    _zero_event = None

    def _wait_zeroed(self) -> None:
        if self._zero_event is not None:
            torch.cuda.current_stream().wait_event(self._zero_event)
            self._zero_event = None

    # ------------------------------------------------------------------ state for checkpoints
    def master_state_dict(self) -> dict[str, torch.Tensor]:
        return {fqn: p.data for fqn, p in self.named_master_parameters()}


def gather_table(u: "Unit", world: int) -> list[tuple[int, int, int, int]]:
    """Copy plan of one block's parameter gather: ``(offset in the block's staging buffer, offset in the owner's row
    buffer, length, owner rank)`` per parameter and rank, in elements.  The staging buffer holds each parameter as
    ``world`` consecutive pieces of ``padded_numel`` elements (rank-major), which is the parameter's full dim-0 layout."""
    return [(sl.full_off - u.full_lo + r * sl.padded_numel, sl.shard_off, sl.padded_numel, r)
            for sl in u.slots for r in range(world)]


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
