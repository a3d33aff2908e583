"""Muon: momentum + Newton–Schulz orthogonalised updates for matrices, Adam for the rest.

Reference: maester/optimizers/muon.py.  Semantics kept: momentum buffer ``m`` per matrix, EMA
``m ← lerp(m, g, 1-μ)`` followed by the Nesterov blend ``u ← lerp(g, m, μ)`` (:153-179); five
quintic Newton–Schulz iterations in bf16 with coefficients (3.4445, −4.7750, 2.0315) after Frobenius
normalisation, on the wide orientation of the matrix (:22-49); update
``p ← p·(1 − lr·wd) − lr·sqrt(max(1, rows/cols))·NS(u)`` (:228-232); parameters whose group has
``use_muon=False`` get a built-in Adam (:184-208).

Distribution: parameters are dim-0 shards of the flat-buffer sharding runtime.  Matrix ``i`` is owned
by rank ``i % world``: the shards of ``u`` are gathered there, orthogonalised once and scattered
back, with up to ``prefetch_factor`` matrices in flight (reference :210-264).  On CUDA with a usable peer-memory
plane the exchange does not go through the process group at all: every rank stages its row chunks of all matrices in
one symmetric buffer, the owners pull them with the library's copy kernel, and the results are pulled back the same
way, two cross-rank barriers per step (``_step_over_peer_memory``).  ``MuonDDP`` is the
replicated-parameter variant: every rank holds full matrices, work is split round-robin and the
results are exchanged with one all-gather per bucket (reference :297-460).

The Newton–Schulz iteration runs on the tcgen05 GEMM: ``A = X Xᵀ``, ``B = c·A·A + b·A`` and
``X ← B·X + a·X`` are three launches per iteration, the axpby terms live in the GEMM epilogue.
"""
from __future__ import annotations

import math
from collections import deque

import torch
import torch.distributed as dist
from torch.optim import Optimizer

from maester_b200.ops import reference as ref

NS_COEFFS = (3.4445, -4.7750, 2.0315)


def syrk(a: torch.Tensor, c: torch.Tensor | None = None, alpha: float = 1.0, beta: float = 0.0) -> torch.Tensor:
    """``alpha·A·Aᵀ + beta·C`` (reference kernel: maester/optimizers/muon_/syrk.py:143-169).

    For bf16 CUDA inputs this is the CTA-pair GEMM with a triangular tile schedule: only the 256x256 tiles on and
    below the diagonal are computed and the epilogue also stores each of them transposed, as the reference kernel
    does with its lower-triangular blocks.
    """
    if a.is_cuda and a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.is_contiguous():
        from maester_b200.ops import cuda as C
        return C.syrk(a, c if (c is not None and beta != 0.0) else None, alpha, beta)
    out = alpha * (a @ a.mT)
    return out + beta * c if (c is not None and beta != 0.0) else out


def newton_schulz(g: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """Approximate ``U Vᵀ`` of ``g = U S Vᵀ`` (bf16)."""
    if not (g.is_cuda and g.dim() == 2 and g.shape[0] % 8 == 0 and g.shape[1] % 8 == 0):
        return ref.newton_schulz(g, steps, eps)
    from maester_b200.ops import cuda as C
    a, b, c = NS_COEFFS
    x = g.to(torch.bfloat16)
    transposed = x.shape[0] > x.shape[1]
    if transposed:
        x = x.t().contiguous()
    x = (x / (x.norm() + eps)).contiguous()
    for _ in range(steps):
        A = C.syrk(x)                                                      # X Xᵀ            [m, m], lower tiles + mirror
        Bm = C.syrk(A, A, alpha=c, beta=b)                                 # c·A·Aᵀ + b·A    (A symmetric: A·A = A·Aᵀ)
        x = C.gemm(Bm, x, b_mn=True, epi=C.EPI_BF16_ADD, aux=x, alpha=1.0, beta=a)  # B·X + a·X
    return x.t().contiguous() if transposed else x


def _adam_update(p, g, state, group) -> None:
    if "exp_avg" not in state:
        state["step"] = 0
        state["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
        state["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
    state["step"] += 1
    b1, b2 = group.get("adam_betas", group.get("betas", (0.9, 0.95)))
    ref.adamw_step(p.data, g.float(), state["exp_avg"], state["exp_avg_sq"], state["step"], group["lr"], b1, b2,
                   group.get("adam_eps", group.get("eps", 1e-8)), group.get("wd", group.get("weight_decay", 0.0)))


class Muon(Optimizer):
    """Muon over (possibly dim-0 sharded) 2-D parameters.

    ``shard_group`` / ``full_shape_of`` describe the sharding: ``full_shape_of(p)`` returns the
    unsharded shape of ``p``.  When they are omitted the parameters are treated as full matrices.
    """

    def __init__(self, params, lr: float = 0.02, momentum: float = 0.95, ns_steps: int = 5, wd: float = 0.01,
                 nesterov: bool = True, use_muon: bool = True, prefetch_factor: int = 8, shard_group=None,
                 full_shape_of=None, **adam_kw):
        # group keys as in the reference's optimizer (lr, momentum, ns_steps, wd, use_muon): they are what a checkpoint
        # stores per group, so both sides can load each other's; ``nesterov`` is a property of the optimizer
        defaults = dict(lr=lr, momentum=momentum, ns_steps=ns_steps, wd=wd, use_muon=use_muon, **adam_kw)
        super().__init__(params, defaults)
        self.nesterov = nesterov
        self.prefetch_factor = prefetch_factor
        self.shard_group = shard_group
        self.full_shape_of = full_shape_of
        self._init_state()

    def _init_state(self) -> None:
        """Every buffer exists from the start, as in the reference ("init buffers ahead of time",
        maester/optimizers/muon.py:129-150): a checkpoint is loaded into the state dict of a freshly built optimizer, and
        what is not there yet would silently not be restored."""
        for group in self.param_groups:
            for p in group["params"]:
                st = self.state[p]
                if group["use_muon"] and p.dim() >= 2:
                    if "m" not in st:
                        st["m"] = torch.zeros(p.shape[0], math.prod(p.shape[1:]), dtype=torch.float32, device=p.device)
                    st["param_shape"] = tuple(self.full_shape_of(p)) if self.full_shape_of else tuple(p.shape)
                elif "exp_avg" not in st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)

    def attach_sharding(self, sharded) -> None:
        """Use the sharding runtime's group and shapes (called by the optimizer builder)."""
        self.shard_group = sharded.group if sharded.world > 1 else None
        self.full_shape_of = lambda p: sharded.slot_of(p).shape
        # expert-parallel parameters are sharded over their own (smaller) group
        self.group_of = lambda p: (lambda d: d.group if d.world > 1 else None)(sharded.domains[sharded.slot_of(p).dom])
        self._init_state()   # the unsharded shapes are known now

    group_of = None

    def _world(self, p=None) -> tuple[object, int, int]:
        g = self.group_of(p) if (self.group_of is not None and p is not None) else self.shard_group
        if g is None or not dist.is_initialized():
            return None, 1, 0
        return g, dist.get_world_size(g), dist.get_rank(g)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        work = []  # (param, group, update-direction shard u)
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not group["use_muon"] or p.dim() < 2:
                    _adam_update(p, p.grad, st, group)
                    continue
                g = p.grad.reshape(p.shape[0], -1).float()
                if "m" not in st:
                    st["m"] = torch.zeros_like(g)
                if "param_shape" not in st:   # the unsharded shape, kept beside the momentum as the reference does
                    st["param_shape"] = tuple(self.full_shape_of(p)) if self.full_shape_of else tuple(p.shape)
                m = st["m"]
                m.lerp_(g, 1 - group["momentum"])
                u = g.lerp(m, group["momentum"]) if self.nesterov else m
                work.append((p, group, u.to(torch.bfloat16)))

        if work and self._peer_exchange_ok(work):
            self._step_over_peer_memory(work)
            return loss

        inflight: deque = deque()

        def launch(i: int):
            p, group, u = work[i]
            pg, world, rank = self._world(p)
            owner = i % world
            if world == 1:
                return (i, None, None, u)
            full_rows = self.full_shape_of(p)[0] if self.full_shape_of else u.shape[0] * world
            chunk = (full_rows + world - 1) // world
            padded = u if u.shape[0] == chunk else torch.cat([u, u.new_zeros(chunk - u.shape[0], u.shape[1])])
            gather_list = [torch.empty_like(padded) for _ in range(world)] if rank == owner else None
            h = dist.gather(padded, gather_list, group_dst=owner, group=pg, async_op=True)
            return (i, h, gather_list, padded)

        def finish(item):
            i, h, gather_list, padded = item
            p, group, u = work[i]
            pg, world, rank = self._world(p)
            owner = i % world
            if world == 1:
                o = newton_schulz(u, group["ns_steps"])
            else:
                h.wait()
                full_rows = self.full_shape_of(p)[0] if self.full_shape_of else u.shape[0] * world
                scatter_list = None
                if rank == owner:
                    full = torch.cat(gather_list)[:full_rows]
                    of = newton_schulz(full, group["ns_steps"])
                    chunk = padded.shape[0]
                    if of.shape[0] < chunk * world:
                        of = torch.cat([of, of.new_zeros(chunk * world - of.shape[0], of.shape[1])])
                    scatter_list = list(of.split(chunk))
                o = torch.empty_like(padded)
                dist.scatter(o, scatter_list, group_src=owner, group=pg)
                o = o[: u.shape[0]]
            shape = self.full_shape_of(p) if self.full_shape_of else p.shape
            rows, cols = shape[0], math.prod(shape[1:])
            scale = max(1.0, rows / cols) ** 0.5
            p.data.mul_(1 - group["lr"] * group["wd"])
            p.data.add_(o.reshape(p.shape).to(p.dtype), alpha=-group["lr"] * scale)

        for i in range(len(work)):
            inflight.append(launch(i))
            if len(inflight) >= self.prefetch_factor:
                finish(inflight.popleft())
        while inflight:
            finish(inflight.popleft())
        return loss


    # ------------------------------------------------------------------ gather / scatter over peer memory
    peer_exchange = True   # class-wide switch (tests compare against the process-group path)

    def _chunk_rows(self, p, world: int) -> int:
        full_rows = self.full_shape_of(p)[0]
        return (full_rows + world - 1) // world

    def _peer_exchange_ok(self, work) -> bool:
        """All matrices are sharded over one NCCL group whose peer-memory plane passed its start-up check, and every
        row chunk is a multiple of 16 bytes (the copy kernel moves 16-byte words)."""
        if not (self.peer_exchange and self.full_shape_of is not None and work[0][2].is_cuda):
            return False
        pg, world, _ = self._world(work[0][0])
        if world == 1:
            return False
        for p, _, u in work:
            g, w, _ = self._world(p)
            if g is not pg or (self._chunk_rows(p, world) * u.shape[1]) % 8:
                return False
        from maester_b200.parallel.symm import symmetric_memory_available
        return symmetric_memory_available(pg)

    def _step_over_peer_memory(self, work) -> None:
        """Every rank stages its row chunks of all update matrices in one symmetric buffer; after ONE cross-rank
        barrier the owner of a matrix (round robin) pulls the other ranks' chunks through their mapped pointers,
        orthogonalises, and leaves the result in its own symmetric buffer; after a SECOND barrier every rank pulls
        its rows of every result from the owner.  Two barriers and plain peer loads replace a gather and a scatter
        collective per matrix (the reference batches point-to-point sends instead:
        maester/optimizers/muon_/muon.py gather / scatter of shards)."""
        from maester_b200.ops import cuda as C
        from maester_b200.parallel.symm import SymmBuffer
        pg, world, rank = self._world(work[0][0])
        dev = work[0][2].device
        chunks = [self._chunk_rows(p, world) for p, _, _ in work]
        cols = [u.shape[1] for _, _, u in work]
        sizes, in_off, out_off, fill = peer_exchange_layout(chunks, cols, world)
        key = (id(pg), in_off[-1], max(fill))
        if getattr(self, "_peer_key", None) != key:                       # collective allocation, first step only
            self._peer_in = SymmBuffer(max(in_off[-1], 8), torch.bfloat16, dev, pg)
            self._peer_out = SymmBuffer(max(max(fill), 8), torch.bfloat16, dev, pg)
            self._peer_key = key
        stage, res = self._peer_in, self._peer_out
        for i, (p, _, u) in enumerate(work):
            dst = stage.tensor[in_off[i]: in_off[i] + sizes[i]].view(chunks[i], cols[i])
            dst[: u.shape[0]].copy_(u)
            if u.shape[0] < chunks[i]:
                dst[u.shape[0]:].zero_()
        stage.barrier()                                                   # every rank's chunks are staged
        for i, (p, group, u) in enumerate(work):
            if i % world != rank:
                continue
            full = torch.empty(world * chunks[i], cols[i], device=dev, dtype=torch.bfloat16)
            for r in range(world):
                C.peer_copy(full[r * chunks[i]:(r + 1) * chunks[i]], stage.peer_ptrs[r] + in_off[i] * 2, sizes[i] * 2)
            rows = self.full_shape_of(p)[0]
            o = res.tensor[out_off[i]: out_off[i] + sizes[i] * world].view(world * chunks[i], cols[i])
            o[:rows].copy_(newton_schulz(full[:rows], group["ns_steps"]))
        res.barrier()                                                     # every owner's results are in place
        for i, (p, group, u) in enumerate(work):
            mine = torch.empty(chunks[i], cols[i], device=dev, dtype=torch.bfloat16)
            C.peer_copy(mine, res.peer_ptrs[i % world] + (out_off[i] + rank * sizes[i]) * 2, sizes[i] * 2)
            shape = self.full_shape_of(p)
            scale = max(1.0, shape[0] / math.prod(shape[1:])) ** 0.5
            p.data.mul_(1 - group["lr"] * group["wd"])
            p.data.add_(mine[: u.shape[0]].reshape(p.shape).to(p.dtype), alpha=-group["lr"] * scale)
        # the next step's staging writes come after its own barrier-free copies; a rank may only overwrite its
        # buffers once every peer has finished pulling from them
        res.barrier()


def peer_exchange_layout(chunks: list[int], cols: list[int], world: int):
    """Buffer layout of the peer-memory exchange, identical on every rank.

    ``sizes[i]``: elements of one rank's row chunk of matrix i.  ``in_off``: where a rank stages its chunk of matrix i
    in its own staging buffer (``in_off[-1]`` = buffer size).  ``out_off[i]``: where the owner of matrix i
    (rank ``i % world``) leaves the orthogonalised matrix, ``world`` chunks back to back, in ITS result buffer;
    ``fill[r]`` = elements rank r's result buffer needs."""
    sizes = [c * n for c, n in zip(chunks, cols)]
    in_off = [0]
    for sz in sizes:
        in_off.append(in_off[-1] + sz)
    out_off, fill = [], [0] * world
    for i, sz in enumerate(sizes):
        out_off.append(fill[i % world])
        fill[i % world] += sz * world
    return sizes, in_off, out_off, fill


class MuonDDP(Optimizer):
    """Muon for replicated parameters: matrices are split round-robin over ranks, each rank
    orthogonalises its share and one all-gather per size bucket returns everybody's results."""

    def __init__(self, params, lr: float = 0.02, momentum: float = 0.95, ns_steps: int = 5, wd: float = 0.01,
                 nesterov: bool = True, group=None):
        super().__init__(params, dict(lr=lr, momentum=momentum, ns_steps=ns_steps, wd=wd, nesterov=nesterov))
        self.group = group

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        distributed = dist.is_initialized() and dist.get_world_size(self.group) > 1
        world = dist.get_world_size(self.group) if distributed else 1
        rank = dist.get_rank(self.group) if distributed else 0
        for group in self.param_groups:
            buckets: dict[tuple, list] = {}
            for p in group["params"]:
                if p.grad is not None:
                    buckets.setdefault(tuple(p.shape), []).append(p)
            for shape, plist in buckets.items():
                # pad the bucket so every rank handles the same number of matrices
                n = (len(plist) + world - 1) // world * world
                mine = []
                for j in range(rank, n, world):
                    if j < len(plist):
                        p = plist[j]
                        g = p.grad.reshape(p.shape[0], -1).float()
                        st = self.state[p]
                        if "m" not in st:
                            st["m"] = torch.zeros_like(g)
                        st["m"].lerp_(g, 1 - group["momentum"])
                        u = g.lerp(st["m"], group["momentum"]) if group["nesterov"] else st["m"]
                        mine.append(newton_schulz(u.to(torch.bfloat16), group["ns_steps"]).reshape(-1))
                    else:
                        mine.append(torch.zeros(math.prod(shape), device=plist[0].device, dtype=torch.bfloat16))
                local = torch.stack(mine)  # [n/world, numel]
                if distributed:
                    out = torch.empty(world, *local.shape, device=local.device, dtype=local.dtype)
                    dist.all_gather_into_tensor(out.view(-1, local.shape[1]), local, group=self.group)
                else:
                    out = local[None]
                rows, cols = shape[0], math.prod(shape[1:])
                scale = max(1.0, rows / cols) ** 0.5
                for j, p in enumerate(plist):
                    o = out[j % world, j // world].reshape(p.shape)
                    p.data.mul_(1 - group["lr"] * group["wd"])
                    p.data.add_(o.to(p.dtype), alpha=-group["lr"] * scale)
        return loss
