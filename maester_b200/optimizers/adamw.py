"""Fused AdamW over flat fp32 buffers: one kernel launch updates every parameter of a shard.

``FusedAdamW`` is a regular ``torch.optim.Optimizer`` (so LR schedulers, state_dict and the
optimizer container work unchanged).  When its parameters are views into one flat fp32 buffer whose
gradients are views into a matching flat buffer (the layout the sharding runtime creates), the whole
update is a single native launch that also emits the bf16 copy consumed by the next forward.
Otherwise it falls back to a per-tensor update with the same arithmetic.
Reference behaviour: torch.optim.AdamW(fused=True) as configured in maester/config.py:147-154.
"""
from __future__ import annotations

import torch
from torch.optim import Optimizer

from maester_b200.ops import reference as ref

CHUNK = 32768


def build_chunk_table(segments, device):
    """segments: iterable of (offset, numel, lr_mult, weight_decay) → (chunks, tensors, nchunks).

    ``chunks`` is an int8 view of packed {int64 offset, int32 len, int32 tensor} records and
    ``tensors`` an fp32 [n, 2] table of (lr_mult, weight_decay).
    """
    import numpy as np

    recs = []
    tens = []
    for ti, (off, n, lrm, wd) in enumerate(segments):
        tens.append((lrm, wd))
        for c0 in range(0, n, CHUNK):
            recs.append((off + c0, min(CHUNK, n - c0), ti))
    arr = np.zeros(len(recs), dtype=np.dtype([("offset", "<i8"), ("len", "<i4"), ("tensor", "<i4")]))
    for i, r in enumerate(recs):
        arr[i] = r
    chunks = torch.from_numpy(arr.view(np.uint8).copy()).to(device)
    tensors = torch.tensor(tens, dtype=torch.float32, device=device).reshape(-1, 2).contiguous()
    return chunks, tensors, len(recs)


class FusedAdamW(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, fused=None, **_):
        # the remaining entries are the ones ``torch.optim.AdamW`` keeps in its groups: a checkpoint written here then
        # has every key that the reference's optimizer asks for when it loads one (and they state what this class does)
        defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay, amsgrad=False, maximize=False,
                        foreach=None, capturable=False, differentiable=False, fused=True, decoupled_weight_decay=True)
        super().__init__(params, defaults)
        self._flat = None  # set by attach_flat()
        self.cleared_grad = False  # the last step() cleared the gradients it consumed
        self._eager = None  # set by eager_begin() for the duration of one step
        self._unit_tables: dict = {}

    def attach_flat(self, master: torch.Tensor, grad: torch.Tensor, lowp: torch.Tensor | None, segments_by_param,
                    m: torch.Tensor | None = None, v: torch.Tensor | None = None):
        """Register the flat layout: ``segments_by_param`` maps each parameter to (offset, numel).

        master / grad are fp32 flat buffers of equal length, lowp the bf16 buffer that receives the
        updated values (may be None).  State tensors exp_avg / exp_avg_sq become views of two more
        flat buffers so that checkpoints keep the per-parameter layout.
        """
        self._flat = dict(master=master, grad=grad, lowp=lowp, seg=segments_by_param,
                          m=m if m is not None else torch.zeros_like(master),
                          v=v if v is not None else torch.zeros_like(master), table=None)
        for group in self.param_groups:
            for p in group["params"]:
                off, n = segments_by_param[p]
                st = self.state[p]
                st["step"] = torch.tensor(0.0)
                st["exp_avg"] = self._flat["m"][off:off + n].view(p.shape)
                st["exp_avg_sq"] = self._flat["v"][off:off + n].view(p.shape)

    def _table(self):
        f = self._flat
        base_lr = self.param_groups[0]["lr"] or 1.0
        # the chunk table holds lr RATIOS, so a schedule that scales every group alike never rebuilds it; the
        # base learning rate lives in a one-element device tensor refreshed when it changes
        key = tuple((round(g["lr"] / base_lr, 9), g["weight_decay"]) for g in self.param_groups)
        if f["table"] is None or f["table"][0] != key:
            segs = []
            for g in self.param_groups:
                for p in g["params"]:
                    off, n = f["seg"][p]
                    segs.append((off, n, g["lr"] / base_lr, g["weight_decay"]))
            dev = f["master"].device
            f["table"] = (key, build_chunk_table(segs, dev), torch.tensor([base_lr], device=dev, dtype=torch.float32))
            f["table_lr"] = base_lr
        if f.get("table_lr") != base_lr:
            f["table"][2].fill_(base_lr)
            f["table_lr"] = base_lr
        return f["table"][1], f["table"][2]

    # ---- per-unit updates under the backward pass (peer-memory sharding runtime) -------------------------------
    def eager_begin(self) -> bool:
        """Announce the coming step before the backward pass that produces its gradients: fixes the step number,
        learning rate and per-tensor table, and registers ``_eager_unit`` with the sharding runtime, which calls it
        for every unit as soon as the unit's gradients are complete on all ranks."""
        f = self._flat
        sharded = f.get("sharded") if f is not None else None
        if sharded is None or not sharded.fused or not f["master"].is_cuda:
            return False
        st = self.state[self.param_groups[0]["params"][0]]
        (_, tensors, _), lr_t = self._table()
        self._eager = dict(step=int(st["step"].item()) + 1, tensors=tensors, lr_t=lr_t, done=set())
        if self._eager_unit not in sharded.eager_hooks:
            sharded.eager_hooks.append(self._eager_unit)
        return True

    @torch.no_grad()
    def _eager_unit(self, u) -> None:
        e, f = self._eager, self._flat
        if e is None or id(u) in e["done"]:
            return
        from maester_b200.ops import cuda as C
        sharded = f["sharded"]
        tab = self._unit_tables.get(id(u))
        if tab is None:  # chunk records of this optimizer's parameters inside the unit (geometry only: cached)
            order = [p for g in self.param_groups for p in g["params"]]
            tensor_of = {id(p): i for i, p in enumerate(order)}
            mine = [sl.master for sl in u.slots if id(sl.master) in tensor_of]
            tab = sharded.fused_chunk_table(mine, tensor_of) if mine else (None, 0)
            self._unit_tables[id(u)] = tab
        fchunks, fn = tab
        if fn:
            g0 = self.param_groups[0]
            b1, b2 = g0["betas"]
            C.fused_rs_adamw_ag(sharded.symm_grad, sharded.symm_full, f["master"], f["m"], f["v"], f["grad"], fchunks,
                                e["tensors"], fn, e["lr_t"], b1, b2, g0["eps"], e["step"], sharded.divide)
        e["done"].add(id(u))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        f = self._flat
        if f is not None and f["master"].is_cuda:
            from maester_b200.ops import cuda as C
            g0 = self.param_groups[0]
            any_p = g0["params"][0]
            st = self.state[any_p]
            st_step = int(st["step"].item()) + 1 if torch.is_tensor(st["step"]) else int(st["step"]) + 1
            (chunks, tensors, nch), lr_t = self._table()
            b1, b2 = g0["betas"]
            sharded = f.get("sharded")
            if sharded is not None and sharded.fused and self._eager is not None:
                # the units were updated one by one under the backward pass; run the ones whose hook did not fire
                st_step = self._eager["step"]
                for u in sharded.units:
                    if id(u) not in self._eager["done"]:
                        self._eager_unit(u)
                self._eager = None
            elif sharded is not None and sharded.fused:
                # reduce-scatter + update + all-gather in one kernel over the peers' buffers
                if f.get("fused_table") is None or f["fused_table"][0] is not chunks:
                    order = [p for g in self.param_groups for p in g["params"]]
                    tensor_of = {id(p): i for i, p in enumerate(order)}
                    f["fused_table"] = (chunks, sharded.fused_chunk_table(order, tensor_of))
                fchunks, fn = f["fused_table"][1]
                C.fused_rs_adamw_ag(sharded.symm_grad, sharded.symm_full, f["master"], f["m"], f["v"], f["grad"],
                                    fchunks, tensors, fn, lr_t, b1, b2, g0["eps"], st_step, sharded.divide)
            else:
                # the kernel emits the bf16 copy itself; any other compute dtype (fp32 oracle runs) is a plain copy
                lp = f["lowp"] if (f["lowp"] is not None and f["lowp"].dtype == torch.bfloat16) else None
                # one rank: the kernel reads the accumulation buffer itself, so it clears what it has read and the
                # next step needs no separate pass over the 4 B/parameter buffer
                clear = bool(sharded is not None and getattr(sharded, "grad_cleared_by_optimizer", None) is not None
                             and sharded.full_grad is sharded.shard_grad and f["grad"] is sharded.shard_grad)
                C.adamw(f["master"], f["grad"], f["m"], f["v"], lp, chunks, tensors, nch, lr_t, b1, b2,
                        g0["eps"], st_step, zero_grad=clear)
                self.cleared_grad = clear
                if lp is None and f["lowp"] is not None:
                    f["lowp"].copy_(f["master"])
            for g in self.param_groups:
                for p in g["params"]:
                    self.state[p]["step"] = torch.tensor(float(st_step))
            return loss
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "exp_avg" not in st:
                    st["step"] = torch.tensor(0.0)
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                st["step"] = st["step"] + 1
                p32 = p.data if p.dtype == torch.float32 else p.data.float()
                ref.adamw_step(p32, p.grad.float(), st["exp_avg"], st["exp_avg_sq"], int(st["step"].item()),
                               group["lr"], b1, b2, group["eps"], group["weight_decay"])
                if p32 is not p.data:
                    p.data.copy_(p32)
        if f is not None and f["lowp"] is not None:
            f["lowp"].copy_(f["master"])
        return loss
