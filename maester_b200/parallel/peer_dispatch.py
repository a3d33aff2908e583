"""Expert-parallel dispatch / combine over NVLink peer memory, without host synchronisation.

Same contract as ``AllToAllDispatcher`` (expert_parallel.py).  What changes is who moves the rows:

1. the per-expert slot counts of all ranks are all-gathered (a few hundred bytes; stays on the device);
2. from that matrix every rank computes, with device tensor ops, where each of its slots lives on the
   destination rank: ``dest_rank = expert // E_local`` and ``dest_row = start of the expert's
   128-padded group on that rank + slots of lower ranks for that expert + position in my group``;
3. ``peer_scatter_rows`` writes the rows into the destination ranks' symmetric buffers, the local
   experts run their grouped GEMMs on the buffer with device-side group offsets, and
   ``peer_gather_rows`` pulls every slot's result back (csrc/ep_comm.cu).

With the native routing plan (``ops.cuda.RoutePlan``) the block takes the token-indexed form of the same
exchange (``PeerDispatcher.fused``): ``mb_ep_plan`` computes every slot's (rank, row) in one kernel,
``peer_dispatch_rows`` writes each token's row (times its gate value) straight from token order into the owners'
buffers, ``peer_combine_rows`` sums a token's k expert rows read from their owners, ``peer_slot_dot`` yields the
gate gradients, only the padding rows of the expert groups are cleared, and the last expert GEMM writes into the
peer-visible buffer itself: no ``[T*k, dim]`` tensor in sorted order, no full-buffer memset, no staging copy.

Backward is the mirror image (gradients of the results are scattered, gradients of the inputs are
gathered).  Cross-rank ordering is by stream-ordered barriers on the symmetric buffers' signal pads.
Buffers hold ``capacity_factor x`` the balanced load; rows beyond that are dropped and counted in
``overflow`` (read it with ``dropped()``; it costs a synchronisation, so only do so when logging).  The largest
row count any call wanted is tracked on the device; ``adapt_capacity()`` (called by the trainer where it reads the
drop counter) grows the buffers to 1.5 x that peak once a rank comes within 80 % of its capacity, so a drifting
router load is answered before it overflows; only a jump past the capacity within one logging interval drops rows.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from maester_b200.ops.functional import GROUP_ALIGN
from maester_b200.parallel.symm import SymmBuffer


class _Plan:
    """Device-side routing plan of one MoE call."""
    __slots__ = ("dest_rank", "dest_row", "offs", "n", "dim", "slot_rank", "slot_row", "T", "k", "allc", "n_local")

    def zero_padding(self, disp, buf) -> None:
        """Clear the padding rows of the local experts' groups in ``buf`` (the rows in front are overwritten by the
        dispatch, the rows behind the last group are never read), instead of the whole twice-oversized buffer."""
        from maester_b200.ops import cuda as C
        C.ep_zero_padding(buf.tensor, self.allc, disp.ep.rank, self.n_local, self.offs, self.dim, disp.cap)


class _Scatter(torch.autograd.Function):
    """rows [n, dim] -> this rank's expert-major buffer [cap, dim] filled by all ranks."""

    @staticmethod
    def forward(ctx, rows, disp, plan, buf):
        from maester_b200.ops import cuda as C
        ctx.disp, ctx.plan = disp, plan
        buf.tensor.zero_()
        disp.barrier()                       # every rank's buffer is cleared
        C.peer_scatter_rows(rows.contiguous(), buf, plan.dest_rank, plan.dest_row, disp.cap, disp.overflow)
        disp.barrier()                       # every rank's rows have landed
        return buf.tensor.view(disp.cap, plan.dim)

    @staticmethod
    def backward(ctx, grad_buf):
        from maester_b200.ops import cuda as C
        disp, plan = ctx.disp, ctx.plan
        ws = disp.workspace(1, plan.dim)
        ws.tensor.view(disp.cap, plan.dim).copy_(grad_buf)
        disp.barrier()
        grad_rows = torch.empty(plan.n, plan.dim, device=grad_buf.device, dtype=grad_buf.dtype)
        C.peer_gather_rows(grad_rows, ws, plan.dest_rank, plan.dest_row, disp.cap, disp.overflow)
        disp.barrier()                       # peers are done reading before the workspace is reused
        return grad_rows, None, None, None


class _Gather(torch.autograd.Function):
    """expert outputs [cap, dim] on every rank -> rows [n, dim] of this rank's slots."""

    @staticmethod
    def forward(ctx, out_buf, disp, plan):
        from maester_b200.ops import cuda as C
        ctx.disp, ctx.plan = disp, plan
        ws = disp.workspace(0, plan.dim)
        ws.tensor.view(disp.cap, plan.dim).copy_(out_buf)
        disp.barrier()
        rows = torch.empty(plan.n, plan.dim, device=out_buf.device, dtype=out_buf.dtype)
        C.peer_gather_rows(rows, ws, plan.dest_rank, plan.dest_row, disp.cap, disp.overflow)
        disp.barrier()
        return rows

    @staticmethod
    def backward(ctx, grad_rows):
        from maester_b200.ops import cuda as C
        disp, plan = ctx.disp, ctx.plan
        ws = disp.workspace(0, plan.dim)
        ws.tensor.zero_()                    # padding rows must carry finite (zero) gradients
        disp.barrier()
        C.peer_scatter_rows(grad_rows.contiguous(), ws, plan.dest_rank, plan.dest_row, disp.cap, disp.overflow)
        disp.barrier()
        # the result is consumed by the experts' backward before any other MoE call touches the workspace
        return ws.tensor.view(disp.cap, plan.dim).clone(), None, None


class _TokenScatter(torch.autograd.Function):
    """Token rows [T, dim] (times their gate values) -> this rank's expert-major buffer, written by every rank
    straight from its token rows: no [T*k, dim] tensor in sorted-slot order in between.  The backward is the
    weighted combine of the buffer gradients plus, for the gate values, a dot product per slot."""

    @staticmethod
    def forward(ctx, x, gate, disp, plan, buf):
        from maester_b200.ops import cuda as C
        ctx.disp, ctx.plan = disp, plan
        ctx.save_for_backward(x if gate is not None else None, gate)
        plan.zero_padding(disp, buf)
        disp.barrier()
        C.peer_dispatch_rows(x, buf, plan.slot_rank, plan.slot_row, gate, plan.k, disp.cap, disp.overflow)
        disp.barrier()
        return buf.tensor.view(disp.cap, plan.dim)

    @staticmethod
    def backward(ctx, grad_buf):
        from maester_b200.ops import cuda as C
        disp, plan = ctx.disp, ctx.plan
        x, gate = ctx.saved_tensors
        ws = disp.workspace(1, plan.dim)
        ws.tensor.view(disp.cap, plan.dim).copy_(grad_buf)
        disp.barrier()
        dx = C.peer_combine_rows(ws, plan.slot_rank, plan.slot_row, gate, plan.T, plan.k, plan.dim, disp.cap, disp.overflow)
        dgate = None
        if gate is not None:
            dgate = C.peer_slot_dot(ws, plan.slot_rank, plan.slot_row, x, plan.k, disp.cap).view_as(gate)
        disp.barrier()                       # peers are done reading before the workspace is reused
        return dx, dgate, None, None, None


class _TokenCombine(torch.autograd.Function):
    """Expert outputs [cap, dim] on every rank -> out[t] = sum of the k rows of token t (times their gate values
    when the block applies them after the experts), read from the rows' owners.  With gate values the outputs
    stay in a per-block symmetric buffer until the backward pass, which needs them for the gate gradients."""

    @staticmethod
    def forward(ctx, out_buf, gate, disp, plan, ws):
        from maester_b200.ops import cuda as C
        ctx.disp, ctx.plan, ctx.ws = disp, plan, ws
        ctx.save_for_backward(gate)
        if out_buf.data_ptr() != ws.tensor.data_ptr():  # not already written in place by the last expert GEMM
            ws.tensor.view(disp.cap, plan.dim).copy_(out_buf)
        disp.barrier()
        out = C.peer_combine_rows(ws, plan.slot_rank, plan.slot_row, gate, plan.T, plan.k, plan.dim, disp.cap, disp.overflow)
        disp.barrier()
        return out

    @staticmethod
    def backward(ctx, g):
        from maester_b200.ops import cuda as C
        disp, plan = ctx.disp, ctx.plan
        (gate,) = ctx.saved_tensors
        g = g.contiguous()
        dgate = None
        if gate is not None:  # the owners' output buffers of this block are untouched since its forward pass
            dgate = C.peer_slot_dot(ctx.ws, plan.slot_rank, plan.slot_row, g, plan.k, disp.cap).view_as(gate)
        ws = disp.workspace(0, plan.dim)
        plan.zero_padding(disp, ws)          # padding rows must carry finite (zero) gradients
        disp.barrier()
        C.peer_dispatch_rows(g, ws, plan.slot_rank, plan.slot_row, gate, plan.k, disp.cap, disp.overflow)
        disp.barrier()
        return ws.tensor.view(disp.cap, plan.dim).clone(), dgate, None, None, None


class PeerDispatcher:
    def __init__(self, ep, capacity_factor: float = 2.0):
        self.ep = ep
        self.capacity_factor = capacity_factor
        self.cap = 0
        self.peak_need: torch.Tensor | None = None   # largest row count any call wanted on this rank (device scalar)
        self._ws: dict[int, SymmBuffer] = {}
        self._inputs: dict[int, SymmBuffer] = {}   # per MoE block: its input buffer is saved for backward
        self._outputs: dict[int, SymmBuffer] = {}  # per MoE block with gates after the experts: outputs kept likewise
        self.overflow: torch.Tensor | None = None

    # ------------------------------------------------------------------ buffers
    def _ensure(self, n_slots: int, n_local: int, dim: int, device: torch.device) -> None:
        if self.cap:   # sized at the first call (and possibly grown by adapt_capacity since)
            assert n_slots <= self._shape[0], "the number of routing slots per rank must not grow between steps"
            return
        cap = int(self.capacity_factor * n_slots) + n_local * GROUP_ALIGN
        cap = (cap + GROUP_ALIGN - 1) // GROUP_ALIGN * GROUP_ALIGN
        if cap > self.cap:
            self.cap = cap
            self._shape = (n_slots, n_local, dim)
            self.overflow = torch.zeros(1, dtype=torch.int32, device=device)
            self.peak_need = torch.zeros((), dtype=torch.int64, device=device)
            # symmetric allocations are collective: make them here, where all ranks are in step
            for which in (0, 1):
                self._ws[which] = SymmBuffer(self.cap * dim, torch.bfloat16, device, self.ep.group)

    def workspace(self, which: int, dim: int) -> SymmBuffer:
        return self._ws[which]

    def input_buffer(self, moe, dim: int) -> SymmBuffer:
        key = id(moe)
        if key not in self._inputs:
            self._inputs[key] = SymmBuffer(self.cap * dim, torch.bfloat16, self.overflow.device, self.ep.group)
        return self._inputs[key]

    def output_buffer(self, moe, dim: int) -> SymmBuffer:
        key = id(moe)
        if key not in self._outputs:
            self._outputs[key] = SymmBuffer(self.cap * dim, torch.bfloat16, self.overflow.device, self.ep.group)
        return self._outputs[key]

    def barrier(self) -> None:
        self.workspace(0, 0).barrier()

    def _note_need(self, allc: torch.Tensor, n_local: int) -> None:
        """Track (on the device) how many buffer rows this rank's experts wanted: the groups' 128-padded sizes."""
        lo = self.ep.rank * n_local
        tot = allc[:, lo: lo + n_local].sum(0, dtype=torch.int64)
        need = ((tot + GROUP_ALIGN - 1) // GROUP_ALIGN * GROUP_ALIGN).sum()
        torch.maximum(self.peak_need, need, out=self.peak_need)

    def adapt_capacity(self, headroom: float = 0.8) -> bool:
        """Grow the buffers when the fullest rank came within ``headroom`` of its capacity (or overflowed) since the
        last call.  Collective over the expert-parallel group and synchronising: call it between steps, where the
        trainer reads the drop counter anyway.  Returns True if the buffers were reallocated (1.5 x the peak)."""
        if self.peak_need is None:
            return False
        peak = self.peak_need.clone()
        dist.all_reduce(peak, op=dist.ReduceOp.MAX, group=self.ep.group)
        peak_rows = int(peak.item())
        self.peak_need.zero_()
        if peak_rows <= headroom * self.cap:
            return False
        n_slots, n_local, dim = self._shape
        new_cap = (int(1.5 * peak_rows) + GROUP_ALIGN - 1) // GROUP_ALIGN * GROUP_ALIGN
        if new_cap <= self.cap:
            return False
        from maester_b200.log_utils import logger
        logger.warning(f"expert-parallel peer dispatch: a rank wanted {peak_rows} of {self.cap} buffer rows; "
                       f"growing the symmetric buffers to {new_cap} rows")
        device = self.overflow.device
        self.cap = new_cap
        self._inputs.clear()
        self._outputs.clear()
        self._ws.clear()
        torch.cuda.synchronize(device)
        for which in (0, 1):
            self._ws[which] = SymmBuffer(self.cap * dim, torch.bfloat16, device, self.ep.group)
        return True

    def dropped(self) -> int:
        """Rows dropped over capacity since the last reset (synchronises with the device: call when logging)."""
        return int(self.overflow.item()) if self.overflow is not None else 0

    def reset_dropped(self) -> None:
        if self.overflow is not None:
            self.overflow.zero_()

    # ------------------------------------------------------------------ routing plan (device only)
    def plan(self, counts: torch.Tensor, sorted_experts: torch.Tensor, n_local: int, dim: int) -> _Plan:
        ep = self.ep
        E = counts.numel()
        allc = torch.empty(ep.size, E, dtype=counts.dtype, device=counts.device)
        dist.all_gather_into_tensor(allc.view(-1), counts.contiguous(), group=ep.group)
        self._note_need(allc, n_local)
        tot = allc.sum(0)                                              # rows per expert over all ranks
        padded = (tot + GROUP_ALIGN - 1) // GROUP_ALIGN * GROUP_ALIGN
        pv = padded.view(ep.size, n_local)
        group_start = (pv.cumsum(1) - pv).reshape(-1)                  # start of each expert's group on its rank
        before_me = allc[:ep.rank].sum(0)                              # slots of lower ranks, per expert
        my_start = counts.cumsum(0) - counts                           # start of my group per expert in my slot order
        slot = torch.arange(sorted_experts.numel(), device=counts.device)
        p = _Plan()
        p.dest_rank = (sorted_experts // n_local).to(torch.int32)
        p.dest_row = (group_start[sorted_experts] + before_me[sorted_experts] + (slot - my_start[sorted_experts])).to(torch.int32)
        mine = pv[ep.rank]
        offs = torch.zeros(n_local + 1, dtype=torch.int64, device=counts.device)
        offs[1:] = mine.cumsum(0)
        p.offs = offs.clamp_max(self.cap).to(torch.int32)
        p.n, p.dim = sorted_experts.numel(), dim
        return p

    # ------------------------------------------------------------------ token-indexed path (native routing plan)
    def fused(self, moe, x: torch.Tensor, route, gate: torch.Tensor) -> torch.Tensor:
        """Dispatch, experts and combine with the gate values applied where the block wants them.  ``route`` is
        the native routing plan of this rank's tokens (``ops.cuda.RoutePlan``), ``gate`` its [T, k] gate values.
        One tiny all-gather of the per-expert counts, one plan kernel, then rows move between the ranks' buffers
        directly from / to token order."""
        from maester_b200.ops import cuda as C
        ep = self.ep
        n_local = moe.experts.num_local_experts
        dim = x.shape[1]
        self._ensure(route.T * route.k, n_local, dim, x.device)
        allc = torch.empty(ep.size, route.E, dtype=torch.int32, device=x.device)
        dist.all_gather_into_tensor(allc.view(-1), route.counts, group=ep.group)
        self._note_need(allc, n_local)
        p = _Plan()
        p.slot_rank, p.slot_row, p.offs = C.ep_plan(allc, ep.rank, n_local, route.idx.view(-1), route.inv, GROUP_ALIGN,
                                                    self.cap)
        p.T, p.k, p.dim = route.T, route.k, dim
        p.allc, p.n_local = allc, n_local
        before = moe.score_before_experts
        buf = _TokenScatter.apply(x, gate if before else None, self, p, self.input_buffer(moe, dim))
        out_ws = self.workspace(0, dim) if before else self.output_buffer(moe, dim)
        # the last expert GEMM writes straight into the peer-visible buffer the combine reads from
        y = moe.experts(buf, p.offs, out=out_ws.tensor[:self.cap * dim].view(self.cap, dim))
        return _TokenCombine.apply(y, None if before else gate, self, p, out_ws)

    # ------------------------------------------------------------------ dispatcher contract
    def __call__(self, moe, x, sorted_scores, token_idx, counts, sorted_experts):
        n_local = moe.experts.num_local_experts
        dim = x.shape[1]
        self._ensure(token_idx.numel(), n_local, dim, x.device)
        routed_in = moe.gather_slots(x, token_idx)
        if moe.score_before_experts:
            routed_in = (routed_in.float() * sorted_scores[:, None]).to(x.dtype)
        plan = self.plan(counts, sorted_experts, n_local, dim)
        buf = _Scatter.apply(routed_in, self, plan, self.input_buffer(moe, dim))
        out = moe.experts(buf, plan.offs)
        routed_out = _Gather.apply(out, self, plan)
        if not moe.score_before_experts:
            routed_out = (routed_out.float() * sorted_scores[:, None]).to(x.dtype)
        return routed_out
