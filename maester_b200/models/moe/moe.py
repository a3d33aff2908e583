"""Token-choice mixture-of-experts block shared by DeepSeek and GLM-4.5.

Reference: maester/models/moe/moe.py.  Semantics kept: fp32 router (gate GEMM with fp32
accumulation, sigmoid or softmax in fp32), selection by ``scores + expert_bias`` while the gate
values come from the unbiased scores (:286-334), optional renormalisation and ``route_scale``,
stable expert-major ordering of the (token, k) slots (:378-398), scores applied before or after the
experts in fp32 (:497-522), shared experts as one dense SwiGLU of width ``hidden * num_shared``,
routed outputs scatter-added onto the shared output, persistent ``expert_bias`` and
non-persistent ``tokens_per_expert`` buffers (:433-448).  Expert weights are stored
``w1, w3: [E, dim, hidden]`` and ``w2: [E, hidden, dim]`` as in the reference, so checkpoints match.

Execution: slots are permuted into an expert-major buffer whose groups are padded to 128 rows;
group offsets stay on the device and feed the grouped tcgen05 GEMM directly, so there is no
device-to-host synchronisation on the routing result (the reference's for-loop path and its EP
dispatch both synchronise).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Literal

import torch
import torch.nn as nn
import torch.nn.functional as F

from maester_b200 import ops
from maester_b200.models.layers import FusedWeight, Linear
from maester_b200.ops.functional import GROUP_ALIGN, grouped_swiglu, padded_group_offsets

# routing, permutation and combine as native kernels (csrc/moe_route.cu); "0" keeps the ATen chain
FUSED_ROUTING = os.environ.get("MB_MOE_FUSED_ROUTE", "1") != "0"


@dataclass
class MoEArgs:
    num_experts: int = 8
    num_shared_experts: int = 1
    score_func: Literal["softmax", "sigmoid"] = "sigmoid"
    route_norm: bool = False
    route_scale: float = 1.0
    score_before_experts: bool = True
    top_k: int = 1
    use_grouped_mm: bool = True
    load_balance_coeff: float | None = 1e-3
    _debug_force_load_balance: bool = False
    aux_loss_coeff: float = 0.0  # optional auxiliary load-balance loss (absent from the reference)


class FeedForward(nn.Module):
    """Dense SwiGLU ``w2(silu(w1 x) * w3 x)``."""

    fused_param_order = ("w1", "w3", "w2")

    def __init__(self, dim: int, hidden_dim: int):
        super().__init__()
        self.w1 = Linear(dim, hidden_dim)
        self.w2 = Linear(hidden_dim, dim)
        self.w3 = Linear(dim, hidden_dim)
        self._w13 = FusedWeight([self.w1, self.w3])

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        return self.w2(ops.glu(ops.linear(x, self._w13.get()), "silu"), residual=residual)

    def init_weights(self, init_std: float = 0.02) -> None:
        nn.init.trunc_normal_(self.w1.weight, mean=0.0, std=0.02)
        for lin in (self.w2, self.w3):
            nn.init.trunc_normal_(lin.weight, mean=0.0, std=init_std)


class GroupedExperts(nn.Module):
    def __init__(self, dim: int, hidden_dim: int, num_experts: int, use_grouped_mm: bool = True):
        super().__init__()
        self.num_experts, self.use_grouped_mm = num_experts, use_grouped_mm
        # expert parallelism replaces the parameters by this rank's E/ep experts and sets these
        self.num_local_experts, self.ep_rank, self.ep_size = num_experts, 0, 1
        self.w1 = nn.Parameter(torch.empty(num_experts, dim, hidden_dim))
        self.w2 = nn.Parameter(torch.empty(num_experts, hidden_dim, dim))
        self.w3 = nn.Parameter(torch.empty(num_experts, dim, hidden_dim))

    def forward(self, x: torch.Tensor, offs: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """x: expert-major rows [rows_cap, dim] with zero padding rows; offs: padded int32 offsets; out: optional
        preallocated result buffer (used when it can be written directly)."""
        return grouped_swiglu(x, self.w1, self.w3, self.w2, offs, out)

    def init_weights(self, init_std: float) -> None:
        gen = None
        if self.ep_size > 1:  # every expert-parallel rank draws different experts
            gen = torch.Generator(device=self.w1.device)
            base = int(torch.randint(0, 2**31 - 1, (1,)).item())  # global RNG: same on all ranks, new per layer
            gen.manual_seed(base + 7919 * (self.ep_rank + 1))
        nn.init.trunc_normal_(self.w1, mean=0.0, std=0.02, generator=gen)
        nn.init.trunc_normal_(self.w2, mean=0.0, std=init_std, generator=gen)
        nn.init.trunc_normal_(self.w3, mean=0.0, std=init_std, generator=gen)


class TokenChoiceTopKRouter(nn.Module):
    def __init__(self, dim: int, num_experts: int, top_k: int, score_func: str, route_norm: bool,
                 route_scale: float, _debug_force_load_balance: bool = False):
        super().__init__()
        self.gate = Linear(dim, num_experts)
        self.num_experts, self.top_k = num_experts, top_k
        self.score_func, self.route_norm, self.route_scale = score_func, route_norm, route_scale
        self._debug_force_load_balance = _debug_force_load_balance

    def forward(self, x: torch.Tensor, expert_bias: torch.Tensor | None = None):
        """x: [T, dim] → (top_scores [T,k] fp32, expert indices [T,k], tokens per expert [E] fp32, scores [T,E])."""
        w = self.gate.weight
        if ops.use_native(x, w) and x.shape[1] % 8 == 0:
            from maester_b200.ops import cuda as C
            logits = _RouterGemm.apply(x, w)
        else:
            logits = F.linear(x.float(), w.float())
        if self.score_func == "sigmoid":
            scores = torch.sigmoid(logits)
        elif self.score_func == "softmax":
            scores = F.softmax(logits, dim=1)
        else:
            raise NotImplementedError(f"Unknown score function {self.score_func}")
        if self._debug_force_load_balance:
            n = scores.shape[0]
            idx = torch.arange(n * self.top_k, device=scores.device).reshape(n, self.top_k) % self.num_experts
            top = scores.gather(1, idx)
        elif expert_bias is not None:
            _, idx = torch.topk(scores + expert_bias, k=self.top_k, dim=1, sorted=False)
            top = scores.gather(1, idx)  # the bias steers selection only
        else:
            top, idx = torch.topk(scores, k=self.top_k, dim=1, sorted=False)
        if self.route_norm:
            top = top / (top.sum(dim=-1, keepdim=True) + 1e-20)
        top = top * self.route_scale
        counts = torch.zeros(self.num_experts, device=x.device, dtype=torch.float32)
        counts.scatter_add_(0, idx.reshape(-1), torch.ones(idx.numel(), device=x.device, dtype=torch.float32))
        return top, idx, counts, scores

    def init_weights(self, init_std: float) -> None:
        nn.init.trunc_normal_(self.gate.weight, mean=0.0, std=init_std)


class _RouterGemm(torch.autograd.Function):
    """fp32-accumulated, fp32-output gate GEMM on the native kernel (bf16 x bf16 products are exact)."""

    @staticmethod
    def forward(ctx, x, w):
        from maester_b200.ops import cuda as C
        ctx.save_for_backward(x, w)
        return C.gemm(x, w, epi=C.EPI_F32)

    @staticmethod
    def backward(ctx, dlogits):
        from maester_b200.ops import cuda as C
        x, w = ctx.saved_tensors
        d = dlogits.to(torch.bfloat16).contiguous()
        if d.shape[1] % 8:
            dx = (dlogits @ w.float()).to(x.dtype)
            dw32 = dlogits.t() @ x.float()
        else:
            dx = C.gemm(d, w, b_mn=True)
            dw32 = C.gemm(d, x, a_mn=True, b_mn=True, epi=C.EPI_F32)
        mg = getattr(w, "main_grad", None)
        if mg is not None:
            mg.add_(dw32)
            return dx, None
        return dx, dw32.to(w.dtype)


class _SlotGather(torch.autograd.Function):
    """rows[p] = x[token of sorted slot p].  Every token owns exactly ``k`` slots, so the backward is a
    gather back to slot order and a sum over k: no scatter-add, no atomics, deterministic."""

    @staticmethod
    def forward(ctx, x, token_idx, inv, k):
        ctx.save_for_backward(inv)
        ctx.k = k
        return x.index_select(0, token_idx)

    @staticmethod
    def backward(ctx, g):
        (inv,) = ctx.saved_tensors
        dim = g.shape[1]
        gx = g.index_select(0, inv).view(-1, ctx.k, dim).sum(dim=1, dtype=torch.float32).to(g.dtype)
        return gx, None, None, None


class _UniqueRowSelect(torch.autograd.Function):
    """rows = buf[idx] for DISTINCT row indices: the backward is a plain row copy into zeros."""

    @staticmethod
    def forward(ctx, buf, idx):
        ctx.save_for_backward(idx)
        ctx.rows = buf.shape[0]
        return buf.index_select(0, idx)

    @staticmethod
    def backward(ctx, g):
        (idx,) = ctx.saved_tensors
        return g.new_zeros(ctx.rows, g.shape[1]).index_copy_(0, idx, g), None


class _SlotCombine(torch.autograd.Function):
    """out[t] = sum over the k slots of token t of rows[sorted position of that slot]."""

    @staticmethod
    def forward(ctx, rows, token_idx, inv, k):
        ctx.save_for_backward(token_idx)
        dim = rows.shape[1]
        return rows.index_select(0, inv).view(-1, k, dim).sum(dim=1, dtype=torch.float32).to(rows.dtype)

    @staticmethod
    def backward(ctx, g):
        (token_idx,) = ctx.saved_tensors
        return g.index_select(0, token_idx), None, None, None


class _FusedRoute(torch.autograd.Function):
    """Scores, top-k and the whole routing plan in three launches (``csrc/moe_route.cu``).  Returns the gate
    values [T, k] and the scores [T, E] (both differentiable); the plan object is appended to ``holder``."""

    @staticmethod
    def forward(ctx, logits, bias, k, softmax, norm, scale, force_balance, holder):
        from maester_b200.ops import cuda as C
        plan = C.moe_route(logits.contiguous(), bias, k, softmax, norm, scale, force_balance, GROUP_ALIGN)
        holder.append(plan)
        ctx.save_for_backward(plan.scores, plan.idx)
        ctx.cfg = (softmax, norm, scale)
        ctx.set_materialize_grads(False)
        return plan.top, plan.scores

    @staticmethod
    def backward(ctx, d_top, d_scores):
        from maester_b200.ops import cuda as C
        scores, idx = ctx.saved_tensors
        softmax, norm, scale = ctx.cfg
        if d_top is None:
            d_top = torch.zeros(idx.shape, device=scores.device, dtype=torch.float32)
        return C.moe_route_bwd(d_top, d_scores, scores, idx, softmax, norm, scale), None, None, None, None, None, None, None


class _RowsGather(torch.autograd.Function):
    """Token rows -> tile-padded expert-major buffer (zeros in the padding), optionally times the gate value."""

    @staticmethod
    def forward(ctx, x, gate, row_slot, slot_row, k):
        from maester_b200.ops import cuda as C
        ctx.k = k
        ctx.save_for_backward(x if gate is not None else None, gate, row_slot, slot_row)
        return C.moe_rows_gather(x, row_slot, gate, k)

    @staticmethod
    def backward(ctx, g):
        from maester_b200.ops import cuda as C
        x, gate, row_slot, slot_row = ctx.saved_tensors
        g = g.contiguous()
        dx = C.moe_rows_combine(g, slot_row, gate, ctx.k)
        dgate = C.moe_slot_dot(g, slot_row, x, ctx.k).view_as(gate) if gate is not None else None
        return dx, dgate, None, None, None


class _RowsCombine(torch.autograd.Function):
    """Expert-major buffer -> one row per token: the sum of its k rows, optionally weighted by the gate values."""

    @staticmethod
    def forward(ctx, buf, gate, row_slot, slot_row, k):
        from maester_b200.ops import cuda as C
        ctx.k = k
        ctx.save_for_backward(buf if gate is not None else None, gate, row_slot, slot_row)
        return C.moe_rows_combine(buf, slot_row, gate, k)

    @staticmethod
    def backward(ctx, g):
        from maester_b200.ops import cuda as C
        buf, gate, row_slot, slot_row = ctx.saved_tensors
        g = g.contiguous()
        dbuf = C.moe_rows_gather(g, row_slot, gate, ctx.k)
        dgate = C.moe_slot_dot(buf, slot_row, g, ctx.k).view_as(gate) if gate is not None else None
        return dbuf, dgate, None, None, None


class TokenReorderer(nn.Module):
    """Stable expert-major ordering of the T*k routing slots."""

    def __init__(self, num_experts: int, top_k: int):
        super().__init__()
        self.num_experts, self.top_k = num_experts, top_k

    def forward(self, top_scores: torch.Tensor, selected: torch.Tensor):
        flat = selected.reshape(-1)
        order = torch.argsort(flat, stable=True)
        self.last_order = order  # sorted position p holds original slot order[p] = token * top_k + j
        counts = torch.zeros(self.num_experts, device=flat.device, dtype=torch.int64)
        counts.scatter_add_(0, flat, torch.ones_like(flat, dtype=torch.int64))
        return top_scores.reshape(-1)[order], order // self.top_k, counts, flat[order]


class MoE(nn.Module):
    def __init__(self, moe_args: MoEArgs, dim: int, hidden_dim: int):
        super().__init__()
        E = moe_args.num_experts
        self.experts = GroupedExperts(dim, hidden_dim, E, moe_args.use_grouped_mm)
        self.router = TokenChoiceTopKRouter(dim, E, moe_args.top_k, moe_args.score_func, moe_args.route_norm,
                                            moe_args.route_scale, moe_args._debug_force_load_balance)
        self.reorderer = TokenReorderer(E, moe_args.top_k)
        self.shared_experts = (FeedForward(dim, hidden_dim * moe_args.num_shared_experts)
                               if moe_args.num_shared_experts > 0 else None)
        self.score_before_experts = moe_args.score_before_experts
        self.load_balance_coeff = moe_args.load_balance_coeff
        self.aux_loss_coeff = moe_args.aux_loss_coeff
        self.top_k = moe_args.top_k
        if self.load_balance_coeff is not None:
            assert self.load_balance_coeff > 0.0
            self.register_buffer("expert_bias", torch.zeros(E, dtype=torch.float32), persistent=True)
        else:
            self.expert_bias = None
        self.register_buffer("tokens_per_expert", torch.zeros(E, dtype=torch.float32), persistent=False)
        self.aux_loss: torch.Tensor | None = None
        self.dispatcher = None  # set by expert parallelism: callable doing dispatch + experts + combine
        self.tp_group = None    # set by expert tensor parallelism

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        bs, slen, dim = x.shape
        x = x.reshape(-1, dim)
        T = x.shape[0]
        if self.tp_group is not None:  # hidden dimension sharded over tp: partial outputs, summed below
            from maester_b200.parallel.expert_parallel import _CopyToTP
            x = _CopyToTP.apply(x, self.tp_group)
        if (FUSED_ROUTING and ops.use_native(x, self.router.gate.weight) and dim % 8 == 0
                and self.router.num_experts <= 256 and self.top_k <= 8):
            out = self._forward_fused(x.contiguous())
            if self.tp_group is not None:
                from maester_b200.parallel.expert_parallel import _ReduceFromTP
                out = _ReduceFromTP.apply(out, self.tp_group)
            return out.reshape(bs, slen, dim)
        top, idx, counts_f, scores = self.router(x, self.expert_bias)
        with torch.no_grad():
            self.tokens_per_expert.add_(counts_f)
        if self.aux_loss_coeff > 0 and self.training:
            # Switch-style balance loss: E * sum_e (fraction of slots on e) * (mean router prob of e)
            frac = counts_f / counts_f.sum().clamp_min(1.0)
            self.aux_loss = self.aux_loss_coeff * scores.shape[1] * (frac * scores.mean(dim=0)).sum()
        sorted_scores, token_idx, counts, sorted_experts = self.reorderer(top, idx)
        order = self.reorderer.last_order
        self._inv = torch.empty_like(order).scatter_(0, order, torch.arange(order.numel(), device=order.device))

        if self.dispatcher is not None:
            routed_out = self.dispatcher(self, x, sorted_scores, token_idx, counts, sorted_experts)
        else:
            # expert-major buffer with every group padded to the GEMM tile height
            offs = padded_group_offsets(counts)
            starts = counts.cumsum(0) - counts
            slot = torch.arange(token_idx.numel(), device=x.device)
            dest = offs[:-1].to(torch.int64)[sorted_experts] + (slot - starts[sorted_experts])
            rows_cap = (T * self.top_k + self.router.num_experts * (GROUP_ALIGN - 1) + GROUP_ALIGN - 1) \
                // GROUP_ALIGN * GROUP_ALIGN
            routed_in = self.gather_slots(x, token_idx)
            if self.score_before_experts:
                routed_in = (routed_in.float() * sorted_scores[:, None]).to(x.dtype)
            buf = torch.zeros(rows_cap, dim, device=x.device, dtype=x.dtype).index_copy(0, dest, routed_in)
            routed_out = _UniqueRowSelect.apply(self.experts(buf, offs), dest)
            if not self.score_before_experts:
                routed_out = (routed_out.float() * sorted_scores[:, None]).to(x.dtype)

        out = _SlotCombine.apply(routed_out, token_idx, self._inv, self.top_k)
        if self.shared_experts is not None:
            out = self.shared_experts(x, residual=out)
        if self.tp_group is not None:
            from maester_b200.parallel.expert_parallel import _ReduceFromTP
            out = _ReduceFromTP.apply(out, self.tp_group)
        return out.reshape(bs, slen, dim)

    def _forward_fused(self, x: torch.Tensor) -> torch.Tensor:
        """Same block with the routing chain, the permutation and the weighted combine as native kernels."""
        r, k = self.router, self.top_k
        logits = _RouterGemm.apply(x, r.gate.weight)
        holder: list = []
        top, scores = _FusedRoute.apply(logits, self.expert_bias, k, r.score_func == "softmax", r.route_norm,
                                        float(r.route_scale), r._debug_force_load_balance, holder)
        plan = holder[0]
        with torch.no_grad():
            self.tokens_per_expert.add_(plan.counts_f)
        if self.aux_loss_coeff > 0 and self.training:
            frac = plan.counts_f / float(plan.T * k)
            self.aux_loss = self.aux_loss_coeff * r.num_experts * (frac * scores.mean(dim=0)).sum()
        if self.dispatcher is not None and hasattr(self.dispatcher, "fused"):
            out = self.dispatcher.fused(self, x, plan, top)  # rows move between ranks straight from token order
        elif self.dispatcher is not None:
            L = plan.as_long()
            self.reorderer.last_order, self._inv = L["order"], L["inv"]
            sorted_scores = top.reshape(-1).index_select(0, L["order"])
            routed_out = self.dispatcher(self, x, sorted_scores, L["token_idx"], L["counts"], L["sorted_experts"])
            out = _SlotCombine.apply(routed_out, L["token_idx"], self._inv, k)
        else:
            before = self.score_before_experts
            buf = _RowsGather.apply(x, top if before else None, plan.row_slot, plan.slot_row, k)
            out = _RowsCombine.apply(self.experts(buf, plan.offs), None if before else top, plan.row_slot,
                                     plan.slot_row, k)
        if self.shared_experts is not None:
            out = self.shared_experts(x, residual=out)
        return out

    def gather_slots(self, x: torch.Tensor, token_idx: torch.Tensor) -> torch.Tensor:
        """Rows of ``x`` in sorted-slot order (used by this block and by the expert-parallel dispatchers)."""
        return _SlotGather.apply(x, token_idx, self._inv, self.top_k)

    def init_weights(self, init_std: float, buffer_device: torch.device | None = None) -> None:
        self.experts.init_weights(init_std)
        self.router.init_weights(init_std)
        if self.shared_experts is not None:
            self.shared_experts.init_weights(init_std)
        dev = buffer_device or self.experts.w1.device
        if dev.type != "meta":
            self.tokens_per_expert = torch.zeros(self.experts.num_experts, dtype=torch.float32, device=dev)
            if self.load_balance_coeff is not None:
                self.expert_bias = torch.zeros(self.experts.num_experts, dtype=torch.float32, device=dev)
