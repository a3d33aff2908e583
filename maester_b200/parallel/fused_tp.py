"""Tensor-parallel linears whose reduce-scatter is fused into the GEMM over NVLink peer memory.

Megatron-style sequence parallelism needs, per transformer block and direction, two all-gathers and
two reduce-scatters of a ``[tokens, dim]`` activation (reference plan:
maester/parallelisms/parallelize_llama.py:107-181, executed there by DTensor + NCCL).  Every
reduce-scatter follows a GEMM: the row-parallel ``wo`` / ``w2`` in forward, the input-gradient GEMMs of
the column-parallel ``wq|wk|wv`` / ``w1|w3`` in backward.  ``FusedTP.gemm_rs`` runs that pair as ONE
kernel: the tcgen05 GEMM's epilogue stores each finished tile's rows directly into the symmetric
buffer of the rank that owns them (``mb_gemm_bf16_rs``), so the transfer of tile i overlaps the math
of tile i+1; the owner then sums the ``tp`` partial slices together with the residual it would add
anyway (``mb_sum_partials``).  Plain stores, no atomics: deterministic.  Every all-gather precedes a GEMM:
``FusedTP.ag_gemm`` runs that pair as one kernel too (``mb_gemm_bf16_ag``: some CTA pairs of the GEMM grid pull
the other ranks' row blocks with bulk copies while the rest multiply the local rows first).

``ag_linear`` / ``linear_rs`` are the two autograd ops built on it; with them a tensor-parallel block
runs the same code path as an unsharded one (the collectives live inside the first and last linear
of attention and FFN).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch.autograd import Function

from maester_b200.parallel.symm import SymmBuffer


class FusedTP:
    def __init__(self, tp, mode: str | None = None):
        import os
        self.tp = tp
        self.mode = mode or os.environ.get("MB_TP_RS_MODE", "pull")
        self.buf: SymmBuffer | None = None
        self.pair: list[SymmBuffer] = []
        self.calls = 0
        # all-gather -> GEMM: "fused" (copying CTA pairs inside the GEMM kernel) or "nccl"
        self.ag_mode = os.environ.get("MB_TP_AG_MODE", "fused")
        self.ag_copiers = int(os.environ.get("MB_TP_AG_COPIERS", "0"))  # CTA pairs that copy; 0: chosen per shape
        self.ag_pair: list[SymmBuffer] = []
        self.ag_flags: torch.Tensor | None = None
        self.ag_calls = 0

    def _ensure(self, numel: int, device: torch.device) -> SymmBuffer:
        if self.buf is None or self.buf.tensor.numel() < numel:
            assert self.buf is None, "activation size must not grow between calls (symmetric allocation is collective)"
            self.buf = SymmBuffer(numel, torch.bfloat16, device, self.tp.group)
        return self.buf

    def gemm_rs(self, a: torch.Tensor, b: torch.Tensor, *, b_mn: bool, residual: torch.Tensor | None = None) -> torch.Tensor:
        """rows [rank*M/tp, (rank+1)*M/tp) of ``sum over ranks (a @ op(b))`` (+ residual) as [M/tp, N].

        Two transports.  ``pull`` (default): the GEMM writes its full partial product into a local
        symmetric buffer and the owner of each row block reads the block from every rank with 512-byte
        coalesced loads while adding the residual; two buffers alternate, so one barrier per call.
        ``push``: the GEMM epilogue stores rows into their owners' buffers tile by tile."""
        from maester_b200.ops import cuda as C
        tp = self.tp
        M = a.shape[0]
        N = b.shape[1] if b_mn else b.shape[0]
        if self.mode == "pull":
            if not self.pair:
                self.pair = [SymmBuffer(M * N, torch.bfloat16, a.device, tp.group) for _ in range(2)]
            assert self.pair[0].tensor.numel() >= M * N
            buf = self.pair[self.calls & 1]
            self.calls += 1
            C.gemm(a, b, b_mn=b_mn, out=buf.tensor[:M * N].view(M, N))
            buf.barrier()  # every rank's partial product is complete (and its previous pull has finished)
            out = torch.empty(M // tp.size, N, device=a.device, dtype=a.dtype)
            C.pull_sum(buf, tp.rank, residual, out)
            return out
        buf = self._ensure(M * N, a.device)
        buf.barrier()  # every rank has consumed the previous partial sums
        C.gemm_rs(a, b, buf, tp.rank, b_mn=b_mn)
        buf.barrier()  # every rank's slices have landed
        out = torch.empty(M // tp.size, N, device=a.device, dtype=a.dtype)
        C.sum_partials(buf.tensor, residual, out, tp.size)
        return out


    def ag_gemm(self, x2: torch.Tensor, b: torch.Tensor, *, b_mn: bool, glu=None):
        """``(all_gather(x2), all_gather(x2) @ op(b).T)`` with the gather inside the GEMM kernel
        (``mb_gemm_bf16_ag``): every rank publishes its row block in a symmetric buffer; a few CTA pairs of the
        GEMM pull the other blocks over NVLink with bulk copies while the rest multiply the local rows, and a
        remote row tile is consumed as soon as its counter shows that it has landed.  Two buffers alternate,
        so one cross-rank barrier per call.  Falls back to NCCL + GEMM for shapes the kernel does not take.

        ``glu = (mode, act, gate_up)`` adds the gated-linear-unit epilogue (``ops.cuda.gemm_ag_glu``): the second
        value is then ``(gate_up, act(gate) * up)`` (mode 1) or ``d[gate | up]`` (mode 2)."""
        from maester_b200.ops import cuda as C
        tp = self.tp
        Ml, K = x2.shape
        M = Ml * tp.size
        if self.ag_mode != "fused" or Ml % 256 or K % 8 or not x2.is_contiguous():
            full = _all_gather_rows(x2, tp)
            if glu is None:
                return full, C.gemm(full, b, b_mn=b_mn)
            mode, act, gate_up = glu
            return full, (C.gemm_glu_fwd(full, b, act) if mode == 1 else C.gemm_glu_bwd(full, b, gate_up, act))
        if not self.ag_pair:
            self.ag_pair = [SymmBuffer(Ml * K, torch.bfloat16, x2.device, tp.group) for _ in range(2)]
            self.ag_flags = torch.zeros(max(M // 256, 1), dtype=torch.int32, device=x2.device)
        assert self.ag_pair[0].tensor.numel() >= Ml * K and self.ag_flags.numel() >= M // 256, \
            "activation size must not grow between calls (symmetric allocation is collective)"
        buf = self.ag_pair[self.ag_calls & 1]
        self.ag_calls += 1
        buf.tensor[:Ml * K].view(Ml, K).copy_(x2)
        full = torch.empty(M, K, device=x2.device, dtype=x2.dtype)
        full[tp.rank * Ml:(tp.rank + 1) * Ml].copy_(x2)
        buf.barrier()  # every rank's block is published (and its reads of the other buffer's last use are over)
        copiers = self.ag_copiers
        if copiers <= 0:
            # A copying CTA pair sustains about 64 GB/s over NVLink (its shared-memory ring bounds the bytes in
            # flight); the blocks have to arrive at the rate at which the computing pairs consume rows, which
            # for a fixed contraction depends on the output width only: pairs >= 27,000 / N (measured on B200:
            # N = 3072 is fastest with 8 pairs, N = 14336 with 2).
            N = b.shape[1] if b_mn else b.shape[0]
            copiers = 1
            while copiers < 8 and copiers * N < 27000:
                copiers *= 2
        if glu is not None:
            mode, act, gate_up = glu
            return full, C.gemm_ag_glu(full, buf, tp.rank, b, self.ag_flags, mode=mode, act=act, gate_up=gate_up,
                                       copiers=copiers)
        return full, C.gemm_ag(full, buf, tp.rank, b, self.ag_flags, b_mn=b_mn, copiers=copiers)


def _all_gather_rows(x2: torch.Tensor, tp) -> torch.Tensor:
    out = torch.empty(tp.size * x2.shape[0], x2.shape[1], device=x2.device, dtype=x2.dtype)
    dist.all_gather_into_tensor(out.view(-1), x2.contiguous().view(-1), group=tp.group)
    return out


def _wgrad(w, dy2, x2):
    from maester_b200.ops import cuda as C
    from maester_b200.ops.functional import _acc_or_return
    return _acc_or_return(w, lambda buf, acc: C.gemm(dy2, x2, a_mn=True, b_mn=True, out=buf,
                                                     epi=C.EPI_F32_ACC if acc else C.EPI_F32))


class _AGLinear(Function):
    """Column-parallel linear on a token-sharded input: ``all_gather(x) @ w.T``; the backward's input
    gradient is a GEMM fused with the reduce-scatter."""

    @staticmethod
    def forward(ctx, x, w, fused: FusedTP):
        from maester_b200.ops import cuda as C
        tp = fused.tp
        x_full, y = fused.ag_gemm(x.reshape(-1, x.shape[-1]).contiguous(), w, b_mn=False)
        ctx.save_for_backward(x_full, w)
        ctx.fused, ctx.x_shape = fused, x.shape
        return y.view(tp.batch, -1, w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x_full, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, w.shape[0])
        if dy2.stride(1) != 1:
            dy2 = dy2.contiguous()
        dx = ctx.fused.gemm_rs(dy2, w, b_mn=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        dw = _wgrad(w, dy2, x_full) if ctx.needs_input_grad[1] else None
        return dx, dw, None


class _LinearRS(Function):
    """Row-parallel linear: ``reduce_scatter(x @ w.T) (+ residual)`` as one GEMM with a routed epilogue."""

    @staticmethod
    def forward(ctx, x, w, residual, fused: FusedTP):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(1) != 1:
            x2 = x2.contiguous()
        ctx.save_for_backward(x2, w)
        ctx.fused, ctx.x_shape, ctx.has_res = fused, x.shape, residual is not None
        res2 = residual.reshape(-1, w.shape[0]).contiguous() if residual is not None else None
        out = fused.gemm_rs(x2, w, b_mn=False, residual=res2)
        return out.view(1, out.shape[0], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from maester_b200.ops import cuda as C
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, w.shape[0]).contiguous()
        if ctx.needs_input_grad[0]:
            dy_full, dx = ctx.fused.ag_gemm(dy2, w, b_mn=True)
            dx = dx.view(ctx.x_shape)
        else:
            dy_full, dx = _all_gather_rows(dy2, ctx.fused.tp), None
        dw = _wgrad(w, dy_full, x2) if ctx.needs_input_grad[1] else None
        return dx, dw, (dy if ctx.has_res else None), None


class _AGGluRS(Function):
    """Tensor-parallel gated MLP on a token-sharded input as ONE autograd node:
    ``reduce_scatter(act(all_gather(x) w_gate^T) * (all_gather(x) w_up^T)) w_down^T) (+ residual)``.
    The gather runs inside the gate|up GEMM whose epilogue also forms the activation; backward gathers dy inside the
    down-projection's input-gradient GEMM whose epilogue applies the activation's derivative; the two remaining
    collectives are GEMM + reduce-scatter kernels.  No stand-alone element-wise pass, no NCCL call."""

    @staticmethod
    def forward(ctx, x, w_gu, w_down, residual, fused: FusedTP, act: int):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        x_full, (gate_up, a) = fused.ag_gemm(x2, w_gu, b_mn=False, glu=(1, act, None))
        res2 = residual.reshape(-1, w_down.shape[0]).contiguous() if residual is not None else None
        out = fused.gemm_rs(a, w_down, b_mn=False, residual=res2)
        ctx.save_for_backward(x_full, w_gu, w_down, gate_up, a)
        ctx.fused, ctx.act, ctx.x_shape, ctx.has_res = fused, act, x.shape, residual is not None
        return out.view(1, out.shape[0], w_down.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x_full, w_gu, w_down, gate_up, a = ctx.saved_tensors
        fused = ctx.fused
        dy2 = dy.reshape(-1, w_down.shape[0]).contiguous()
        dy_full, d_gu = fused.ag_gemm(dy2, w_down, b_mn=True, glu=(2, ctx.act, gate_up))
        dw_down = _wgrad(w_down, dy_full, a) if ctx.needs_input_grad[2] else None
        dx = fused.gemm_rs(d_gu, w_gu, b_mn=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        dw_gu = _wgrad(w_gu, d_gu, x_full) if ctx.needs_input_grad[1] else None
        return dx, dw_gu, dw_down, (dy if ctx.has_res else None), None, None


def glu_mlp_tp(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, activation: str,
               residual: torch.Tensor | None, fused: FusedTP) -> torch.Tensor:
    """Gated MLP of a tensor-parallel block (``w_gate_up``: this rank's ``[gate rows | up rows]``, ``w_down``: this
    rank's columns) on the token-sharded residual stream; returns this rank's token rows of the summed result."""
    from maester_b200.ops.functional import _ACT
    return _AGGluRS.apply(x, w_gate_up, w_down, residual, fused, _ACT[activation])


def ag_linear(x: torch.Tensor, w: torch.Tensor, fused: FusedTP) -> torch.Tensor:
    return _AGLinear.apply(x, w, fused)


def linear_rs(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None, fused: FusedTP) -> torch.Tensor:
    return _LinearRS.apply(x, w, residual, fused)


def fused_tp_available(tp, device: torch.device) -> bool:
    from maester_b200.parallel.symm import symmetric_memory_available
    return device.type == "cuda" and tp.size <= 8 and symmetric_memory_available(tp.group)
