"""Thin tensor-level wrappers over the native launchers (no autograd here).

Every wrapper checks layouts, passes raw pointers plus the current CUDA stream, and raises on a
non-zero return code.  ``check_status()`` reads the host-mapped status word that kernels set when a
bounded wait expires.
"""
from __future__ import annotations

import ctypes
import math
import os

import torch

from maester_b200.ops import _lib

EPI_BF16, EPI_F32, EPI_F32_ACC, EPI_BF16_ADD = 0, 1, 2, 3

_STATUS_NAMES = {
    1: "consumer timed out waiting for a TMA stage",
    2: "producer timed out waiting for a free stage",
    3: "epilogue timed out waiting for the accumulator",
    4: "MMA warp timed out waiting for a drained accumulator",
    5: "timed out waiting on a peer GPU's flag",
    6: "softmax warps timed out",
    7: "pipeline wait timed out",
    8: "bad argument detected on device",
    9: "a loss whose gradients were produced during forward received a different output gradient in backward",
    10: "checked build: a store outside its tensor was skipped",
}

launch_count = 0  # number of native kernel launches issued through this module
GEMM_TWO_CTA = os.environ.get("MB_GEMM_2CTA", "1") != "0"
# grouped weight gradients (contraction over an expert's rows) on the CTA-pair kernel
GROUPED_CONTR_TWO_CTA = os.environ.get("MB_GROUPED_CONTR_2CTA", "1") != "0"


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _ck(rc: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if rc != 0:
        raise RuntimeError(f"maester_b200 native call {what} failed with code {rc}")


def check_status(sync: bool = True) -> None:
    """Raise if any kernel recorded a bounded-wait expiry since the last clear."""
    if sync:
        torch.cuda.synchronize()
    l = _lib.lib()
    s = l.mb_status()
    if s != 0:
        l.mb_status_clear()
        raise RuntimeError(f"maester_b200 kernel reported status {s}: {_STATUS_NAMES.get(s, 'unknown')}")


def _rows_pitch(t: torch.Tensor) -> int:
    assert t.dim() == 2 and t.stride(1) == 1, f"expected a row-major 2-D tensor, got strides {t.stride()}"
    return t.stride(0)


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: torch.Tensor | None = None, epi: int = EPI_BF16, alpha: float = 1.0,
         aux: torch.Tensor | None = None, alpha_dev: torch.Tensor | None = None,
         two_cta: bool | None = None, beta: float = 1.0) -> torch.Tensor:
    """``C = alpha * op(A) @ op(B).T`` on the tcgen05 GEMM.

    ``two_cta`` selects the CTA-pair kernel (256x256 tiles, ``cta_group::2``); by default it is used
    whenever the problem has more than one 128-row tile.

    a_mn=False: A is [M, K];  a_mn=True: A is stored [K, M].
    b_mn=False: B is [N, K];  b_mn=True: B is stored [K, N].
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    if out is None:
        out = torch.empty(M, N, device=a.device, dtype=torch.bfloat16 if epi in (EPI_BF16, EPI_BF16_ADD) else torch.float32)
    assert out.shape == (M, N)
    l = _lib.lib()
    if two_cta is None:
        two_cta = GEMM_TWO_CTA and M > 128
    fn = l.mb_gemm_bf16_2cta if two_cta else l.mb_gemm_bf16
    rc = fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), _ptr(aux), M, N, K,
            _rows_pitch(a), _rows_pitch(b), _rows_pitch(out), _rows_pitch(aux) if aux is not None else 0,
            int(a_mn), int(b_mn), epi, float(alpha), float(beta), _ptr(alpha_dev), _stream())
    _ck(rc, "gemm_bf16")
    return out


def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor | None, eps: float, unit_offset: bool,
                residual: torch.Tensor | None = None):
    D = x.shape[-1]
    x2 = x.reshape(-1, D)
    assert x2.is_contiguous()
    M = x2.shape[0]
    y = torch.empty_like(x2)
    rstd = torch.empty(M, device=x.device, dtype=torch.float32)
    r2 = residual.reshape(-1, D) if residual is not None else None
    if r2 is not None:
        assert r2.is_contiguous()
    _ck(_lib.lib().mb_rmsnorm_fwd(x2.data_ptr(), _ptr(w), _ptr(r2), y.data_ptr(), rstd.data_ptr(), M, D,
                                  float(eps), int(unit_offset), _stream()), "rmsnorm_fwd")
    return y.view(x.shape), rstd


def set_norm_pipeline(on: bool) -> None:
    """Select the bulk-copy pipelined RMSNorm kernels (csrc/norm_tma.cu) for tall inputs instead of the default
    row-per-warp kernels (measured slightly slower at the benchmark shape; kept selectable and tested)."""
    _lib.lib().mb_set_norm_pipeline(int(bool(on)))


def rmsnorm_bwd(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor | None, rstd: torch.Tensor,
                unit_offset: bool, dw_acc: torch.Tensor | None, dres_add: torch.Tensor | None = None):
    D = x.shape[-1]
    dy2, x2 = dy.reshape(-1, D), x.reshape(-1, D)
    assert dy2.is_contiguous() and x2.is_contiguous()
    dx = torch.empty_like(x2)
    a2 = dres_add.reshape(-1, D) if dres_add is not None else None
    _ck(_lib.lib().mb_rmsnorm_bwd(dy2.data_ptr(), x2.data_ptr(), _ptr(w), rstd.data_ptr(), _ptr(a2),
                                  dx.data_ptr(), _ptr(dw_acc), x2.shape[0], D, int(unit_offset), _stream()),
        "rmsnorm_bwd")
    return dx.view(x.shape)


def qknorm_rope_fwd(qkv: torch.Tensor, qw, kw, pos: torch.Tensor, cs: torch.Tensor | None, H: int, KV: int,
                    hd: int, layout: int, eps: float, unit_offset: bool) -> torch.Tensor:
    """qkv: [T, (H+2KV)*hd] -> rotated/normalised q,k packed as [T, (H+KV)*hd]."""
    T = qkv.shape[0]
    assert qkv.stride(1) == 1
    out = torch.empty(T, (H + KV) * hd, device=qkv.device, dtype=qkv.dtype)
    rot = cs.shape[1] * 2 if cs is not None else 0
    _ck(_lib.lib().mb_qknorm_rope_fwd(qkv.data_ptr(), _ptr(qw), _ptr(kw), _ptr(pos), _ptr(cs), out.data_ptr(), T,
                                      H, KV, hd, rot, layout, float(eps), int(unit_offset), qkv.stride(0),
                                      out.stride(0), _stream()), "qknorm_rope_fwd")
    return out


def qknorm_rope_bwd(dqk: torch.Tensor, qkv: torch.Tensor, qw, kw, pos, cs, dqw, dkw, H: int, KV: int, hd: int,
                    layout: int, eps: float, unit_offset: bool) -> None:
    """In place on the q,k columns of ``dqk`` (row pitch arbitrary)."""
    T = qkv.shape[0]
    rot = cs.shape[1] * 2 if cs is not None else 0
    _ck(_lib.lib().mb_qknorm_rope_bwd(dqk.data_ptr(), qkv.data_ptr(), _ptr(qw), _ptr(kw), _ptr(pos), _ptr(cs),
                                      _ptr(dqw), _ptr(dkw), T, H, KV, hd, rot, layout, float(eps),
                                      int(unit_offset), dqk.stride(0), qkv.stride(0), _stream()),
        "qknorm_rope_bwd")


def glu_fwd(gate_up: torch.Tensor, act: int) -> torch.Tensor:
    F2 = gate_up.shape[-1]
    g2 = gate_up.reshape(-1, F2)
    assert g2.stride(1) == 1
    out = torch.empty(g2.shape[0], F2 // 2, device=g2.device, dtype=g2.dtype)
    _ck(_lib.lib().mb_glu_fwd(g2.data_ptr(), out.data_ptr(), g2.shape[0], F2 // 2, act, g2.stride(0), _stream()),
        "glu_fwd")
    return out.view(*gate_up.shape[:-1], F2 // 2)


def glu_bwd(gate_up: torch.Tensor, dout: torch.Tensor, act: int) -> torch.Tensor:
    F2 = gate_up.shape[-1]
    g2 = gate_up.reshape(-1, F2)
    d2 = dout.reshape(-1, F2 // 2)
    assert d2.is_contiguous() and g2.stride(1) == 1
    din = torch.empty(g2.shape[0], F2, device=g2.device, dtype=g2.dtype)
    _ck(_lib.lib().mb_glu_bwd(g2.data_ptr(), d2.data_ptr(), din.data_ptr(), g2.shape[0], F2 // 2, act,
                              g2.stride(0), _stream()), "glu_bwd")
    return din.view(gate_up.shape)


def syrk(a: torch.Tensor, aux: torch.Tensor | None = None, alpha: float = 1.0, beta: float = 0.0) -> torch.Tensor:
    """``alpha * a @ a.T (+ beta * aux)`` (bf16): only the tiles on and below the diagonal are computed, the rest
    is mirrored by the epilogue."""
    M, K = a.shape
    out = torch.empty(M, M, device=a.device, dtype=a.dtype)
    _ck(_lib.lib().mb_syrk_bf16(a.data_ptr(), out.data_ptr(), _ptr(aux), M, K, _rows_pitch(a), M,
                                _rows_pitch(aux) if aux is not None else 0, float(alpha), float(beta), _stream()), "syrk")
    return out


def gemm_glu_fwd(x: torch.Tensor, w_gu: torch.Tensor, act: int):
    """``gate_up = x @ w_gu.T`` ([M, 2F]) and ``act(gate) * up`` ([M, F]) from one GEMM (CTA-pair kernel)."""
    M, K = x.shape
    F = w_gu.shape[0] // 2
    gate_up = torch.empty(M, 2 * F, device=x.device, dtype=x.dtype)
    out = torch.empty(M, F, device=x.device, dtype=x.dtype)
    _ck(_lib.lib().mb_gemm_glu_fwd(x.data_ptr(), w_gu.data_ptr(), gate_up.data_ptr(), out.data_ptr(), M, F, K,
                                   _rows_pitch(x), _rows_pitch(w_gu), 2 * F, F, int(act), _stream()), "gemm_glu_fwd")
    return gate_up, out


def gemm_glu_bwd(dy: torch.Tensor, w_down: torch.Tensor, gate_up: torch.Tensor, act: int) -> torch.Tensor:
    """``d[gate | up]`` ([M, 2F]) from ``d(act) = dy @ w_down`` (never stored) and the saved ``gate_up``."""
    M, D = dy.shape
    F = w_down.shape[1]
    d_gu = torch.empty(M, 2 * F, device=dy.device, dtype=dy.dtype)
    _ck(_lib.lib().mb_gemm_glu_bwd(dy.data_ptr(), w_down.data_ptr(), gate_up.data_ptr(), d_gu.data_ptr(), M, F, D,
                                   _rows_pitch(dy), _rows_pitch(w_down), _rows_pitch(gate_up), 2 * F, int(act),
                                   _stream()), "gemm_glu_bwd")
    return d_gu


def embedding_fwd(tokens: torch.Tensor, w: torch.Tensor, scale: float | None) -> torch.Tensor:
    tok = tokens.reshape(-1).to(torch.int64).contiguous()
    D = w.shape[1]
    out = torch.empty(tok.numel(), D, device=w.device, dtype=w.dtype)
    s = 1.0 if scale is None else float(torch.tensor(scale, dtype=w.dtype).float())
    _ck(_lib.lib().mb_embedding_fwd(tok.data_ptr(), w.data_ptr(), out.data_ptr(), tok.numel(), D, s,
                                    int(scale is not None), _stream()), "embedding_fwd")
    return out.view(*tokens.shape, D)


def embedding_bwd(tokens: torch.Tensor, dout: torch.Tensor, dw_acc: torch.Tensor, scale: float | None) -> None:
    tok = tokens.reshape(-1).to(torch.int64).contiguous()
    D = dout.shape[-1]
    d2 = dout.reshape(-1, D)
    assert d2.is_contiguous() and dw_acc.dtype == torch.float32 and dw_acc.is_contiguous()
    s = 1.0 if scale is None else float(torch.tensor(scale, dtype=dout.dtype).float())
    _ck(_lib.lib().mb_embedding_bwd(tok.data_ptr(), d2.data_ptr(), dw_acc.data_ptr(), tok.numel(), D, s, _stream()),
        "embedding_bwd")


def ce_fwd_bwd(logits: torch.Tensor, labels: torch.Tensor, loss_sum: torch.Tensor, grad_scale: torch.Tensor,
               logit_scale: float = 1.0, write_grad: bool = True, lse_out: torch.Tensor | None = None) -> None:
    R, V = logits.shape
    _ck(_lib.lib().mb_ce_fwd_bwd(logits.data_ptr(), labels.data_ptr(), loss_sum.data_ptr(), grad_scale.data_ptr(),
                                 float(logit_scale), R, V, logits.stride(0), -100, int(write_grad), _ptr(lse_out),
                                 _stream()), "ce_fwd_bwd")


CE_TILE = 256  # columns per statistics record of gemm_ce (the CTA-pair GEMM's tile width)


def gemm_ce(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, v0: int = 0, logit_scale: float = 1.0,
            logits: torch.Tensor | None = None, store_logits: bool = True):
    """Logits GEMM with cross-entropy statistics in its epilogue.

    Returns ``(logits, stats, tgt)``: logits ``[M, V]`` bf16 = ``logit_scale * h @ w.T`` (None when
    ``store_logits`` is false), stats fp32 ``[tiles, M, 2]`` = (max, sum exp(x - max)) per row and 256-column tile,
    tgt fp32 ``[M]`` = the logit at column ``labels - v0`` where that column exists in ``w``, else 0."""
    M, K = h.shape
    V = w.shape[0]
    tiles = (V + CE_TILE - 1) // CE_TILE
    if store_logits and logits is None:
        logits = torch.empty(M, V, device=h.device, dtype=torch.bfloat16)
    stats = torch.empty(tiles, M, 2, device=h.device, dtype=torch.float32)
    tgt = torch.empty(M, device=h.device, dtype=torch.float32)
    _ck(_lib.lib().mb_gemm_ce(h.data_ptr(), w.data_ptr(), logits.data_ptr() if store_logits else None,
                              labels.data_ptr(), stats.data_ptr(), tgt.data_ptr(), M, V, K, _rows_pitch(h),
                              _rows_pitch(w), logits.stride(0) if store_logits else 0, int(v0), float(logit_scale), M,
                              _stream()), "gemm_ce")
    return (logits if store_logits else None), stats, tgt


def ce_merge(stats: torch.Tensor, tgt: torch.Tensor, rec: torch.Tensor) -> None:
    """Fold the per-tile statistics of every row into ``rec[row] = (max, sum, target, 0)`` (fp32 ``[M, 4]``)."""
    tiles, M, _ = stats.shape
    _ck(_lib.lib().mb_ce_merge(stats.data_ptr(), tgt.data_ptr(), rec.data_ptr(), M, tiles, M, _stream()), "ce_merge")


def ce_grad(logits: torch.Tensor | None, labels: torch.Tensor, rec_ptrs: list[int], loss_sum: torch.Tensor | None,
            grad_scale: torch.Tensor, v0: int = 0, write_grad: bool = True, rows: int | None = None) -> None:
    """Row losses from the records of all vocabulary slices (``rec_ptrs``: one device address per rank, at this
    chunk's first row) and, in place, ``logits <- (softmax - onehot) * grad_scale``."""
    R = rows if rows is not None else logits.shape[0]
    V = logits.shape[1] if logits is not None else 0
    arr = (ctypes.c_void_p * len(rec_ptrs))(*rec_ptrs)
    _ck(_lib.lib().mb_ce_grad(_ptr(logits), labels.data_ptr(), arr, len(rec_ptrs), _ptr(loss_sum),
                              grad_scale.data_ptr(), R, V, logits.stride(0) if logits is not None else 8, int(v0),
                              -100, int(write_grad and logits is not None), _stream()), "ce_grad")


def expect_scalar(x: torch.Tensor, want: float) -> None:
    """Records a status error (read by ``check_status``) unless the fp32 device scalar ``x`` equals ``want``."""
    _ck(_lib.lib().mb_expect_scalar(x.data_ptr(), float(want), _stream()), "expect_scalar")


def adamw(p, g, m, v, lp, chunks, tensors, nchunks, lr_t, beta1, beta2, eps, step, grad_scale=1.0,
          zero_grad=False) -> None:
    bc1 = 1.0 - beta1 ** step
    bc2s = math.sqrt(1.0 - beta2 ** step)
    _ck(_lib.lib().mb_adamw(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), _ptr(lp), chunks.data_ptr(),
                            tensors.data_ptr(), nchunks, lr_t.data_ptr(), beta1, beta2, eps, bc1, bc2s,
                            float(grad_scale), int(zero_grad), _stream()), "adamw")


def fused_rs_adamw_ag(symm_grad, symm_full, master, m, v, shard_grad_out, chunks, tensors, nchunks, lr_t, beta1,
                      beta2, eps, step, divide: float) -> None:
    """Reduce-scatter + AdamW + all-gather in one kernel over peer memory (``symm_*``: SymmBuffer)."""
    bc1 = 1.0 - beta1 ** step
    bc2s = math.sqrt(1.0 - beta2 ** step)
    use_mc = bool(symm_grad.multicast_ptr and symm_full.multicast_ptr)
    _ck(_lib.lib().mb_fused_rs_adamw_ag(
        symm_grad.multicast_ptr if use_mc else None, symm_full.multicast_ptr if use_mc else None,
        symm_grad.ptr_array, symm_full.ptr_array, symm_grad.world, master.data_ptr(), m.data_ptr(), v.data_ptr(),
        _ptr(shard_grad_out), chunks.data_ptr(), tensors.data_ptr(), nchunks, lr_t.data_ptr(), beta1, beta2, eps,
        bc1, bc2s, 1.0 / divide, _stream()), "fused_rs_adamw_ag")


def push_shards(master: torch.Tensor, symm_full, chunks: torch.Tensor, nchunks: int) -> None:
    """bf16 copy of this rank's fp32 shard into every rank's param-major parameter buffer."""
    mc = symm_full.multicast_ptr or None
    _ck(_lib.lib().mb_push_shards(master.data_ptr(), mc, symm_full.ptr_array, symm_full.world, chunks.data_ptr(),
                                  nchunks, _stream()), "push_shards")


def peer_scatter_rows(src: torch.Tensor, symm_dst, dest_rank: torch.Tensor, dest_row: torch.Tensor, cap_rows: int,
                      overflow: torch.Tensor) -> None:
    """Write row i of ``src`` [n, dim] into rank dest_rank[i]'s symmetric buffer at row dest_row[i]."""
    n, dim = src.shape
    assert src.is_contiguous() and dest_rank.dtype == torch.int32 and dest_row.dtype == torch.int32
    _ck(_lib.lib().mb_peer_scatter_rows(src.data_ptr(), symm_dst.ptr_array, symm_dst.world, dest_rank.data_ptr(),
                                        dest_row.data_ptr(), n, dim, cap_rows, overflow.data_ptr(), _stream()),
        "peer_scatter_rows")


def peer_gather_rows(dst: torch.Tensor, symm_src, src_rank: torch.Tensor, src_row: torch.Tensor, cap_rows: int,
                     overflow: torch.Tensor) -> None:
    """Fill row i of ``dst`` [n, dim] from rank src_rank[i]'s symmetric buffer row src_row[i]."""
    n, dim = dst.shape
    assert dst.is_contiguous() and src_rank.dtype == torch.int32 and src_row.dtype == torch.int32
    _ck(_lib.lib().mb_peer_gather_rows(dst.data_ptr(), symm_src.ptr_array, symm_src.world, src_rank.data_ptr(),
                                       src_row.data_ptr(), n, dim, cap_rows, overflow.data_ptr(), _stream()),
        "peer_gather_rows")


def mla_pack_fwd(q: torch.Tensor, kvb: torch.Tensor, kpe: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor,
                 H: int, nope: int, rope: int, vdim: int, P: int) -> torch.Tensor:
    """q [T, H*(nope+rope)], kvb [T, H*(nope+vdim)], kpe [T, rope] (row-strided view) -> packed [T, 3*H*P] with RoPE on
    the rope channels (interleaved pairs) and zero padding up to the head size P of the attention kernel."""
    T = q.shape[0]
    assert q.is_contiguous() and kvb.is_contiguous() and kpe.stride(1) == 1 and pos.dtype == torch.int64
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == rope
    out = torch.empty(T, 3 * H * P, device=q.device, dtype=q.dtype)
    _ck(_lib.lib().mb_mla_pack_fwd(q.data_ptr(), kvb.data_ptr(), kpe.data_ptr(), kpe.stride(0), pos.data_ptr(),
                                   inv_freq.data_ptr(), T, H, nope, rope, vdim, P, out.data_ptr(), _stream()),
        "mla_pack_fwd")
    return out


def mla_pack_bwd(dout: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, H: int, nope: int, rope: int, vdim: int,
                 P: int):
    T = dout.shape[0]
    assert dout.is_contiguous() and dout.shape[1] == 3 * H * P
    dq = torch.empty(T, H * (nope + rope), device=dout.device, dtype=dout.dtype)
    dkvb = torch.empty(T, H * (nope + vdim), device=dout.device, dtype=dout.dtype)
    dkpe = torch.empty(T, rope, device=dout.device, dtype=dout.dtype)
    _ck(_lib.lib().mb_mla_pack_bwd(dout.data_ptr(), pos.data_ptr(), inv_freq.data_ptr(), T, H, nope, rope, vdim, P,
                                   dq.data_ptr(), dkvb.data_ptr(), dkpe.data_ptr(), _stream()), "mla_pack_bwd")
    return dq, dkvb, dkpe


def ep_plan(allc: torch.Tensor, me: int, n_local: int, idx: torch.Tensor, inv: torch.Tensor, align: int, cap: int):
    """Destination (rank, row) of every routing slot from the all-gathered per-expert counts ``allc`` [ep, E];
    also the padded group offsets [n_local + 1] of this rank's experts.  All on the device."""
    ep, E = allc.shape
    n = idx.numel()
    assert allc.dtype == torch.int32 and idx.dtype == torch.int32 and inv.dtype == torch.int32 and allc.is_contiguous()
    out = torch.empty(2 * n + n_local + 1, device=idx.device, dtype=torch.int32)
    slot_rank, slot_row, offs = torch.split(out, [n, n, n_local + 1])
    _ck(_lib.lib().mb_ep_plan(allc.data_ptr(), ep, me, E, n_local, idx.data_ptr(), inv.data_ptr(), n, align, cap,
                              slot_rank.data_ptr(), slot_row.data_ptr(), offs.data_ptr(), _stream()), "ep_plan")
    return slot_rank, slot_row, offs


def ep_zero_padding(buf: torch.Tensor, allc: torch.Tensor, me: int, n_local: int, offs: torch.Tensor, dim: int,
                    cap: int) -> None:
    """Zero only the padding rows of the local experts' groups in this rank's [cap, dim] expert-major buffer."""
    ep, E = allc.shape
    assert buf.dtype == torch.bfloat16 and buf.numel() >= cap * dim and offs.dtype == torch.int32
    _ck(_lib.lib().mb_ep_zero_padding(buf.data_ptr(), allc.data_ptr(), ep, me, E, n_local, offs.data_ptr(), dim, cap,
                                      _stream()), "ep_zero_padding")


def peer_dispatch_rows(x: torch.Tensor, symm_dst, slot_rank: torch.Tensor, slot_row: torch.Tensor,
                       slot_scale: torch.Tensor | None, k: int, cap_rows: int, overflow: torch.Tensor) -> None:
    """Row t of ``x`` (times its gate value) into the buffers of the ranks that own its k experts."""
    T, dim = x.shape
    assert x.is_contiguous() and x.dtype == torch.bfloat16 and slot_rank.numel() == T * k
    _ck(_lib.lib().mb_peer_dispatch_rows(x.data_ptr(), symm_dst.ptr_array, symm_dst.world, slot_rank.data_ptr(),
                                         slot_row.data_ptr(), _ptr(slot_scale), T, k, dim, cap_rows, overflow.data_ptr(),
                                         _stream()), "peer_dispatch_rows")


def peer_combine_rows(symm_src, slot_rank: torch.Tensor, slot_row: torch.Tensor, slot_scale: torch.Tensor | None,
                      T: int, k: int, dim: int, cap_rows: int, overflow: torch.Tensor) -> torch.Tensor:
    """out[t] = sum over the k slots of token t of the (weighted) rows read from the owning ranks' buffers."""
    out = torch.empty(T, dim, device=slot_rank.device, dtype=torch.bfloat16)
    _ck(_lib.lib().mb_peer_combine_rows(out.data_ptr(), symm_src.ptr_array, symm_src.world, slot_rank.data_ptr(),
                                        slot_row.data_ptr(), _ptr(slot_scale), T, k, dim, cap_rows, overflow.data_ptr(),
                                        _stream()), "peer_combine_rows")
    return out


def peer_slot_dot(symm_src, slot_rank: torch.Tensor, slot_row: torch.Tensor, g: torch.Tensor, k: int,
                  cap_rows: int) -> torch.Tensor:
    """d[t*k+j] = <row of slot (t, j) in its owner's buffer, g[t]> in fp32."""
    T, dim = g.shape
    assert g.is_contiguous() and g.dtype == torch.bfloat16
    out = torch.empty(T * k, device=g.device, dtype=torch.float32)
    _ck(_lib.lib().mb_peer_slot_dot(out.data_ptr(), symm_src.ptr_array, symm_src.world, slot_rank.data_ptr(),
                                    slot_row.data_ptr(), g.data_ptr(), T, k, dim, cap_rows, _stream()), "peer_slot_dot")
    return out


def gemm_rs(a: torch.Tensor, b: torch.Tensor, symm_out, my_rank: int, *, a_mn: bool = False, b_mn: bool = False,
            alpha: float = 1.0) -> None:
    """``op(A) @ op(B).T`` with the output rows scattered to their owner ranks' symmetric buffers
    ``symm_out`` ([world, M/world, N] bf16 on every rank; this rank writes slot ``my_rank`` everywhere)."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    M, K = (a.shape[1], a.shape[0]) if a_mn else a.shape
    N = b.shape[1] if b_mn else b.shape[0]
    _ck(_lib.lib().mb_gemm_bf16_rs(a.data_ptr(), b.data_ptr(), symm_out.ptr_array, symm_out.world, my_rank, M, N, K,
                                   _rows_pitch(a), _rows_pitch(b), N, int(a_mn), int(b_mn), float(alpha), _stream()),
        "gemm_bf16_rs")


def gemm_ag(a_full: torch.Tensor, symm_blocks, my_rank: int, b: torch.Tensor, flags: torch.Tensor, *,
            b_mn: bool = False, copiers: int = 4) -> torch.Tensor:
    """``a_full @ op(b).T`` where ``a_full`` [M, K] holds only this rank's row block so far: the other ranks' blocks
    are pulled from their symmetric buffers by ``copiers`` CTA pairs of the same kernel (fused all-gather)."""
    M, K = a_full.shape
    N = b.shape[1] if b_mn else b.shape[0]
    assert a_full.is_contiguous() and a_full.dtype == torch.bfloat16 and (b.shape[0] if b_mn else b.shape[1]) == K
    assert flags.dtype == torch.int32 and flags.numel() >= M // 256
    out = torch.empty(M, N, device=a_full.device, dtype=torch.bfloat16)
    _ck(_lib.lib().mb_gemm_bf16_ag(a_full.data_ptr(), symm_blocks.ptr_array, symm_blocks.world, my_rank, b.data_ptr(),
                                   out.data_ptr(), M, N, K, _rows_pitch(b), N, int(b_mn), copiers, flags.data_ptr(),
                                   _stream()), "gemm_ag")
    return out


def gemm_ag_glu(a_full: torch.Tensor, symm_blocks, my_rank: int, b: torch.Tensor, flags: torch.Tensor, *, mode: int,
                act: int, gate_up: torch.Tensor | None = None, copiers: int = 4):
    """The all-gather GEMM with a gated-linear-unit epilogue.

    mode 1 (forward): ``b`` = fused weight ``[2F, K]``; returns ``(gate_up [M, 2F], act(gate) * up [M, F])``.
    mode 2 (backward): ``a_full`` gathers dy ``[M, K]``, ``b`` = down-projection weight ``[K, F]``, ``gate_up`` the
    tensor saved by the forward pass; returns ``d[gate | up]`` ``[M, 2F]``."""
    M, K = a_full.shape
    assert a_full.is_contiguous() and a_full.dtype == torch.bfloat16 and flags.numel() >= M // 256
    if mode == 1:
        F = b.shape[0] // 2
        assert b.shape[1] == K
        c = torch.empty(M, 2 * F, device=a_full.device, dtype=torch.bfloat16)
        io = torch.empty(M, F, device=a_full.device, dtype=torch.bfloat16)
    else:
        F = b.shape[1]
        assert b.shape[0] == K and gate_up is not None and gate_up.shape == (M, 2 * F) and gate_up.is_contiguous()
        c = torch.empty(M, 2 * F, device=a_full.device, dtype=torch.bfloat16)
        io = gate_up
    _ck(_lib.lib().mb_gemm_bf16_ag_glu(a_full.data_ptr(), symm_blocks.ptr_array, symm_blocks.world, my_rank,
                                       b.data_ptr(), c.data_ptr(), M, F, K, _rows_pitch(b), 2 * F, copiers,
                                       flags.data_ptr(), int(mode), int(act), io.data_ptr(), _rows_pitch(io), _stream()),
        "gemm_ag_glu")
    return (c, io) if mode == 1 else c


def wait_flag(flag: torch.Tensor, expect: int, timeout_ms: float, observed: torch.Tensor | None = None) -> None:
    """Stream-ordered bounded wait until ``flag[0] >= expect`` (int32 device tensor, may be peer memory).
    On expiry the library status word is set (``check_status`` raises) and the stream simply continues."""
    assert flag.dtype == torch.int32 and (observed is None or observed.dtype == torch.int32)
    _ck(_lib.lib().mb_wait_flag_probe(flag.data_ptr(), int(expect), float(timeout_ms), _ptr(observed), _stream()),
        "wait_flag_probe")


def symm_barrier(pad_array, world: int, me: int, base: int, epoch: int, timeout_ms: float) -> None:
    """Stream-ordered cross-rank barrier on per-rank signal pads (``pad_array``: ``void*[world]``); bounded wait."""
    _ck(_lib.lib().mb_symm_barrier(pad_array, int(world), int(me), int(base), int(epoch), float(timeout_ms),
                                   _stream()), "symm_barrier")


def pull_sum(symm_parts, my_rank: int, res: torch.Tensor | None, out: torch.Tensor) -> None:
    """out [M/world, N] = (res or 0) + sum over ranks of rows [my_rank*M/world, ...) of their [M, N] partials."""
    assert out.is_contiguous() and (res is None or res.is_contiguous())
    _ck(_lib.lib().mb_pull_sum(symm_parts.ptr_array, symm_parts.world, my_rank, _ptr(res), out.data_ptr(),
                               out.shape[0], out.shape[1], _stream()), "pull_sum")


def sum_partials(parts: torch.Tensor, res: torch.Tensor | None, out: torch.Tensor, world: int) -> None:
    """out = (res or 0) + sum of the ``world`` slices of ``parts`` ([world * out.numel()] bf16)."""
    assert out.is_contiguous() and (res is None or res.is_contiguous())
    _ck(_lib.lib().mb_sum_partials(parts.data_ptr(), _ptr(res), out.data_ptr(), out.numel(), world, _stream()),
        "sum_partials")


def peer_copy(dst: torch.Tensor, src_ptr: int, nbytes: int) -> None:
    """``dst`` (local, contiguous) <- ``nbytes`` from the device address ``src_ptr``, which may be a peer GPU's
    memory mapped into this process (plain loads and stores of this library's own kernel)."""
    assert dst.is_contiguous() and dst.numel() * dst.element_size() >= nbytes
    _ck(_lib.lib().mb_peer_copy(dst.data_ptr(), int(src_ptr), int(nbytes), _stream()), "peer_copy")


def peer_gather(dst: torch.Tensor, symm_shards, descs: torch.Tensor, slices: int = 8) -> None:
    """Fill ``dst`` (local bf16 staging buffer) from the ranks' shard buffers (``symm_shards``: SymmBuffer) as listed
    by ``descs`` (int64 ``[n, 4]``: destination offset, source offset, length in elements; source rank), with the
    library's own copy kernel over peer-mapped memory."""
    assert dst.is_contiguous() and descs.dtype == torch.int64 and descs.is_contiguous() and descs.shape[1] == 4
    _ck(_lib.lib().mb_peer_gather(dst.data_ptr(), dst.numel(), symm_shards.ptr_array, symm_shards.world,
                                  descs.data_ptr(), descs.shape[0], int(slices), _stream()), "peer_gather")


def peer_add_bf16(dst: torch.Tensor, src_ptr: int, n: int) -> None:
    """``dst[:n] += *src_ptr`` (bf16; the source may be peer memory)."""
    assert dst.is_contiguous() and dst.dtype == torch.bfloat16 and dst.numel() >= n
    _ck(_lib.lib().mb_peer_add_bf16(dst.data_ptr(), int(src_ptr), int(n), _stream()), "peer_add_bf16")


def attn_merge(acc: torch.Tensor, lse: torch.Tensor, part: torch.Tensor, lse_part: torch.Tensor, row_off: int,
               init: bool) -> None:
    """Fold a partial attention result ``part`` [B, c, H, hd] (bf16) with log-sum-exp ``lse_part`` [B, H, c] into the
    fp32 accumulator ``acc`` [B, S, H, hd] / ``lse`` [B, H, S] at rows ``row_off .. row_off + c``."""
    B, S, H, hd = acc.shape
    c = part.shape[1]
    assert acc.is_contiguous() and lse.is_contiguous() and part.is_contiguous() and lse_part.is_contiguous()
    assert acc.dtype == torch.float32 and part.dtype == torch.bfloat16 and row_off + c <= S
    _ck(_lib.lib().mb_attn_merge(acc.data_ptr(), lse.data_ptr(), part.data_ptr(), lse_part.data_ptr(), B, c, H, hd, S,
                                 int(row_off), int(bool(init)), _stream()), "attn_merge")


def multi_sqnorm(flat: torch.Tensor, chunks: torch.Tensor, nchunks: int, out: torch.Tensor | None,
                 scale: torch.Tensor | None = None) -> None:
    """``out[t] += sum(x_t ** 2)`` for every tensor t of the flat fp32 buffer (one launch; chunk table as for AdamW);
    with ``scale`` (device scalar) the buffer is also multiplied by it."""
    assert flat.dtype == torch.float32 and (out is None or out.dtype == torch.float32)
    _ck(_lib.lib().mb_multi_sqnorm(flat.data_ptr(), chunks.data_ptr(), int(nchunks), _ptr(out), _ptr(scale), _stream()),
        "multi_sqnorm")


def cast_f32_bf16(x: torch.Tensor, y: torch.Tensor, scale: float = 1.0) -> None:
    _ck(_lib.lib().mb_cast_f32_bf16(x.data_ptr(), y.data_ptr(), x.numel(), float(scale), _stream()), "cast")


def _plan_ptrs(plan):
    if plan is None:
        return None, None, None, None, None
    return _ptr(plan.doc), _ptr(plan.lo_blk), _ptr(plan.hi_blk), _ptr(plan.kv_start), _ptr(plan.q_end)


def attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, causal: bool, window: int | None,
             plan=None):
    """q: [B,S,H,hd] (last two dims dense, token stride arbitrary); k, v: [B,S,KV,hd].  ``plan`` is the
    ``ops.functional.AttnPlan`` of the mask (None: causal / window bounds only)."""
    B, S, H, hd = q.shape
    KV = k.shape[2]
    for t in (q, k, v):
        assert t.stride(3) == 1 and t.stride(2) == hd and t.stride(0) == S * t.stride(1)
    out = torch.empty(B, S, H, hd, device=q.device, dtype=q.dtype)
    lse = torch.empty(B, H, S, device=q.device, dtype=torch.float32)
    doc, lo, _, kv_start, _ = _plan_ptrs(plan)
    _ck(_lib.lib().mb_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), doc, lo,
                               kv_start, B, S, H, KV, hd, q.stride(1), k.stride(1), v.stride(1),
                               int(causal), -1 if window is None or window <= 0 else int(window), float(scale),
                               _stream()), "attn_fwd")
    return out, lse


def attn_bwd(q, k, v, out, dout, lse, dqkv, scale, causal, window, plan=None) -> None:
    """Fills ``dqkv`` [B*S, (H+2KV)*hd] with the gradients of q, k (post norm/rope) and v."""
    B, S, H, hd = q.shape
    KV = k.shape[2]
    assert out.is_contiguous() and dout.is_contiguous() and dqkv.stride(1) == 1
    delta = torch.empty(B, H, S, device=q.device, dtype=torch.float32)
    doc, lo, hi, kv_start, q_end = _plan_ptrs(plan)
    _ck(_lib.lib().mb_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(),
                               lse.data_ptr(), delta.data_ptr(), dqkv.data_ptr(), doc, lo, hi, kv_start, q_end,
                               B, S, H, KV, hd, q.stride(1), k.stride(1), v.stride(1),
                               dqkv.stride(0), int(causal), -1 if window is None or window <= 0 else int(window),
                               float(scale), _stream()), "attn_bwd")


def gemm_grouped_rows(a: torch.Tensor, b: torch.Tensor, offs: torch.Tensor, *, b_mn: bool,
                      out: torch.Tensor | None = None, epi: int = EPI_BF16, alpha: float = 1.0) -> torch.Tensor:
    """Per-group GEMM over row groups of ``a`` ([rows_cap, K]); ``offs`` are padded (x128) int32 device offsets.

    b_mn=True : b is [E, K, N] and out_e = a_e @ b_e;  b_mn=False: b is [E, N, K] and out_e = a_e @ b_e.T
    """
    rows_cap, K = a.shape
    E = b.shape[0]
    N = b.shape[2] if b_mn else b.shape[1]
    assert (b.shape[1] if b_mn else b.shape[2]) == K and b.is_contiguous() and offs.dtype == torch.int32
    if out is None:
        out = torch.empty(rows_cap, N, device=a.device, dtype=torch.bfloat16 if epi == EPI_BF16 else torch.float32)
    b2 = b.view(E * b.shape[1], b.shape[2])
    _ck(_lib.lib().mb_gemm_bf16_grouped_rows(a.data_ptr(), b2.data_ptr(), out.data_ptr(), offs.data_ptr(), E,
                                             rows_cap, N, K, _rows_pitch(a), _rows_pitch(b2), _rows_pitch(out),
                                             int(b_mn), epi, float(alpha), _stream()), "gemm_grouped_rows")
    return out


def gemm_grouped_contr(a: torch.Tensor, b: torch.Tensor, offs: torch.Tensor, out: torch.Tensor,
                       epi: int = EPI_F32_ACC, alpha: float = 1.0) -> torch.Tensor:
    """out[e] (+)= a_e.T @ b_e for row groups of a ([rows_cap, M]) and b ([rows_cap, N]); out is [E, M, N]."""
    rows_cap, M = a.shape
    N = b.shape[1]
    E = out.shape[0]
    assert out.shape == (E, M, N) and out.is_contiguous() and offs.dtype == torch.int32
    pair = GROUPED_CONTR_TWO_CTA and epi in (EPI_F32, EPI_F32_ACC) and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0
    fn = _lib.lib().mb_gemm_bf16_2cta_grouped_contr if pair else _lib.lib().mb_gemm_bf16_grouped_contr
    _ck(fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), offs.data_ptr(), E, rows_cap, M, N, _rows_pitch(a), _rows_pitch(b),
           N, epi, float(alpha), _stream()), "gemm_grouped_contr")
    return out


class RoutePlan:
    """Device-side routing plan of one MoE block (all int32 / fp32 tensors, no host values)."""
    __slots__ = ("T", "E", "k", "rows_cap", "scores", "top", "idx", "counts", "counts_f", "offs", "order", "inv",
                 "slot_row", "row_slot", "sorted_scores", "token_idx", "sorted_experts", "_ints", "_sizes")

    def as_long(self) -> dict[str, torch.Tensor]:
        """int64 copies of the index vectors (one conversion launch) for code that indexes with them."""
        names = ("counts", "offs", "order", "inv", "slot_row", "token_idx", "sorted_experts", "row_slot")
        return dict(zip(names, torch.split(self._ints.long(), self._sizes)))


def moe_route(logits: torch.Tensor, bias: torch.Tensor | None, k: int, softmax: bool, norm: bool, scale: float,
              force_balance: bool, align: int) -> RoutePlan:
    """Score function, (biased) top-k, histogram and a stable expert-major ordering of the T*k slots."""
    T, E = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    dev = logits.device
    p = RoutePlan()
    p.T, p.E, p.k = T, E, k
    p.rows_cap = (T * k + E * (align - 1) + align - 1) // align * align
    n = T * k
    f32 = dict(device=dev, dtype=torch.float32)
    i32 = dict(device=dev, dtype=torch.int32)
    p.scores = torch.empty(T, E, **f32)
    p.top = torch.empty(T, k, **f32)
    p.idx = torch.empty(T, k, **i32)
    p.counts_f = torch.empty(E, **f32)
    ints = torch.empty(E + (E + 1) + 5 * n + p.rows_cap, **i32)  # one allocation for the index vectors
    p._ints, p._sizes = ints, [E, E + 1, n, n, n, n, n, p.rows_cap]
    parts = torch.split(ints, p._sizes)
    p.counts, p.offs, p.order, p.inv, p.slot_row, p.token_idx, p.sorted_experts, p.row_slot = parts
    p.sorted_scores = torch.empty(n, **f32)
    scratch = torch.empty((T + 63) // 64 * E + E, **i32)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == E
    _ck(_lib.lib().mb_moe_route(logits.data_ptr(), _ptr(bias), T, E, k, int(softmax), int(norm), float(scale),
                                int(force_balance), align, p.rows_cap, p.scores.data_ptr(), p.top.data_ptr(),
                                p.idx.data_ptr(), p.counts.data_ptr(), p.counts_f.data_ptr(), p.offs.data_ptr(),
                                p.order.data_ptr(), p.inv.data_ptr(), p.slot_row.data_ptr(), p.row_slot.data_ptr(),
                                p.sorted_scores.data_ptr(), p.token_idx.data_ptr(), p.sorted_experts.data_ptr(),
                                scratch.data_ptr(), _stream()), "moe_route")
    return p


def moe_route_bwd(d_top: torch.Tensor, d_scores: torch.Tensor | None, scores: torch.Tensor, idx: torch.Tensor,
                  softmax: bool, norm: bool, scale: float) -> torch.Tensor:
    T, E = scores.shape
    k = idx.shape[1]
    d_top = d_top.contiguous().float()
    if d_scores is not None:
        d_scores = d_scores.contiguous().float()
    out = torch.empty_like(scores)
    _ck(_lib.lib().mb_moe_route_bwd(d_top.data_ptr(), _ptr(d_scores), scores.data_ptr(), idx.data_ptr(), T, E, k,
                                    int(softmax), int(norm), float(scale), out.data_ptr(), _stream()), "moe_route_bwd")
    return out


def moe_rows_gather(x: torch.Tensor, row_slot: torch.Tensor, slot_scale: torch.Tensor | None, k: int) -> torch.Tensor:
    """buf[r] = x[row_slot[r] // k] (* slot_scale[row_slot[r]]); zero rows where row_slot[r] < 0."""
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and row_slot.dtype == torch.int32
    rows, dim = row_slot.numel(), x.shape[1]
    buf = torch.empty(rows, dim, device=x.device, dtype=x.dtype)
    _ck(_lib.lib().mb_moe_rows_gather(x.data_ptr(), row_slot.data_ptr(), _ptr(slot_scale), k, rows, dim, buf.data_ptr(),
                                      _stream()), "moe_rows_gather")
    return buf


def moe_rows_combine(buf: torch.Tensor, slot_row: torch.Tensor, slot_scale: torch.Tensor | None, k: int) -> torch.Tensor:
    """out[t] = sum_j buf[slot_row[t*k+j]] (* slot_scale[t*k+j]) with fp32 accumulation."""
    assert buf.dtype == torch.bfloat16 and buf.is_contiguous() and slot_row.dtype == torch.int32
    T, dim = slot_row.numel() // k, buf.shape[1]
    out = torch.empty(T, dim, device=buf.device, dtype=buf.dtype)
    _ck(_lib.lib().mb_moe_rows_combine(buf.data_ptr(), slot_row.data_ptr(), _ptr(slot_scale), k, T, dim, buf.shape[0],
                                       out.data_ptr(), _stream()), "moe_rows_combine")
    return out


def moe_slot_dot(buf: torch.Tensor, slot_row: torch.Tensor, g: torch.Tensor, k: int) -> torch.Tensor:
    """d[t*k+j] = <buf[slot_row[t*k+j]], g[t]> in fp32."""
    assert buf.dtype == torch.bfloat16 and g.dtype == torch.bfloat16 and buf.is_contiguous() and g.is_contiguous()
    T, dim = g.shape
    out = torch.empty(T * k, device=buf.device, dtype=torch.float32)
    _ck(_lib.lib().mb_moe_slot_dot(buf.data_ptr(), slot_row.data_ptr(), g.data_ptr(), k, T, dim, buf.shape[0],
                                   out.data_ptr(), _stream()), "moe_slot_dot")
    return out
