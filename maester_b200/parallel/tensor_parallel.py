"""Tensor parallelism with sequence parallelism and loss parallelism.

Reference plan (maester/parallelisms/parallelize_llama.py:107-181): ``wq/wk/wv/w1/w3`` column-parallel,
``wo/w2`` row-parallel with sequence-sharded outputs (reduce-scatter along the sequence), norms and
residual stream on sequence shards, all-gather along the sequence in front of attention and FFN,
``output`` column-parallel with vocabulary-sharded logits feeding a loss that exchanges per-row
(max, sum-exp, target logit).  The reference expresses this with DTensor styles; here the model code
calls the four communication primitives below explicitly, each an autograd function whose backward
is the mirrored collective, and ``apply_tp`` re-shapes the parameters of a model that still lives on
the meta device.

Embedding and norm weights are replicated across the TP group and see only this rank's sequence
slice (the embedding looks up only this rank's tokens), so their gradients are partial sums that are
summed over the group after backward (``tp_replicated`` flag, handled by the sharding runtime).  A tied,
replicated head scores this rank's token slice against the whole vocabulary; an untied head is
vocabulary-parallel and its dH is a partial sum that the backward of the sequence gather reduces.  On
CUDA the loss-parallel cross-entropy runs on the native kernels: the ranks read each other's per-row
(max, sum-exp, target) records through symmetric memory instead of all-reducing them.

Gemma (maester/parallelisms/parallelize_gemma.py:77-178) follows the same scheme with its own block layout
(``_apply_tp_gemma``): the fused ``qkv_proj`` is split by head groups (``qkv_segments``), the four block norms and the
QK-norms are replicated, and the tied head is the replicated form above.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn

from maester_b200.log_utils import logger


@dataclass
class TPInfo:
    group: object
    size: int
    rank: int
    loss_parallel: bool = True
    batch: int = 1  # batch size of the current forward (set by the model; restores [B, S, D] after a gather)


# ------------------------------------------------------------------------------ primitives
# "Sequence-sharded" activations are sharded along the FLATTENED token dimension: rank r holds rows
# [r*T/tp, (r+1)*T/tp) of the [B*S, D] matrix, shaped [1, T/tp, D].  Token-local ops (norms, residual
# adds) do not care, and gathers / reduce-scatters are plain contiguous collectives without any
# permutation copy.
def _all_gather_seq(x: torch.Tensor, tp: TPInfo) -> torch.Tensor:
    """[1, T/tp, D] → [B, S, D]."""
    D = x.shape[-1]
    t = x.numel() // D
    out = torch.empty(tp.size * t, D, device=x.device, dtype=x.dtype)
    dist.all_gather_into_tensor(out.view(-1), x.contiguous().view(-1), group=tp.group)
    return out.view(tp.batch, -1, D)


def _reduce_scatter_seq(x: torch.Tensor, tp: TPInfo) -> torch.Tensor:
    """Sum over the group of [B, S, D], keep this rank's rows of the flattened tokens [1, T/tp, D]."""
    D = x.shape[-1]
    T = x.numel() // D
    out = torch.empty(1, T // tp.size, D, device=x.device, dtype=x.dtype)
    dist.reduce_scatter_tensor(out.view(-1), x.contiguous().view(-1), op=dist.ReduceOp.SUM, group=tp.group)
    return out


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _all_gather_seq(x, tp)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_seq(g, ctx.tp), None


class _ReduceScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _reduce_scatter_seq(x, tp)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_seq(g, ctx.tp), None


class _ScatterSeq(torch.autograd.Function):
    """Keep this rank's sequence slice of a replicated tensor; backward all-gathers the slices."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        D = x.shape[-1]
        t = (x.numel() // D) // tp.size
        return x.reshape(-1, D)[tp.rank * t:(tp.rank + 1) * t].contiguous().view(1, t, D)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_seq(g, ctx.tp), None


class _GatherSeqSameGrad(torch.autograd.Function):
    """All-gather of sequence slices whose consumers compute the same thing on every rank (a replicated loss on the
    gathered tensor): the incoming gradient is already complete and identical everywhere, so backward keeps this
    rank's slice instead of summing the ranks' copies."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _all_gather_seq(x, tp)

    @staticmethod
    def backward(ctx, g):
        tp = ctx.tp
        D = g.shape[-1]
        t = (g.numel() // D) // tp.size
        return g.reshape(-1, D)[tp.rank * t:(tp.rank + 1) * t].contiguous().view(1, t, D), None


class _SumOverGroup(torch.autograd.Function):
    """Sum of per-rank partial losses; every rank's partial enters the total with weight one."""

    @staticmethod
    def forward(ctx, x, group):
        y = x.detach().clone()
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


def gather_seq(x: torch.Tensor, tp: TPInfo | None, same_grad: bool = False) -> torch.Tensor:
    """[1, T/tp, D] -> [B, S, D].  ``same_grad``: what follows is replicated on every rank (see
    ``_GatherSeqSameGrad``); otherwise the ranks' gradients are partial sums and backward reduce-scatters them."""
    if tp is None or tp.size == 1:
        return x
    return _GatherSeqSameGrad.apply(x, tp) if same_grad else _GatherSeq.apply(x, tp)


def local_tokens(tokens: torch.Tensor, tp: TPInfo) -> torch.Tensor:
    """This rank's slice of the flattened tokens (or labels), shaped [1, T/tp]."""
    flat = tokens.reshape(-1)
    t = flat.numel() // tp.size
    return flat[tp.rank * t:(tp.rank + 1) * t].view(1, t)


def sum_over_group(x: torch.Tensor, tp: TPInfo) -> torch.Tensor:
    return _SumOverGroup.apply(x, tp.group)


def reduce_scatter_seq(x: torch.Tensor, tp: TPInfo | None) -> torch.Tensor:
    return x if tp is None or tp.size == 1 else _ReduceScatterSeq.apply(x, tp)


def scatter_seq(x: torch.Tensor, tp: TPInfo | None) -> torch.Tensor:
    return x if tp is None or tp.size == 1 else _ScatterSeq.apply(x, tp)


# ------------------------------------------------------------------------------ loss parallel
class _VocabParallelCE(torch.autograd.Function):
    """Mean CE over vocabulary-sharded logits ``h @ W_localᵀ`` (W_local = rows [v0, v0+Vl) of W).

    Per chunk of rows: local logits, local log-sum-exp and target logit, two small all-reduces over
    the TP group to form the global log-sum-exp and target logit, then the local gradient
    ``softmax_global − onehot``.  Backward turns the kept gradient chunks into dH and dW_local.

    dH is this rank's PARTIAL sum (its vocabulary slice only): ``h`` comes out of the sequence gather, whose backward
    reduce-scatters, i.e. sums the ranks' partial gradients.
    """

    CHUNK = 4096

    @staticmethod
    def forward(ctx, h, w, labels, tp: TPInfo):
        M, D = h.shape
        Vl = w.shape[0]
        v0 = tp.rank * Vl
        labels = labels.reshape(-1)
        valid = labels != -100
        nvalid = valid.sum().clamp_min(1).float()
        local = (labels >= v0) & (labels < v0 + Vl) & valid
        loss_sum = h.new_zeros((), dtype=torch.float32)
        grads = []
        for r0 in range(0, M, _VocabParallelCE.CHUNK):
            r1 = min(M, r0 + _VocabParallelCE.CHUNK)
            logits = torch.nn.functional.linear(h[r0:r1], w).float() if not h.is_cuda else _native_logits(h[r0:r1], w)
            m_loc = logits.max(dim=1).values
            m_glob = m_loc.clone()
            dist.all_reduce(m_glob, op=dist.ReduceOp.MAX, group=tp.group)
            e = torch.exp(logits - m_glob[:, None])
            stats = torch.stack([e.sum(dim=1), torch.zeros_like(m_loc)])
            lab = (labels[r0:r1] - v0).clamp(0, Vl - 1)
            tgt = logits.gather(1, lab[:, None]).squeeze(1)
            stats[1] = torch.where(local[r0:r1], tgt, torch.zeros_like(tgt))
            dist.all_reduce(stats, op=dist.ReduceOp.SUM, group=tp.group)
            lse = m_glob + stats[0].log()
            v = valid[r0:r1]
            loss_sum = loss_sum + torch.where(v, lse - stats[1], torch.zeros_like(lse)).sum()
            g = e / stats[0][:, None]
            g.scatter_add_(1, lab[:, None], -local[r0:r1].to(g.dtype)[:, None])
            g = g * (v.to(g.dtype) / nvalid)[:, None]
            grads.append(g.to(h.dtype))
        ctx.save_for_backward(h, w, *grads)
        ctx.tp = tp
        return loss_sum / nvalid

    @staticmethod
    def backward(ctx, gout):
        h, w, *grads = ctx.saved_tensors
        dh = torch.empty_like(h)
        mg = getattr(w, "main_grad", None)
        dw = mg if mg is not None else torch.zeros(w.shape, device=w.device, dtype=torch.float32)
        from maester_b200 import ops
        native = ops.use_native(h, w) and w.shape[0] % 8 == 0 and h.shape[1] % 8 == 0
        if native:
            from maester_b200.ops import cuda as C
            scale = gout.detach().to(torch.float32).reshape(1).contiguous()
        for i, r0 in enumerate(range(0, h.shape[0], _VocabParallelCE.CHUNK)):
            g = grads[i]
            r1 = r0 + g.shape[0]
            if native:  # bf16 tensor-core GEMMs, fp32 accumulation straight into the gradient buffer
                C.gemm(g, w, b_mn=True, out=dh[r0:r1], alpha_dev=scale)
                C.gemm(g, h[r0:r1], a_mn=True, b_mn=True, out=dw, epi=C.EPI_F32_ACC, alpha_dev=scale)
            else:
                dh[r0:r1] = ((g.float() @ w.float()) * gout).to(h.dtype)
                dw.add_((g.float().t() @ h[r0:r1].float()) * gout)
        return dh, (None if mg is not None else dw.to(w.dtype)), None, None


def _native_logits(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    from maester_b200 import ops
    if ops.use_native(h, w):
        from maester_b200.ops import cuda as C
        return C.gemm(h.contiguous(), w, epi=C.EPI_F32)
    return torch.nn.functional.linear(h, w).float()


class _RecordExchange:
    """Symmetric fp32 buffer ``[2, M, 4]`` through which the ranks of a tensor-parallel group read one another's
    per-row (max, sum-exp, target) records; the two halves alternate between calls, so a rank that runs ahead into
    its next loss never overwrites records a slower peer is still reading."""

    def __init__(self, tp: TPInfo, M: int, device):
        from maester_b200.parallel.symm import SymmBuffer
        self.M = M
        self.buf = SymmBuffer(2 * M * 4, torch.float32, device, tp.group)
        self.calls = 0

    def next_half(self):
        half = self.calls & 1
        self.calls += 1
        return self.buf.tensor.view(2, self.M, 4)[half], [p + half * self.M * 16 for p in self.buf.peer_ptrs]


_EXCHANGES: dict = {}


def _record_exchange(tp: TPInfo, M: int, device) -> _RecordExchange:
    key = (id(tp.group), M, device.index)
    if key not in _EXCHANGES:
        _EXCHANGES[key] = _RecordExchange(tp, M, device)
    return _EXCHANGES[key]


class _VocabParallelCENative(torch.autograd.Function):
    """The loss-parallel cross-entropy on the native kernels: every rank's logits GEMM leaves per-row records of its
    vocabulary slice, the ranks read each other's records through symmetric memory (one bounded barrier per chunk,
    no all-reduce of statistics), and every rank turns its own logits into ``softmax_global - onehot`` in place.
    Gradients are produced during forward when the output gradient is promised (``ops.loss_backward_scale``).
    dH is this rank's partial sum over its vocabulary slice; the backward of the sequence gather that produced ``h``
    sums the ranks' parts."""

    @staticmethod
    def forward(ctx, h, w, labels, tp: TPInfo, ahead):
        from maester_b200.ops import cuda as C
        import maester_b200.ops.functional as Fm
        M, D = h.shape
        Vl = w.shape[0]
        v0 = tp.rank * Vl
        labels = labels.reshape(-1).to(torch.int64).contiguous()
        nvalid = (labels != -100).sum().clamp_min(1).to(torch.float32)
        gs = (1.0 / nvalid).reshape(1)
        need = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
        ahead = ahead if need else None
        gsl = gs * (ahead if ahead is not None else 1.0)
        loss_sum = torch.zeros(1, device=h.device, dtype=torch.float32)
        ex = _record_exchange(tp, M, h.device)
        rec, peers = ex.next_half()
        mg = getattr(w, "main_grad", None)
        grads, dh, dw = [], None, None
        if ahead is not None:
            dh = torch.zeros(M, D, device=h.device, dtype=torch.float32)   # fp32: the GEMM may cut the long contraction
            dw = mg if mg is not None else torch.zeros(w.shape, device=w.device, dtype=torch.float32)
        rows = Fm.CE_CHUNK_ROWS
        buf = torch.empty(min(M, rows), Vl, device=h.device, dtype=torch.bfloat16) if ahead is not None else None
        for r0 in range(0, M, rows):
            r1 = min(M, r0 + rows)
            logits, stats, tgt = C.gemm_ce(h[r0:r1], w, labels[r0:r1], v0, 1.0,
                                           logits=None if buf is None else buf[: r1 - r0], store_logits=need)
            C.ce_merge(stats, tgt, rec[r0:r1])
            ex.buf.barrier()     # every rank's records of this chunk are written
            C.ce_grad(logits, labels[r0:r1], [p + r0 * 16 for p in peers], loss_sum, gsl, v0, need, rows=r1 - r0)
            if ahead is not None:
                C.gemm(logits, w, b_mn=True, out=dh[r0:r1], epi=C.EPI_F32_ACC)
                C.gemm(logits, h[r0:r1], a_mn=True, b_mn=True, out=dw, epi=C.EPI_F32_ACC)
            elif need:
                grads.append(logits)
        ctx.tp, ctx.ahead, ctx.has_mg = tp, ahead, mg is not None
        if ahead is not None:
            ctx.save_for_backward(dh.to(h.dtype), *(() if mg is not None else (dw,)))
        else:
            ctx.save_for_backward(h, w, *grads)
        return (loss_sum * gs).reshape(())

    @staticmethod
    def backward(ctx, gout):
        from maester_b200.ops import cuda as C
        import maester_b200.ops.functional as Fm
        if ctx.ahead is not None:
            dh, *rest = ctx.saved_tensors
            C.expect_scalar(gout.detach().reshape(1).to(torch.float32).contiguous(), ctx.ahead)
            return dh, (None if ctx.has_mg else rest[0].to(dh.dtype)), None, None, None
        h, w, *grads = ctx.saved_tensors
        dh = torch.zeros(h.shape, device=h.device, dtype=torch.float32)
        mg = getattr(w, "main_grad", None)
        dw = mg if mg is not None else torch.zeros(w.shape, device=w.device, dtype=torch.float32)
        scale = gout.detach().to(torch.float32).reshape(1).contiguous()
        r0 = 0
        for g in grads:
            r1 = r0 + g.shape[0]
            C.gemm(g, w, b_mn=True, out=dh[r0:r1], epi=C.EPI_F32_ACC, alpha_dev=scale)
            C.gemm(g, h[r0:r1], a_mn=True, b_mn=True, out=dw, epi=C.EPI_F32_ACC, alpha_dev=scale)
            r0 = r1
        return dh.to(h.dtype), (None if mg is not None else dw.to(w.dtype)), None, None, None


def vocab_parallel_cross_entropy(h: torch.Tensor, w_local: torch.Tensor, labels: torch.Tensor, tp: TPInfo):
    from maester_b200 import ops
    from maester_b200.parallel.symm import symmetric_memory_available
    h2 = h.reshape(-1, h.shape[-1])
    if (ops.use_native(h2, w_local) and w_local.shape[0] % 8 == 0 and h2.shape[1] % 8 == 0 and tp.size <= 8
            and symmetric_memory_available(tp.group)):
        import maester_b200.ops.functional as Fm
        return _VocabParallelCENative.apply(h2.contiguous(), w_local, labels, tp, Fm._BACKWARD_SCALE)
    return _VocabParallelCE.apply(h2, w_local, labels, tp)


# ------------------------------------------------------------------------------ applying the plan
def _reshape_linear(lin: nn.Module, out_features: int, in_features: int, tp_dim: int) -> None:
    """Replace the weight by this rank's slice; ``tp_dim`` (0: output rows, 1: input columns) is kept on
    the parameter so that checkpoints can describe the tensor-parallel layout."""
    lin.weight = nn.Parameter(torch.empty(out_features, in_features, device=lin.weight.device,
                                          dtype=lin.weight.dtype))
    lin.weight.tp_dim = tp_dim
    lin.in_features, lin.out_features = in_features, out_features


def apply_tp(model: nn.Module, parallel_dims, cfg) -> None:
    """Shard a Llama-family ``Transformer`` or a Gemma text model over the ``tp`` mesh dimension (model still on
    meta)."""
    from maester_b200.models.llama.model import Transformer

    group = parallel_dims.mesh_group("tp")
    tp = TPInfo(group, dist.get_world_size(group), dist.get_rank(group), parallel_dims.loss_parallel_enabled)
    from maester_b200.models.gemma.model import GemmaTextModel
    inner = getattr(model, "language_model", model)
    if isinstance(inner, GemmaTextModel):
        return _apply_tp_gemma(inner, tp, cfg)
    if not isinstance(model, Transformer):
        raise NotImplementedError(
            f"tensor parallelism is implemented for the Llama and Gemma families; got {type(model).__name__}")
    a = model.model_args
    n_kv = a.n_kv_heads or a.n_heads
    assert a.n_heads % tp.size == 0 and n_kv % tp.size == 0, "heads must divide by the TP degree"
    # only an untied head is split over the vocabulary; a tied one is replicated and scores token slices
    assert a.tied_embeddings or a.vocab_size % tp.size == 0, "vocabulary must divide by the TP degree"
    fused = None
    from maester_b200.parallel.fused_tp import FusedTP, fused_tp_available
    from maester_b200.utils import device_for_training
    if getattr(cfg, "fused_collectives", False) and fused_tp_available(tp, device_for_training()):
        fused = FusedTP(tp)  # GEMM + reduce-scatter kernels over peer memory
    for layer in model.layers.values():
        att, ff = layer.attention, layer.feed_forward
        hd = att.head_dim
        att.n_heads //= tp.size
        att.n_kv_heads //= tp.size
        _reshape_linear(att.wq, att.n_heads * hd, a.dim, 0)
        _reshape_linear(att.wk, att.n_kv_heads * hd, a.dim, 0)
        _reshape_linear(att.wv, att.n_kv_heads * hd, a.dim, 0)
        _reshape_linear(att.wo, a.dim, att.n_heads * hd, 1)
        hidden = ff.w1.out_features
        assert hidden % tp.size == 0
        _reshape_linear(ff.w1, hidden // tp.size, a.dim, 0)
        _reshape_linear(ff.w3, hidden // tp.size, a.dim, 0)
        _reshape_linear(ff.w2, a.dim, hidden // tp.size, 1)
        layer.tp = tp
        if fused is not None:
            att.tp_fused = ff.tp_fused = fused
        for norm in (layer.attention_norm, layer.ffn_norm):
            for p in norm.parameters():
                p.tp_replicated = True
    if not a.tied_embeddings:
        _reshape_linear(model.output, a.vocab_size // tp.size, a.dim, 0)
    model.tok_embeddings.weight.tp_replicated = True
    for p in model.norm.parameters():
        p.tp_replicated = True
    model.tp = tp
    logger.info(f"Applied tensor parallelism (degree {tp.size}, sequence parallel, "
                f"loss parallel={tp.loss_parallel}, fused GEMM+reduce-scatter={fused is not None})")


def qkv_segments(n_heads: int, n_kv_heads: int, head_dim: int, tp_size: int, tp_rank: int):
    """Row ranges ``((first row, rows), ...)`` of the fused ``[q heads | k heads | v heads]`` projection that belong
    to one tensor-parallel rank: its query heads, its key heads and its value heads (a head-group-aware split: a rank
    holds the query heads that attend to its own key / value heads)."""
    q, kv = n_heads // tp_size * head_dim, n_kv_heads // tp_size * head_dim
    q_all, kv_all = n_heads * head_dim, n_kv_heads * head_dim
    return ((tp_rank * q, q), (q_all + tp_rank * kv, kv), (q_all + kv_all + tp_rank * kv, kv))


def _apply_tp_gemma(model, tp: TPInfo, cfg=None) -> None:
    """Shard a Gemma text model over the ``tp`` group (model still on meta).  The reference's plan for this family
    (maester/parallelisms/parallelize_gemma.py:77-178) column-shards the fused ``qkv_proj`` as one matrix, which mixes
    query, key and value heads across ranks; here every rank takes its query heads and the key / value heads they
    attend to (``qkv_segments``), ``o_proj`` and ``down_proj`` are row-parallel, ``gate_proj`` / ``up_proj``
    column-parallel, the four block norms, the QK-norms, the final norm and the tied embedding / head are replicated
    and work on this rank's token rows (sequence parallel).  With ``fused_collectives`` on a CUDA device the
    all-gathers and reduce-scatters live inside the blocks' GEMM kernels (``fused_tp``), else they are the process
    group's."""
    fused = None
    from maester_b200.parallel.fused_tp import FusedTP, fused_tp_available
    from maester_b200.utils import device_for_training
    if getattr(cfg, "fused_collectives", False) and fused_tp_available(tp, device_for_training()):
        fused = FusedTP(tp)
    cfg = model.config
    H, KV, hd = cfg.n_heads, cfg.num_key_value_heads, cfg.head_dim
    assert H % tp.size == 0 and KV % tp.size == 0, "query and key / value heads must divide by the TP degree"
    assert cfg.intermediate_size % tp.size == 0
    for layer in model.model.layers:
        att, mlp = layer.self_attn, layer.mlp
        att.num_heads, att.num_kv_heads = H // tp.size, KV // tp.size
        att.q_size, att.kv_size = att.num_heads * hd, att.num_kv_heads * hd
        _reshape_linear(att.qkv_proj, att.q_size + 2 * att.kv_size, cfg.dim, 0)
        att.qkv_proj.weight.tp_segments = qkv_segments(H, KV, hd, tp.size, tp.rank)
        _reshape_linear(att.o_proj, cfg.dim, att.q_size, 1)
        _reshape_linear(mlp.gate_proj, cfg.intermediate_size // tp.size, cfg.dim, 0)
        _reshape_linear(mlp.up_proj, cfg.intermediate_size // tp.size, cfg.dim, 0)
        _reshape_linear(mlp.down_proj, cfg.dim, cfg.intermediate_size // tp.size, 1)
        layer.tp = tp
        if fused is not None:
            att.tp_fused = mlp.tp_fused = fused
        for norm in (layer.input_layernorm, layer.post_attention_layernorm, layer.pre_feedforward_layernorm,
                     layer.post_feedforward_layernorm, att.query_norm, att.key_norm):
            if norm is not None:
                for p in norm.parameters():
                    p.tp_replicated = True
    model.tok_embeddings.weight.tp_replicated = True
    for p in model.model.norm.parameters():
        p.tp_replicated = True
    model.tp = tp
    logger.info(f"Applied tensor parallelism to the Gemma model (degree {tp.size}, sequence parallel, head-group split "
                f"of qkv_proj, replicated tied head, fused collective GEMMs={fused is not None})")


# ------------------------------------------------------------------------------ checkpoints / tests
_COLWISE = ("attention.wq.", "attention.wk.", "attention.wv.", "feed_forward.w1.", "feed_forward.w3.", "output.",
            "mlp.gate_proj.", "mlp.up_proj.")
_ROWWISE = ("attention.wo.", "feed_forward.w2.", "self_attn.o_proj.", "mlp.down_proj.")


def tp_slice_state_dict(full_state: dict[str, torch.Tensor], tp_size: int, tp_rank: int,
                        heads: tuple[int, int, int] | None = None) -> dict[str, torch.Tensor]:
    """This rank's tensor-parallel slices of an unsharded state dict (column-parallel weights split on dim 0,
    row-parallel on dim 1, everything else replicated).  ``heads = (query heads, key / value heads, head size)`` is
    needed for a fused ``qkv_proj`` (Gemma), which is split by head groups."""
    out = {}
    for k, v in full_state.items():
        if "qkv_proj." in k and v.dim() == 2:
            assert heads is not None, "qkv_proj needs the head counts"
            out[k] = torch.cat([v[a:a + n] for a, n in qkv_segments(*heads, tp_size, tp_rank)]).contiguous()
        elif any(t in k for t in _COLWISE) and v.dim() == 2:
            out[k] = v.chunk(tp_size, dim=0)[tp_rank].contiguous()
        elif any(t in k for t in _ROWWISE) and v.dim() == 2:
            out[k] = v.chunk(tp_size, dim=1)[tp_rank].contiguous()
        else:
            out[k] = v
    return out
