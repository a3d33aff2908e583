"""Expert parallelism for the MoE block (reference: maester/parallelisms/expert_parallel.py).

``apply_ep`` gives every rank of the ``ep`` group ``E / ep`` consecutive experts (the reference's
``Shard(0)`` on the expert dimension, :135-140) and installs a dispatcher on each MoE block:

* dispatch: the routing slots are already in expert-major order, hence contiguous per destination
  rank; per-expert counts are exchanged, then the rows (reference ``_token_dispatch`` :71-133).  The
  received rows arrive source-rank-major and are permuted to local-expert-major with every group
  padded to the grouped-GEMM tile height (``generate_permute_indices``).
* combine: inverse permutation and the reverse exchange (reference ``_token_combine`` :143-154).

Two dispatchers share that contract:

``AllToAllDispatcher``
    ``all_to_all_single`` with split sizes read back to the host (one synchronisation per MoE block,
    as in the reference).  Works on any backend; it is the CPU path and the oracle.
``PeerDispatcher`` (see ``peer_dispatch.py``)
    rows are written straight into the destination GPU's symmetric buffer by a kernel that computes
    its offsets from the all-gathered count matrix on the device: no host synchronisation.

Tensor parallelism of the experts (reference ``TensorParallel`` :23-59, ``ExpertTensorParallel``
:167-213) shards the hidden dimension: ``w1``/``w3`` by columns, ``w2`` by rows, inputs replicated over
``tp`` and the block output summed over ``tp``.  ``ReordererSequenceParallel`` (:218-278, defined but
unused there) splits the routing work of replicated tokens over the TP ranks.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn

from maester_b200.models.moe.kernels import generate_permute_indices
from maester_b200.ops.functional import GROUP_ALIGN


@dataclass
class EPInfo:
    group: object
    size: int
    rank: int
    peer_dispatcher: object = None


class _AllToAll(torch.autograd.Function):
    """Row exchange with per-rank split sizes; the backward is the exchange with the splits swapped."""

    @staticmethod
    def forward(ctx, x, in_splits, out_splits, group):
        ctx.meta = (in_splits, out_splits, group)
        out = x.new_empty(sum(out_splits), *x.shape[1:])
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        in_splits, out_splits, group = ctx.meta
        gin = g.new_empty(sum(in_splits), *g.shape[1:])
        dist.all_to_all_single(gin, g.contiguous(), in_splits, out_splits, group=group)
        return gin, None, None, None


def permute_to_local_experts(recv: torch.Tensor, recv_counts: torch.Tensor, n_local: int, n_ranks: int):
    """Rows received rank-major/expert-minor → local-expert-major rows with padded groups.

    Returns (buffer, int32 offsets [n_local + 1], index vector used, number of received rows)."""
    n, dim = recv.shape
    max_len = (n + n_local * GROUP_ALIGN + GROUP_ALIGN - 1) // GROUP_ALIGN * GROUP_ALIGN
    perm, _, m_offsets = generate_permute_indices(recv_counts.reshape(-1), n_local, n_ranks, max_len, GROUP_ALIGN)
    idx = torch.where(perm < 0, torch.full_like(perm, n), perm).to(torch.int64)  # padding → the zero row
    from maester_b200.models.moe.moe import _UniqueRowSelect
    # indices repeat only for the zero row, whose gradient is discarded: a copy-based backward is exact
    buf = _UniqueRowSelect.apply(torch.cat([recv, recv.new_zeros(1, dim)]), idx)
    offs = torch.cat([m_offsets.new_zeros(1), m_offsets]).to(torch.int32)
    return buf, offs, idx, n


def unpermute_from_local_experts(out: torch.Tensor, idx: torch.Tensor, n: int) -> torch.Tensor:
    return out.new_zeros(n + 1, out.shape[1]).index_copy(0, idx, out)[:n]


class AllToAllDispatcher:
    def __init__(self, ep: EPInfo):
        self.ep = ep

    def __call__(self, moe, x, sorted_scores, token_idx, counts, sorted_experts):
        ep = self.ep
        n_local = moe.experts.num_local_experts
        routed_in = moe.gather_slots(x, token_idx)
        if moe.score_before_experts:
            routed_in = (routed_in.float() * sorted_scores[:, None]).to(x.dtype)
        send_counts = counts.view(ep.size, n_local).contiguous()
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts.view(-1), send_counts.view(-1), group=ep.group)
        host = torch.stack([send_counts.sum(1), recv_counts.sum(1)]).cpu()  # the one host synchronisation
        in_splits, out_splits = host[0].tolist(), host[1].tolist()
        recv = _AllToAll.apply(routed_in, in_splits, out_splits, ep.group)
        buf, offs, idx, n = permute_to_local_experts(recv, recv_counts, n_local, ep.size)
        out = unpermute_from_local_experts(moe.experts(buf, offs), idx, n)
        routed_out = _AllToAll.apply(out, out_splits, in_splits, ep.group)
        if not moe.score_before_experts:
            routed_out = (routed_out.float() * sorted_scores[:, None]).to(x.dtype)
        return routed_out


# ---------------------------------------------------------------------------------------------------
# installing expert parallelism
def _moe_blocks(model: nn.Module):
    from maester_b200.models.moe.moe import MoE
    return [m for m in model.modules() if isinstance(m, MoE)]


def _local_param(old: nn.Parameter, sl: tuple) -> nn.Parameter:
    """The slice ``old[sl]`` as a new leaf parameter (shape-only on the meta device)."""
    if old.device.type == "meta":
        shape = torch.empty(old.shape, device="meta")[sl].shape
        new = nn.Parameter(torch.empty(shape, device="meta", dtype=old.dtype), requires_grad=old.requires_grad)
    else:
        new = nn.Parameter(old.data[sl].clone(), requires_grad=old.requires_grad)
    for attr in ("ep_local", "tp_replicated"):
        if getattr(old, attr, False):
            setattr(new, attr, True)
    if hasattr(old, "tp_dim"):
        new.tp_dim = old.tp_dim
    return new


def apply_ep(model: nn.Module, parallel_dims, use_peer_memory: bool = False, capacity_factor: float = 2.0) -> EPInfo:
    """Keep ``E / ep`` experts per rank and route tokens between ranks (call before sharding)."""
    group = parallel_dims.mesh_group("ep")
    assert group is not None, "expert parallelism needs an 'ep' mesh dimension of size > 1"
    ep = EPInfo(group, dist.get_world_size(group), dist.get_rank(group))
    shared = None
    if use_peer_memory:  # one dispatcher for all blocks: they run one after another and share the workspaces
        from maester_b200.parallel.peer_dispatch import PeerDispatcher
        shared = PeerDispatcher(ep, capacity_factor)
    for moe in _moe_blocks(model):
        ex = moe.experts
        assert ex.num_experts % ep.size == 0, f"{ex.num_experts} experts do not divide over ep={ep.size}"
        n_local = ex.num_experts // ep.size
        rows = slice(ep.rank * n_local, (ep.rank + 1) * n_local)
        for name in ("w1", "w2", "w3"):
            new = _local_param(getattr(ex, name), (rows,))
            new.ep_local = True
            setattr(ex, name, new)
        ex.num_local_experts, ex.ep_rank, ex.ep_size = n_local, ep.rank, ep.size
        moe.dispatcher = shared if shared is not None else AllToAllDispatcher(ep)
    model.ep = ep
    ep.peer_dispatcher = shared  # None with the all-to-all dispatcher (which never drops rows)
    return ep


# ---------------------------------------------------------------------------------------------------
# tensor parallelism of the MoE block
class _CopyToTP(torch.autograd.Function):
    """Identity forward; the input gradient is the sum of the ranks' partial gradients."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    """Sum of the ranks' partial outputs forward; identity backward."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def apply_expert_tp(model: nn.Module, parallel_dims) -> None:
    """Shard the hidden dimension of routed and shared experts over ``tp``; the router stays replicated
    (reference ``NoParallel``, expert_parallel.py:285-330) and its gradient is summed over ``tp``.
    Works alone (TP-only experts) or after ``apply_ep`` (experts split over ep, each split by tp)."""
    group = parallel_dims.mesh_group("tp")
    size, rank = dist.get_world_size(group), dist.get_rank(group)
    for moe in _moe_blocks(model):
        ex = moe.experts
        hidden = ex.w1.shape[2]
        assert hidden % size == 0
        h = hidden // size
        cols = slice(rank * h, (rank + 1) * h)
        ex.w1 = _local_param(ex.w1, (slice(None), slice(None), cols))
        ex.w3 = _local_param(ex.w3, (slice(None), slice(None), cols))
        ex.w2 = _local_param(ex.w2, (slice(None), cols))
        ex.w1.tp_dim, ex.w3.tp_dim, ex.w2.tp_dim = 2, 2, 1  # which dimension the checkpoint reassembles over tp
        sh = moe.shared_experts
        if sh is not None:
            hs = sh.w1.weight.shape[0]
            assert hs % size == 0
            r = slice(rank * hs // size, (rank + 1) * hs // size)
            sh.w1.weight = _local_param(sh.w1.weight, (r,))
            sh.w3.weight = _local_param(sh.w3.weight, (r,))
            sh.w2.weight = _local_param(sh.w2.weight, (slice(None), r))
            sh.w1.weight.tp_dim, sh.w3.weight.tp_dim, sh.w2.weight.tp_dim = 0, 0, 1
            from maester_b200.models.layers import FusedWeight
            sh._w13 = FusedWeight([sh.w1, sh.w3])
        moe.router.gate.weight.tp_replicated = True
        moe.tp_group = group


class ReordererSequenceParallel:
    """Split the routing slots of TP-replicated tokens over the TP ranks before dispatch and put them
    back afterwards, so that with unsharded experts each TP rank sends a distinct 1/tp of the slots
    (reference: expert_parallel.py:218-278, where it is defined but not wired in).

    ``split`` keeps rows ``[rank*n/tp, (rank+1)*n/tp)`` of the T*k slot arrays (token indices are kept
    global); ``merge`` all-gathers the per-rank routed outputs back into slot order."""

    def __init__(self, group):
        self.group = group
        self.size, self.rank = dist.get_world_size(group), dist.get_rank(group)

    def split(self, top_scores: torch.Tensor, selected: torch.Tensor):
        n = top_scores.shape[0]
        assert n % self.size == 0, "token count must divide by the TP degree"
        c = n // self.size
        sl = slice(self.rank * c, (self.rank + 1) * c)
        return top_scores[sl], selected[sl], self.rank * c

    def merge(self, routed_out: torch.Tensor) -> torch.Tensor:
        out = routed_out.new_empty(self.size * routed_out.shape[0], *routed_out.shape[1:])
        dist.all_gather_into_tensor(out.view(-1), routed_out.contiguous().view(-1), group=self.group)
        return out
