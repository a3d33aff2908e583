"""Permutation indices for expert-parallel token exchange.

``generate_permute_indices`` maps tokens received rank-major / expert-minor (the order an
all-to-all delivers them) to expert-major order with every local expert's group padded to
``alignment`` rows; it returns the index vector (−1 marks padding), the padded group sizes and their
exclusive offsets.  Same contract as the reference (maester/models/moe/kernels.py:139-212), whose
Triton kernel this replaces with a vectorised device computation (no host synchronisation) plus a
straightforward loop version used as the oracle in tests.
"""
from __future__ import annotations

import torch


def fill_indices_cpu(tokens_per_expert_group: torch.Tensor, start_index_values: torch.Tensor,
                     write_offsets: torch.Tensor, experts_per_rank: int, num_ranks: int,
                     max_len: int) -> torch.Tensor:
    """Loop oracle: for local expert e, concatenate its chunks from rank 0..R-1."""
    out = torch.full((max_len,), -1, dtype=torch.int32)
    for e in range(experts_per_rank):
        w = int(write_offsets[e])
        for r in range(num_ranks):
            i = r * experts_per_rank + e
            s, n = int(start_index_values[i]), int(tokens_per_expert_group[i])
            if n > 0:
                out[w:w + n] = torch.arange(s, s + n, dtype=torch.int32)
                w += n
    return out


def generate_permute_indices(tokens_per_expert_group: torch.Tensor, experts_per_rank: int, num_ranks: int,
                             max_len: int, alignment: int, use_cpu: bool = False):
    """tokens_per_expert_group: [num_ranks * experts_per_rank] counts in rank-major order.

    Returns (permuted_indices [max_len] int32, m_sizes [experts_per_rank] int32, m_offsets [experts_per_rank] int32
    inclusive cumulative sum of m_sizes, as the reference returns).
    """
    t = tokens_per_expert_group.to(torch.int64)
    start = t.cumsum(0) - t                                         # where each (rank, expert) chunk starts
    per_expert = t.view(num_ranks, experts_per_rank).sum(0)         # total per local expert
    m_sizes = (torch.clamp_min(per_expert, alignment) + alignment - 1) // alignment * alignment
    m_offsets = m_sizes.cumsum(0)
    write = m_offsets - m_sizes
    if use_cpu:
        perm = fill_indices_cpu(t.cpu(), start.cpu(), write.cpu(), experts_per_rank, num_ranks, max_len)
        return perm.to(tokens_per_expert_group.device), m_sizes.to(torch.int32), m_offsets.to(torch.int32)
    dev = t.device
    # chunk (r, e) lands at write[e] + sum_{r' < r} t[r', e]
    tv = t.view(num_ranks, experts_per_rank)
    within = tv.cumsum(0) - tv
    chunk_dst = (write[None, :] + within).reshape(-1)
    total = int(max_len)
    pos = torch.arange(total, device=dev)
    # for every source token position find its chunk by searching the chunk starts
    n_src = t.sum()
    chunk_of = torch.searchsorted(start + t, pos, right=True).clamp_max(t.numel() - 1)
    dst = chunk_dst[chunk_of] + (pos - start[chunk_of])
    valid = pos < n_src
    perm = torch.full((total,), -1, dtype=torch.int32, device=dev)
    dst = torch.where(valid, dst, torch.full_like(dst, total))      # park invalid entries out of range
    perm = torch.cat([perm, perm.new_zeros(1)]).scatter(0, dst.clamp_max(total), pos.to(torch.int32))[:total]
    return perm, m_sizes.to(torch.int32), m_offsets.to(torch.int32)
