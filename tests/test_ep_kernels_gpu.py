"""Expert-parallel plan and row-exchange kernels (csrc/ep_comm.cu) on ONE GPU: the peer table holds local buffers,
one per emulated rank, so the kernels run exactly as over NVLink but every "peer" pointer is local memory."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


class _LocalPeers:
    """Stands in for a symmetric buffer: ``world`` separate local tensors and the pointer table the launchers take."""

    def __init__(self, world: int, numel: int):
        self.world = world
        self.tensors = [torch.full((numel,), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(world)]
        self.ptr_array = (ctypes.c_void_p * world)(*[t.data_ptr() for t in self.tensors])
        self.tensor = self.tensors[0]


def _plan_reference(allc, me, n_local, idx, inv, align):
    ep, E = allc.shape
    tot = allc.sum(0)
    padded = (tot + align - 1) // align * align
    pv = padded.view(ep, n_local)
    group_start = (pv.cumsum(1) - pv).reshape(-1)
    before = allc[:me].sum(0)
    mine = allc[me]
    start = mine.cumsum(0) - mine
    e = idx.long()
    rank = e // n_local
    row = group_start[e] + before[e] + (inv.long() - start[e])
    offs = torch.cat([pv.new_zeros(1), pv[me].cumsum(0)])
    return rank, row, offs


@pytest.mark.parametrize("ep,E,k,T", [(2, 8, 3, 500), (4, 64, 6, 1000), (1, 16, 4, 300)])
def test_ep_plan_matches_formula(ep, E, k, T):
    from maester_b200.ops import cuda as C
    n_local = E // ep
    plans = [C.moe_route(torch.randn(T, E, device="cuda"), None, k, True, False, 1.0, False, 128) for _ in range(ep)]
    allc = torch.stack([p.counts for p in plans]).contiguous()
    cap = 1 << 30
    for me, p in enumerate(plans):
        rank, row, offs = C.ep_plan(allc, me, n_local, p.idx.view(-1), p.inv, 128, cap)
        wr, wrow, woffs = _plan_reference(allc.long(), me, n_local, p.idx.view(-1), p.inv, 128)
        assert torch.equal(rank.long(), wr) and torch.equal(row.long(), wrow) and torch.equal(offs.long(), woffs)
    # all ranks together fill every destination row exactly once
    seen = {}
    for me, p in enumerate(plans):
        rank, row, _ = C.ep_plan(allc, me, n_local, p.idx.view(-1), p.inv, 128, cap)
        for r in range(ep):
            rows = row[rank == r]
            seen.setdefault(r, []).append(rows)
    for r, parts in seen.items():
        rows = torch.cat(parts)
        assert rows.unique().numel() == rows.numel()


@pytest.mark.parametrize("scaled", [False, True])
def test_dispatch_combine_slot_dot_and_padding(scaled):
    from maester_b200.ops import cuda as C
    ep, E, k, T, D = 2, 8, 3, 400, 264
    n_local = E // ep
    x = [torch.randn(T, D, device="cuda").to(torch.bfloat16) for _ in range(ep)]
    plans = [C.moe_route(torch.randn(T, E, device="cuda"), None, k, False, True, 1.0, False, 128) for _ in range(ep)]
    allc = torch.stack([p.counts for p in plans]).contiguous()
    cap = int(((allc.sum(0) + 127) // 128 * 128).view(ep, n_local).sum(1).max().item()) + 256
    peers = _LocalPeers(ep, cap * D)
    overflow = torch.zeros(1, dtype=torch.int32, device="cuda")
    routes = [C.ep_plan(allc, me, n_local, plans[me].idx.view(-1), plans[me].inv, 128, cap) for me in range(ep)]
    for me in range(ep):  # every emulated rank clears its padding and dispatches its tokens
        C.ep_zero_padding(peers.tensors[me], allc, me, n_local, routes[me][2], D, cap)
    for me in range(ep):
        rank, row, _ = routes[me]
        C.peer_dispatch_rows(x[me], peers, rank, row, plans[me].top if scaled else None, k, cap, overflow)
    assert overflow.item() == 0
    bufs = [t.view(cap, D) for t in peers.tensors]
    for me in range(ep):
        rank, row, offs = routes[me]
        gate = plans[me].top.reshape(-1) if scaled else torch.ones(T * k, device="cuda")
        want = (x[me].float().repeat_interleave(k, 0) * gate[:, None]).to(torch.bfloat16)
        got = torch.stack([bufs[int(r)][int(w)] for r, w in zip(rank[:64].tolist(), row[:64].tolist())])
        assert torch.equal(got, want[:64])
        # every row inside the groups is either a dispatched row or zero padding: nothing of the NaN fill is left
        used = bufs[me][: int(offs[-1].item())]
        assert not torch.isnan(used.float()).any()
        out = C.peer_combine_rows(peers, rank, row, plans[me].top if scaled else None, T, k, D, cap, overflow)
        ref = (want.float() * (gate[:, None] if scaled else 1.0)).view(T, k, D).sum(1)
        assert ((out.float() - ref).norm() / ref.norm()).item() < 5e-3
        g = torch.randn(T, D, device="cuda").to(torch.bfloat16)
        dots = C.peer_slot_dot(peers, rank, row, g, k, cap)
        wantd = (want.float().view(T, k, D) * g.float()[:, None, :]).sum(-1).reshape(-1)
        assert torch.allclose(dots, wantd, atol=2e-2, rtol=1e-3)
    C.check_status()
