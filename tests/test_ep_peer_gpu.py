"""Expert parallelism over peer memory (2 GPUs): same losses and weights as the all-to-all dispatcher."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _rank(rank, world, full, batches, peer, flavor):
    import torch.distributed as dist
    from test_expert_parallel_cpu import _cfg, _gather_params, _load
    from maester_b200.trainer import Trainer
    tr = Trainer(_cfg(data_parallel_shard_degree=world, expert_parallel_degree=world, ep_peer_dispatch=peer,
                      fused_collectives=False, flavor=flavor))
    _load(tr, full)
    losses = []
    for b in batches:
        mine = {k: v[tr.dp_rank * 2:(tr.dp_rank + 1) * 2] for k, v in b.items()}
        losses.append(tr.train_step(mine).item())
    dropped = 0
    if peer:
        from maester_b200.models.moe.moe import MoE
        d = next(m.dispatcher for m in tr.model.modules() if isinstance(m, MoE))
        dropped = d.dropped()
    from maester_b200.ops import cuda as C
    C.check_status()
    return losses, {k: (v[0].float().cpu(), v[1], v[2]) for k, v in _gather_params(tr).items()}, dropped


def _worker(rank, world, port, full, batches, peer, out_dir, flavor):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        torch.save(_rank(rank, world, full, batches, peer, flavor), os.path.join(out_dir, f"r{rank}_{int(peer)}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("native_routing,flavor", [("1", "debug_flex"), ("0", "debug_flex"),
                                                   ("1", "debug_flex_gate_after")])
def test_peer_dispatch_matches_all_to_all(tmp_path, native_routing, flavor, monkeypatch):
    """native_routing=1: routing plan kernels + token-indexed peer dispatch / combine (gate values applied before
    or after the experts); 0: ATen routing chain and the sorted-slot scatter / gather kernels."""
    import torch.multiprocessing as mp
    monkeypatch.setenv("MB_MOE_FUSED_ROUTE", native_routing)  # read at import time by the spawned ranks
    from test_expert_parallel_cpu import _cfg
    from test_parallel_cpu import _batches, _free_port, _full_weights
    full = _full_weights(_cfg(train_batch_size=4, flavor=flavor))
    batches = _batches(3, 4, 32, 2000)
    res = {}
    for peer in (False, True):
        mp.spawn(_worker, args=(2, _free_port(), full, batches, peer, str(tmp_path), flavor), nprocs=2, join=True)
        res[peer] = [torch.load(os.path.join(tmp_path, f"r{r}_{int(peer)}.pt"), weights_only=False) for r in range(2)]
    for r in range(2):
        a, b = res[False][r], res[True][r]
        print(f"rank {r}: all-to-all {a[0]} peer {b[0]} dropped {b[2]}")
        assert b[2] == 0
        assert a[0] == pytest.approx(b[0], abs=2e-2)
        for k in a[1]:
            x, y = a[1][k][0], b[1][k][0]
            assert ((x - y).norm() / (x.norm() + 1e-12)).item() < 2e-2, k


def _grow_worker(rank, world, port, full, batches, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from test_expert_parallel_cpu import _cfg, _load
        from maester_b200.ops import cuda as C
        from maester_b200.trainer import Trainer
        # a capacity far below the balanced load: the first step must drop rows
        tr = Trainer(_cfg(data_parallel_shard_degree=world, expert_parallel_degree=world, ep_peer_dispatch=True,
                          fused_collectives=False, flavor="debug_flex", ep_capacity_factor=0.25, seq_len=256))
        _load(tr, full)
        disp = tr.model.ep.peer_dispatcher
        mine = lambda b: {k: v[tr.dp_rank * 2:(tr.dp_rank + 1) * 2] for k, v in b.items()}
        tr.train_step(mine(batches[0]))
        cap0 = disp.cap
        dropped0 = tr.pop_dropped_rows()          # reads the counter, then grows the buffers (collective)
        cap1 = disp.cap
        tr.train_step(mine(batches[1]))
        dropped1 = tr.pop_dropped_rows()
        tr.train_step(mine(batches[2]))
        dropped2 = tr.pop_dropped_rows()
        C.check_status()
        torch.save((cap0, cap1, disp.cap, dropped0, dropped1, dropped2), os.path.join(out_dir, f"g{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_peer_dispatch_grows_its_buffers_when_the_load_outgrows_them(tmp_path):
    import torch.multiprocessing as mp
    from test_expert_parallel_cpu import _cfg
    from test_parallel_cpu import _batches, _free_port, _full_weights
    full = _full_weights(_cfg(train_batch_size=4, flavor="debug_flex", seq_len=256))
    batches = _batches(3, 4, 256, 2000)   # 1536 routing slots per rank against 896 buffer rows
    mp.spawn(_grow_worker, args=(2, _free_port(), full, batches, str(tmp_path)), nprocs=2, join=True)
    out = [torch.load(os.path.join(tmp_path, f"g{r}.pt"), weights_only=False) for r in range(2)]
    assert out[0][:3] == out[1][:3]                       # every rank made the same decision
    cap0, cap1, cap2, d0, d1, d2 = out[0]
    assert sum(o[3] for o in out) > 0                     # the undersized buffers dropped rows ...
    assert cap1 > cap0                                    # ... and were reallocated at the first read of the counter
    assert all(o[4] == 0 and o[5] == 0 for o in out)      # nothing is dropped afterwards
