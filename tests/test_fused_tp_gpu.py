"""Tensor parallelism with GEMM + reduce-scatter fused over peer memory (2 GPUs) equals the NCCL path."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, full, batches, fused, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from test_parallel_cpu import _cfg, _load_full
        from maester_b200.ops import cuda as C
        from maester_b200.trainer import Trainer
        tr = Trainer(_cfg(tensor_parallel_degree=2, data_parallel_shard_degree=1, fused_collectives=fused, seq_len=256))
        assert (tr.model.layers["0"].attention.tp_fused is not None) == fused
        _load_full(tr, full, tp=(2, rank))
        losses = [tr.train_step(b).item() for b in batches]
        C.check_status()
        params = {sl.fqn: sl.param.data.float().cpu() for u in tr.sharded.units for sl in u.slots}
        torch.save((losses, params), os.path.join(out_dir, f"r{rank}_{int(fused)}.pt"))
    finally:
        dist.destroy_process_group()


def _ag_worker(rank, world, port, out_dir):
    """all-gather fused into the GEMM kernel against NCCL all-gather + fp32 matmul, several calls in a row."""
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from maester_b200.ops import cuda as C
        from maester_b200.parallel.fused_tp import FusedTP, _all_gather_rows
        from maester_b200.parallel.tensor_parallel import TPInfo
        tp = TPInfo(dist.group.WORLD, world, rank)
        worst = 0.0
        for (Ml, K, N, b_mn, copiers) in [(256, 512, 384, False, 1), (1024, 1024, 768, True, 2),
                                          (2048, 4096, 3072, False, 4), (512, 264, 136, False, 8)]:
            f = FusedTP(tp)
            f.ag_mode, f.ag_copiers = "fused", copiers
            g = torch.Generator(device="cuda").manual_seed(10 * rank + 1)
            w = (torch.randn((K, N) if b_mn else (N, K), device="cuda", generator=g.manual_seed(5)) * 0.05).to(torch.bfloat16)
            g.manual_seed(10 * rank + 1)
            for call in range(5):  # both buffers of the alternating pair are reused
                x = torch.randn(Ml, K, device="cuda", generator=g).to(torch.bfloat16)
                full, y = f.ag_gemm(x, w, b_mn=b_mn)
                want_full = _all_gather_rows(x, tp)
                assert torch.equal(full, want_full), (Ml, K, call)
                want = want_full.float() @ (w.float() if b_mn else w.float().t())
                err = ((y.float() - want).norm() / want.norm()).item()
                worst = max(worst, err)
                assert err < 1e-2, (Ml, K, N, call, err)
            C.check_status()
        torch.save(worst, os.path.join(out_dir, f"ag{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_all_gather_fused_into_gemm(tmp_path):
    import torch.multiprocessing as mp
    from test_parallel_cpu import _free_port
    mp.spawn(_ag_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert all(torch.load(os.path.join(tmp_path, f"ag{r}.pt")) < 1e-2 for r in range(2))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_gemm_reduce_scatter_matches_nccl(tmp_path):
    import torch.multiprocessing as mp
    from test_parallel_cpu import _batches, _cfg, _free_port, _full_weights
    full = _full_weights(_cfg(seq_len=256))
    batches = _batches(3, 2, 256, 512)
    res = {}
    for fused in (False, True):
        mp.spawn(_worker, args=(2, _free_port(), full, batches, fused, str(tmp_path)), nprocs=2, join=True)
        res[fused] = [torch.load(os.path.join(tmp_path, f"r{r}_{int(fused)}.pt"), weights_only=False) for r in range(2)]
    for r in range(2):
        a, b = res[False][r], res[True][r]
        print(f"rank {r}: nccl {a[0]} fused {b[0]}")
        assert a[0] == pytest.approx(b[0], abs=2e-2)
        for k in a[1]:
            assert ((a[1][k] - b[1][k]).norm() / (a[1][k].norm() + 1e-12)).item() < 2e-2, k
