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


def _ce_worker(rank, world, port, out_dir):
    """Loss-parallel cross-entropy on the native kernels (records exchanged through symmetric memory) against the
    fp32 definition over the whole vocabulary; stored and produced-during-forward gradients; repeated calls."""
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from maester_b200 import ops
        from maester_b200.ops import cuda as C
        from maester_b200.ops import reference as ref
        import maester_b200.ops.functional as Fm
        from maester_b200.parallel.tensor_parallel import (TPInfo, _VocabParallelCENative,
                                                            vocab_parallel_cross_entropy)
        tp = TPInfo(dist.group.WORLD, world, rank)
        Fm.CE_CHUNK_ROWS = 256
        M, D, V = 700, 256, 4000
        Vl = V // world
        g = torch.Generator(device="cuda").manual_seed(11)       # same tensors on every rank
        worst = 0.0
        for call in range(4):
            h = torch.randn(M, D, device="cuda", generator=g).to(torch.bfloat16).requires_grad_()
            wfull = (torch.randn(V, D, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
            labels = torch.randint(0, V, (M,), device="cuda", generator=g)
            labels[::6] = -100
            w = wfull[rank * Vl:(rank + 1) * Vl].clone().requires_grad_()
            ahead = 0.5 if call % 2 else None
            with ops.loss_backward_scale(ahead):
                loss = vocab_parallel_cross_entropy(h, w, labels, tp)
            assert isinstance(loss.grad_fn, _VocabParallelCENative._backward_cls), "the native path did not run"
            (loss * 0.5).backward()
            # every rank holds the part of dH that belongs to its vocabulary slice (in the model the backward of
            # the sequence gather sums the parts)
            dh = h.grad.float()
            dist.all_reduce(dh)
            h.grad = dh.to(h.dtype)
            hf, wf = h.detach().float().requires_grad_(), wfull.float().requires_grad_()
            want = ref.linear_cross_entropy(hf, wf, labels, 1.0)
            (want * 0.5).backward()
            rel = lambda a, b: ((a.float() - b).norm() / b.norm()).item()
            errs = (abs(loss.item() - want.item()), rel(h.grad, hf.grad), rel(w.grad, wf.grad[rank * Vl:(rank + 1) * Vl]))
            assert errs[0] < 2e-2 and errs[1] < 2e-2 and errs[2] < 2e-2, (call, errs)
            worst = max(worst, *errs)
        C.check_status()
        torch.save(worst, os.path.join(out_dir, f"ce{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_loss_parallel_cross_entropy_exchanges_records_through_peer_memory(tmp_path):
    import torch.multiprocessing as mp
    from test_parallel_cpu import _free_port
    mp.spawn(_ce_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert all(torch.load(os.path.join(tmp_path, f"ce{r}.pt")) < 2e-2 for r in range(2))
