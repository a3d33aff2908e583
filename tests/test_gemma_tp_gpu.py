"""Gemma under tensor parallelism on 2 GPUs (native kernels, NCCL collectives) follows the single-GPU run."""
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
        from test_parallel_cpu import GEMMA_HEADS, _gemma_cfg, _load_full
        from maester_b200.ops import cuda as C
        from maester_b200.trainer import Trainer
        tr = Trainer(_gemma_cfg(tensor_parallel_degree=2, data_parallel_shard_degree=1, seq_len=256, ac_mode="selective",
                                fused_collectives=fused))
        assert (tr.model.model.layers[0].self_attn.tp_fused is not None) == fused
        _load_full(tr, full, tp=(2, rank, GEMMA_HEADS))
        before = C.launch_count
        losses = [tr.train_step(b).item() for b in batches]
        C.check_status()
        assert C.launch_count > before, "native kernels did not run"
        params = {sl.fqn: sl.param.data.float().cpu() for u in tr.sharded.units for sl in u.slots}
        torch.save((losses, params), os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("fused", [False, True], ids=["nccl", "fused_gemms"])
def test_gemma_tensor_parallel_follows_the_single_gpu_run(tmp_path, fused):
    import torch.multiprocessing as mp
    from test_parallel_cpu import GEMMA_HEADS, _batches, _free_port, _full_weights, _gemma_cfg, _load_full
    from maester_b200.parallel.tensor_parallel import tp_slice_state_dict
    from maester_b200.trainer import Trainer
    full = _full_weights(_gemma_cfg(seq_len=256))
    g = torch.Generator().manual_seed(7)
    for k, v in full.items():
        if "norm" in k:
            v.copy_(0.2 * torch.randn(v.shape, generator=g))
    batches = _batches(3, 2, 256, 512)
    mp.spawn(_worker, args=(2, _free_port(), full, batches, fused, str(tmp_path)), nprocs=2, join=True)
    os.environ.pop("WORLD_SIZE", None)
    os.environ.pop("RANK", None)
    tr = Trainer(_gemma_cfg(seq_len=256, ac_mode="selective"))
    _load_full(tr, full)
    want_losses = [tr.train_step({k: v.cuda() for k, v in b.items()}).item() for b in batches]
    want_params = {sl.fqn: sl.param.data.float().cpu() for u in tr.sharded.units for sl in u.slots}
    for r in range(2):
        losses, params = torch.load(os.path.join(tmp_path, f"r{r}.pt"))
        assert losses == pytest.approx(want_losses, abs=3e-2), (losses, want_losses)
        want = tp_slice_state_dict(want_params, 2, r, GEMMA_HEADS)
        for k in want:
            err = ((params[k] - want[k]).norm() / (want[k].norm() + 1e-12)).item()
            assert err < 2e-2, (k, err)
