"""Two-GPU check of ring context parallelism: zig-zag shards with the peers' K / V pulled over NVLink by this library's
copy kernel, partial results merged by log-sum-exp, dK / dV contributions returned through symmetric memory.  Must train
like the all-to-all form (which runs the unchanged attention kernel over the whole sequence)."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ADAMW = [{"opt_class": "torch.optim.AdamW", "opt_cfg": {"lr": 1e-3, "betas": (0.9, 0.95), "weight_decay": 0.0},
          "min_dim": 0}]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir, batch):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from maester_b200.config import Config
    from maester_b200.datasets.synthetic import SyntheticLoader
    from maester_b200.ops import cuda as C
    from maester_b200.trainer import Trainer
    out = {}
    for mode in ("alltoall", "ring"):
        torch.manual_seed(0)
        cfg = Config(model_name="llama3", flavor="debugmodel", seq_len=1024, train_batch_size=batch,
                     data_parallel_shard_degree=1, context_parallel_degree=world, context_parallel_mode=mode,
                     ac_mode="none", enable_checkpoint=False, optimizer_groups=ADAMW, scheduler="constant",
                     synthetic_vocab_size=2048,
                     fused_collectives=False)  # NCCL reduce-scatter: the reduced gradient shards can be compared
        tr = Trainer(cfg)
        loader = SyntheticLoader(batch, 1024, 2048, "full", seed=5, rank=0)   # the CP group shares one batch
        # gradients of the first step (reduced over the group, this rank's rows) before any optimizer arithmetic
        tr.optimizers.zero_grad()
        tr.forward_backward(next(loader))
        g0 = tr.sharded.shard_grad.clone()
        losses = [tr.train_step(next(loader)).item() for _ in range(4)]
        C.check_status()
        out[mode] = (losses, tr.sharded.master.clone(), g0)
        del tr
    rel = ((out["ring"][1] - out["alltoall"][1]).norm() / out["alltoall"][1].norm()).item()
    rel_g = ((out["ring"][2] - out["alltoall"][2]).norm() / out["alltoall"][2].norm()).item()
    torch.save((out["alltoall"][0], out["ring"][0], rel, rel_g), os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("batch", [2, 1])   # batch 1: the chunks of a rank's sequence are views, not copies
def test_ring_context_parallel_trains_like_the_all_to_all_form(batch):
    world = 2
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(world, _free_port(), d, batch), nprocs=world, join=True)
        a2a = [torch.load(os.path.join(d, f"r{r}.pt"), weights_only=False) for r in range(world)]
        # the two forms shard the sequence differently, so compare the mean loss over the CP group
        mean_a2a = [sum(a2a[r][0][i] for r in range(world)) / world for i in range(4)]
        mean_ring = [sum(a2a[r][1][i] for r in range(world)) / world for i in range(4)]
        assert mean_ring == pytest.approx(mean_a2a, abs=2e-2)
        for r in range(world):
            assert a2a[r][3] < 1.5e-2, ("gradients", a2a[r][3])   # bf16 kernels, different summation order
            assert a2a[r][2] < 1e-2, ("weights after four Adam steps", a2a[r][2])
