"""Multi-process (gloo, CPU) checks of the sharding runtime, tensor parallelism and the trainer."""
import copy
import os
import socket
import sys
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from maester_b200.config import Config

# eps well above the rounding noise of fp32 gradients: with a tiny eps Adam turns noise-level gradient entries (the
# q / k projections of a freshly initialised model) into +-lr steps, and parity between two summation orders is lost
ADAMW = [{"opt_class": "torch.optim.AdamW", "opt_cfg": {"lr": 1e-3, "betas": (0.9, 0.95), "weight_decay": 0.1, "eps": 1e-4},
          "min_dim": 0}]


def _close(a, b, tol=5e-3):
    """Adam turns rounding-level gradient differences into +-lr steps on near-zero-gradient entries,
    so compare in the Frobenius norm rather than element-wise."""
    return ((a - b).norm() / (b.norm() + 1e-12)).item() < tol


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, args, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    # the ranks share the machine's cores: without a limit every rank starts one intra-op thread per core
    if world > 1:
        torch.set_num_threads(max(1, torch.get_num_threads() // world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        res = fn(rank, world, *args)
        torch.save(res, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def run_ranks(world, fn, *args):
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(world, _free_port(), fn, args, d), nprocs=world, join=True)
        return [torch.load(os.path.join(d, f"r{r}.pt"), weights_only=False) for r in range(world)]


def _cfg(**kw):
    base = dict(model_name="llama3", flavor="tiny", seq_len=64, train_batch_size=2, enable_checkpoint=False,
                synthetic_vocab_size=512, optimizer_groups=ADAMW, scheduler="constant", ac_mode="none",
                data_parallel_shard_degree=1)
    base.update(kw)
    return Config(**base)


def _full_weights(cfg):
    """Deterministic unsharded fp32 weights for the tiny model."""
    from maester_b200.trainer import build_model_args
    from maester_b200.models import model_name_to_cls
    torch.manual_seed(1234)
    args = build_model_args(cfg, cfg.synthetic_vocab_size)
    model = model_name_to_cls[cfg.model_name].from_model_args(args)
    if hasattr(model, "init_weights"):
        model.init_weights()
    return {k: v.detach().clone() for k, v in model.state_dict().items()}


def _load_full(trainer, full, tp=None):
    from maester_b200.parallel.tensor_parallel import tp_slice_state_dict
    sd = tp_slice_state_dict(full, *tp) if tp else full
    sh = trainer.sharded
    with torch.no_grad():
        for u in sh.units:
            for sl in u.slots:
                sl.param.data.copy_(sd[sl.fqn])
    sh.init_master_from_full()


def _batches(n, bs, seq, vocab, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        t = torch.randint(2, vocab, (bs, seq + 1), generator=g)
        out.append({"input_ids": t[:, :-1].contiguous(), "labels": t[:, 1:].contiguous()})
    return out


def _single(cfg, full, batches):
    from maester_b200.trainer import Trainer
    tr = Trainer(cfg)
    _load_full(tr, full)
    losses = [tr.train_step(b).item() for b in batches]
    return losses, {sl.fqn: sl.param.data.clone() for u in tr.sharded.units for sl in u.slots}


def _fsdp_rank(rank, world, cfg_kw, full, batches):
    from maester_b200.trainer import Trainer
    tr = Trainer(_cfg(**cfg_kw))
    _load_full(tr, full)
    losses = []
    for b in batches:
        mine = {k: v[rank * 2:(rank + 1) * 2] for k, v in b.items()}  # this rank's half of the global batch
        losses.append(tr.train_step(mine).item())
    return losses, {sl.fqn: sl.param.data.clone() for u in tr.sharded.units for sl in u.slots}


@pytest.mark.parametrize("mode", ["shard", "replicate"])
def test_two_rank_data_parallel_matches_single_process(mode):
    cfg1 = _cfg(train_batch_size=4)
    full = _full_weights(cfg1)
    batches = _batches(3, 4, 64, 512)
    want_losses, want_params = _single(cfg1, full, batches)
    kw = dict(data_parallel_shard_degree=2) if mode == "shard" else \
        dict(data_parallel_shard_degree=1, data_parallel_replicate_degree=2)
    res = run_ranks(2, _fsdp_rank, kw, full, batches)
    for r in range(2):
        losses, params = res[r]
        for k in want_params:
            assert _close(params[k], want_params[k]), (mode, k)
    mean_losses = [(a + b) / 2 for a, b in zip(res[0][0], res[1][0])]
    assert mean_losses == pytest.approx(want_losses, abs=1e-4)


def _tp_rank(rank, world, full, batches):
    from maester_b200.trainer import Trainer
    tr = Trainer(_cfg(tensor_parallel_degree=2, data_parallel_shard_degree=1))
    _load_full(tr, full, tp=(2, rank))
    losses = [tr.train_step(b).item() for b in batches]
    return losses, {sl.fqn: sl.param.data.clone() for u in tr.sharded.units for sl in u.slots}


def test_tensor_parallel_matches_single_process():
    from maester_b200.parallel.tensor_parallel import tp_slice_state_dict
    cfg1 = _cfg(tied_override=None) if False else _cfg()
    # the tiny flavor ties embeddings; use an untied variant so the loss-parallel path is exercised
    full = _full_weights(_cfg(flavor="debugmodel", seq_len=64))
    batches = _batches(2, 2, 64, 512)
    want_losses, want_params = _single(_cfg(flavor="debugmodel"), full, batches)
    res = run_ranks(2, _tp_rank_debug, full, batches)
    for r in range(2):
        losses, params = res[r]
        assert losses == pytest.approx(want_losses, abs=1e-4)
        want = tp_slice_state_dict(want_params, 2, r)
        for k in want:
            assert _close(params[k], want[k]), k


def test_tensor_parallel_with_a_tied_replicated_head_matches_single_process():
    """Tied embeddings: the head is replicated, every rank scores its own token slice; embedding and head gradients
    are partial sums completed by the all-reduce of replicated parameters.  (With Adam's eps far below the gradient
    scale a gradient that is too large by the group size would go unnoticed: eps is 1e-4 here.)"""
    from maester_b200.parallel.tensor_parallel import tp_slice_state_dict
    full = _full_weights(_cfg())
    batches = _batches(2, 2, 64, 512)
    want_losses, want_params = _single(_cfg(), full, batches)
    res = run_ranks(2, _tp_rank, full, batches)
    for r in range(2):
        losses, params = res[r]
        assert losses == pytest.approx(want_losses, abs=1e-4)
        want = tp_slice_state_dict(want_params, 2, r)
        for k in want:
            assert _close(params[k], want[k], tol=1e-3), k


GEMMA_HEADS = (4, 2, 64)  # query heads, key / value heads, head size of the gemma3 "debug_gqa" flavor


def _gemma_cfg(**kw):
    return _cfg(model_name="gemma3", flavor="debug_gqa", **kw)


def _tp_rank_gemma(rank, world, full, batches):
    from maester_b200.trainer import Trainer
    tr = Trainer(_gemma_cfg(tensor_parallel_degree=2, data_parallel_shard_degree=1))
    _load_full(tr, full, tp=(2, rank, GEMMA_HEADS))
    losses = [tr.train_step(b).item() for b in batches]
    return losses, {sl.fqn: sl.param.data.clone() for u in tr.sharded.units for sl in u.slots}


def test_gemma_tensor_parallel_matches_single_process():
    """Gemma: head-group split of the fused qkv projection, sequence-parallel norms (block norms, QK-norms, final
    norm: replicated weights with partial gradients), tied replicated head."""
    from maester_b200.parallel.tensor_parallel import tp_slice_state_dict
    full = _full_weights(_gemma_cfg())
    # norm weights start at zero, where several gradient paths vanish: move them off zero
    g = torch.Generator().manual_seed(7)
    for k, v in full.items():
        if "norm" in k:
            v.copy_(0.2 * torch.randn(v.shape, generator=g))
    batches = _batches(2, 2, 64, 512)
    want_losses, want_params = _single(_gemma_cfg(), full, batches)
    res = run_ranks(2, _tp_rank_gemma, full, batches)
    for r in range(2):
        losses, params = res[r]
        assert losses == pytest.approx(want_losses, abs=1e-4)
        want = tp_slice_state_dict(want_params, 2, r, GEMMA_HEADS)
        assert set(want) == set(params)
        for k in want:
            assert params[k].shape == want[k].shape, k
            assert _close(params[k], want[k], tol=1e-3), k


def _tp_rank_debug(rank, world, full, batches):
    from maester_b200.trainer import Trainer
    tr = Trainer(_cfg(flavor="debugmodel", tensor_parallel_degree=2, data_parallel_shard_degree=1))
    _load_full(tr, full, tp=(2, rank))
    losses = [tr.train_step(b).item() for b in batches]
    return losses, {sl.fqn: sl.param.data.clone() for u in tr.sharded.units for sl in u.slots}


def _accum_rank(rank, world, full, batches):
    from maester_b200.trainer import Trainer
    tr = Trainer(_cfg(data_parallel_shard_degree=2, gradient_accumulation_steps=2))
    _load_full(tr, full)
    micro = [{k: v[rank * 2:(rank + 1) * 2] for k, v in b.items()} for b in batches]
    loss = tr.train_step(micro).item()
    return loss, {sl.fqn: sl.param.data.clone() for u in tr.sharded.units for sl in u.slots}


def test_gradient_accumulation_equals_one_big_batch():
    cfg1 = _cfg(train_batch_size=8)
    full = _full_weights(cfg1)
    b = _batches(2, 4, 64, 512)
    big = {k: torch.cat([b[0][k], b[1][k]]) for k in b[0]}
    _, want = _single(cfg1, full, [big])
    res = run_ranks(2, _accum_rank, full, b)
    for k in want:
        assert _close(res[0][1][k], want[k]), k


def test_gradient_clipping_on_sharded_buffers_matches_single_process():
    """Clipping on the flat shard buffers (per-tensor norms, all-reduce over the sharding group, one scale) gives the
    same losses and weights on two ranks as in one process, and the clip is active (tiny max norm)."""
    kw = dict(clip_gradients=True, max_grad_norm=0.05)
    cfg1 = _cfg(train_batch_size=4, **kw)
    full = _full_weights(cfg1)
    batches = _batches(3, 4, 64, 512)
    want_losses, want_params = _single(cfg1, full, batches)
    unclipped_losses, _ = _single(_cfg(train_batch_size=4), full, batches)
    assert abs(unclipped_losses[-1] - want_losses[-1]) > 1e-4  # the clip changed the trajectory
    res = run_ranks(2, _fsdp_rank, dict(data_parallel_shard_degree=2, **kw), full, batches)
    for r in range(2):
        _, params = res[r]
        for k in want_params:
            assert _close(params[k], want_params[k]), k
    mean_losses = [(a + b) / 2 for a, b in zip(res[0][0], res[1][0])]
    assert mean_losses == pytest.approx(want_losses, abs=1e-4)


def _reshard_rank(rank, world, cfg_kw, full, batches, accum):
    from maester_b200.trainer import Trainer
    tr = Trainer(_cfg(**cfg_kw))
    assert tr.sharded.resharded and tr.sharded.full is None
    tr.sharded.load_full_weights(full)
    losses = []
    for b in batches:
        mine = {k: v[rank * 2 * accum:(rank + 1) * 2 * accum] for k, v in b.items()}
        micro = [{k: v[j * 2:(j + 1) * 2] for k, v in mine.items()} for j in range(accum)]
        losses.append(tr.train_step(micro if accum > 1 else micro[0]).item())
    # reassemble this rank's view of the weights from the master shards of both ranks is done by the caller
    return losses, {sl.fqn: (sl.master.data.clone(), sl.shape) for u in tr.sharded.units for sl in u.slots}


@pytest.mark.parametrize("ac,accum,offload", [("none", 1, False), ("full", 1, False), ("none", 2, False), ("none", 1, True)])
def test_resharding_mode_matches_single_process(ac, accum, offload):
    """fsdp_reshard_after_forward=always: blocks are gathered into two staging buffers when they run and their
    gradients are reduce-scattered block by block; losses and weights equal the single-process run, with full
    activation recomputation (the block is re-gathered for its recomputation), with gradient accumulation (reduced
    after every micro-batch) and with the optimizer state kept on the host."""
    per_rank = 2 * accum
    cfg1 = _cfg(train_batch_size=2, gradient_accumulation_steps=2 * accum, ac_mode=ac)
    full = _full_weights(cfg1)
    batches = _batches(3, 2 * per_rank, 64, 512)

    from maester_b200.trainer import Trainer
    tr = Trainer(cfg1)
    _load_full(tr, full)
    want_losses = []
    for b in batches:
        micro = [{k: v[j * 2:(j + 1) * 2] for k, v in b.items()} for j in range(2 * accum)]
        want_losses.append(tr.train_step(micro).item())
    want = {sl.fqn: sl.param.data.clone() for u in tr.sharded.units for sl in u.slots}

    kw = dict(data_parallel_shard_degree=2, fsdp_reshard_after_forward="always", ac_mode=ac,
              gradient_accumulation_steps=accum, enable_cpu_offload=offload)
    res = run_ranks(2, _reshard_rank, kw, full, batches, accum)
    mean_losses = [(a + b) / 2 for a, b in zip(res[0][0], res[1][0])]
    assert mean_losses == pytest.approx(want_losses, abs=1e-4)
    for fqn, w in want.items():
        pieces = [res[r][1][fqn][0].reshape(-1, *w.shape[1:]) if w.dim() > 0 else res[r][1][fqn][0].reshape(1)
                  for r in range(2)]
        got = torch.cat(pieces, dim=0)[: max(1, w.shape[0] if w.dim() > 0 else 1)].reshape(w.shape)
        assert _close(got, w), fqn


def _gather_tables_rank(rank, world):
    from maester_b200.parallel.fsdp import gather_table
    from maester_b200.trainer import Trainer
    tr = Trainer(_cfg(data_parallel_shard_degree=world, fsdp_reshard_after_forward="always"))
    sh = tr.sharded
    out = []
    for u in sh.units[:-1]:
        table = gather_table(u, world)
        size = u.full_hi - u.full_lo
        covered = sorted((d, d + n) for d, s, n, r in table)
        # the pieces tile the parameters' ranges of the staging buffer without overlap ...
        assert all(a[1] <= b[0] for a, b in zip(covered, covered[1:])) and covered[-1][1] <= size
        assert sum(n for _, _, n, _ in table) == sum(sl.padded_numel * world for sl in u.slots)
        # ... every source range lies inside the owner's rows of this unit, and each (parameter, rank) appears once
        assert all(u.shard_lo <= s and s + n <= u.shard_hi and 0 <= r < world for _, s, n, r in table)
        assert len({(s, r) for _, s, _, r in table}) == len(table)
        # what the table describes is what the collective path produces: compare against the staged block
        sh._ensure_block(sh.units.index(u))
        buf = sh.stage[sh.units.index(u) % sh.STAGES]
        rows = [torch.empty_like(sh.shard_lp) for _ in range(world)]
        import torch.distributed as dist
        dist.all_gather(rows, sh.shard_lp)
        for d, s, n, r in table:
            assert torch.equal(buf[d:d + n], rows[r][s:s + n])
        out.append(len(table))
    return out


def test_block_gather_tables_describe_the_all_gathered_blocks():
    """The copy plan that the peer-memory gather of the resharding mode executes on a GPU, checked on CPU against the
    block that the process-group all-gather stages: same bytes at the same places."""
    res = run_ranks(2, _gather_tables_rank)
    assert res[0] == res[1] and all(n > 0 for n in res[0])
