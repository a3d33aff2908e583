"""Expert parallelism, expert FSDP and expert tensor parallelism on gloo ranks equal one process."""
import pytest
import torch

from test_parallel_cpu import ADAMW, _batches, _close, _full_weights, run_ranks
from maester_b200.config import Config


def _cfg(**kw):
    base = dict(model_name="deepseek", flavor="debug_flex", seq_len=32, train_batch_size=2, enable_checkpoint=False,
                optimizer_groups=ADAMW, scheduler="constant", ac_mode="none", data_parallel_shard_degree=1)
    base.update(kw)
    return Config(**base)


def _load(trainer, full, tp=None):
    """Load unsharded weights: expert-parallel slots take their experts, TP slots their hidden slice."""
    sh = trainer.sharded
    with torch.no_grad():
        for u in sh.units:
            for sl in u.slots:
                w = full[sl.fqn]
                if sl.dom == 1:
                    w = w[sl.row_base: sl.row_base + sl.rows]
                if tp is not None and tuple(w.shape) != tuple(sl.shape):
                    r, n = tp
                    for d in range(w.dim()):
                        if w.shape[d] != sl.shape[d]:
                            c = w.shape[d] // n
                            w = w.narrow(d, r * c, c)
                sl.param.data.copy_(w)
    sh.init_master_from_full()


def _gather_params(tr):
    return {sl.fqn: (sl.param.data.clone(), sl.row_base, sl.dom) for u in tr.sharded.units for sl in u.slots}


def _single(cfg, full, batches):
    from maester_b200.trainer import Trainer
    tr = Trainer(cfg)
    _load(tr, full)
    losses = [tr.train_step(b).item() for b in batches]
    return losses, {k: v[0] for k, v in _gather_params(tr).items()}


def _ep_rank(rank, world, cfg_kw, full, batches, per_rank):
    from maester_b200.trainer import Trainer
    tr = Trainer(_cfg(**cfg_kw))
    tp = None
    if cfg_kw.get("tensor_parallel_degree", 1) > 1:
        import torch.distributed as dist
        g = tr.parallel_dims.mesh_group("tp")
        tp = (dist.get_rank(g), dist.get_world_size(g))
    _load(tr, full, tp)
    losses = []
    for b in batches:
        i = tr.dp_rank
        mine = {k: v[i * per_rank:(i + 1) * per_rank] for k, v in b.items()}
        losses.append(tr.train_step(mine).item())
    return losses, _gather_params(tr), tp


def _check(res, want_losses, want, world, dp):
    mean = [sum(r[0][i] for r in res) / world for i in range(len(want_losses))]
    assert mean == pytest.approx(want_losses, abs=2e-4)
    for losses, params, tp in res:
        for k, (got, base, dom) in params.items():
            ref = want[k]
            if dom == 1:
                ref = ref[base: base + got.shape[0]]
            if tp is not None and tuple(ref.shape) != tuple(got.shape):
                r, n = tp
                for d in range(ref.dim()):
                    if ref.shape[d] != got.shape[d]:
                        c = ref.shape[d] // n
                        ref = ref.narrow(d, r * c, c)
            assert _close(got, ref), k


@pytest.mark.parametrize("world,ep", [(2, 2), (4, 2)])
def test_expert_parallel_matches_single_process(world, ep):
    cfg1 = _cfg(train_batch_size=2 * world)
    full = _full_weights(cfg1)
    batches = _batches(2, 2 * world, 32, 2000)
    want_losses, want = _single(cfg1, full, batches)
    res = run_ranks(world, _ep_rank, dict(data_parallel_shard_degree=world, expert_parallel_degree=ep), full,
                    batches, 2)
    _check(res, want_losses, want, world, world)


def test_tensor_parallel_experts_match_single_process():
    cfg1 = _cfg(train_batch_size=2)
    full = _full_weights(cfg1)
    batches = _batches(2, 2, 32, 2000)
    want_losses, want = _single(cfg1, full, batches)
    res = run_ranks(2, _ep_rank, dict(tensor_parallel_degree=2), full, batches, 2)
    _check(res, want_losses, want, 2, 1)


def test_expert_parallel_with_tensor_parallel_experts_matches_single_process():
    """ep 4 x tp 2 on four ranks (two data-parallel ranks of two tensor-parallel ranks each): experts are split over
    the two ``dp_shard_in_ep`` ranks and every expert's hidden dimension over ``tp``
    (reference ExpertTensorParallel: maester/parallelisms/expert_parallel.py:167-213)."""
    cfg1 = _cfg(train_batch_size=4)
    full = _full_weights(cfg1)
    batches = _batches(2, 4, 32, 2000)
    want_losses, want = _single(cfg1, full, batches)
    res = run_ranks(4, _ep_rank, dict(data_parallel_shard_degree=2, tensor_parallel_degree=2, expert_parallel_degree=4),
                    full, batches, 2)
    # the two tensor-parallel ranks of a data-parallel rank see the same batch and report the same loss
    mean = [sum(r[0][i] for r in res) / 4 for i in range(len(want_losses))]
    assert mean == pytest.approx(want_losses, abs=2e-4)
    _check(res, want_losses, want, 4, 2)
