"""Context parallelism (sequence split + head-scatter all-to-all) on two gloo ranks equals one process."""
import pytest
import torch

from test_parallel_cpu import _batches, _cfg, _close, _full_weights, _load_full, _single, run_ranks


def _cp_rank(rank, world, full, batches):
    from maester_b200.trainer import Trainer
    tr = Trainer(_cfg(flavor="debugmodel", context_parallel_degree=2, data_parallel_shard_degree=1))
    assert tr.cp is not None and tr.sharded.world == 2  # parameters are sharded over dp_shard x cp
    _load_full(tr, full)
    losses = [tr.train_step(b).item() for b in batches]
    return losses, {sl.fqn: sl.param.data.clone() for u in tr.sharded.units for sl in u.slots}


def test_context_parallel_matches_single_process():
    full = _full_weights(_cfg(flavor="debugmodel", seq_len=64))
    batches = _batches(2, 2, 64, 512)
    # give the batches documents so that masking across the sequence split is exercised
    for b in batches:
        doc = torch.zeros(2, 64, dtype=torch.int32)
        doc[:, 20:] = 1
        doc[:, 45:] = 2
        b["document_ids"] = doc
    want_losses, want_params = _single(_cfg(flavor="debugmodel"), full, batches)
    res = run_ranks(2, _cp_rank, full, batches)
    mean_losses = [(a + b) / 2 for a, b in zip(res[0][0], res[1][0])]
    assert mean_losses == pytest.approx(want_losses, abs=1e-4)
    for r in range(2):
        for k in want_params:
            assert _close(res[r][1][k], want_params[k]), k


def _ring_rank(rank, world, full, batches, flavor):
    from maester_b200.trainer import Trainer
    tr = Trainer(_cfg(flavor=flavor, context_parallel_degree=world, data_parallel_shard_degree=1,
                      context_parallel_mode="ring"))
    assert tr.cp is not None and tr.cp.mode == "ring"
    _load_full(tr, full)
    losses = [tr.train_step(b).item() for b in batches]
    return losses, {sl.fqn: sl.param.data.clone() for u in tr.sharded.units for sl in u.slots}


@pytest.mark.parametrize("world", [2, 4])
def test_ring_context_parallel_matches_single_process(world):
    """Zig-zag sequence shards with K / V gathered from the other ranks (here: the dense reference path on gloo):
    same losses and weights as one process, for a model whose 3 kv heads... do not divide by the CP degree."""
    flavor = "debugmodel"
    full = _full_weights(_cfg(flavor=flavor, seq_len=64))
    batches = _batches(2, 2, 64, 512)
    want_losses, want_params = _single(_cfg(flavor=flavor), full, batches)
    res = run_ranks(world, _ring_rank, full, batches, flavor)
    mean_losses = [sum(r[0][i] for r in res) / world for i in range(len(want_losses))]
    assert mean_losses == pytest.approx(want_losses, abs=1e-4)
    for r in range(world):
        for k in want_params:
            assert _close(res[r][1][k], want_params[k]), k


def test_ring_mode_refuses_packed_documents():
    from maester_b200.parallel.context_parallel import CPInfo
    from maester_b200.parallel.ring_attention import ring_attention_block, zigzag_index
    idx = zigzag_index(16, 2, 1)
    assert idx.tolist() == [4, 5, 6, 7, 8, 9, 10, 11]
    assert zigzag_index(16, 2, 0).tolist() == [0, 1, 2, 3, 12, 13, 14, 15]
    with pytest.raises(NotImplementedError):
        ring_attention_block(torch.zeros(1, 8, 3 * 16), None, None, None, None, None, 1, 1, 16,
                             CPInfo(None, 2, 0, mode="ring"), doc_ids=torch.zeros(1, 8))
