"""DCP checkpoints of the sharding runtime: round trip, resume equality, resharding, expert layout,
weights-only export, corrupted checkpoints (all on CPU, gloo for the multi-rank cases)."""
import os
import shutil

import pytest
import torch

from test_parallel_cpu import ADAMW, _batches, _cfg, _close, _full_weights, _load_full, run_ranks


def _mk(tmp, **kw):
    return _cfg(enable_checkpoint=True, dump_dir=str(tmp), job_name="job", checkpoint_interval=2, **kw)


def _trainer_with_ckpt(cfg):
    from train import TrainState
    from maester_b200.checkpoint import CheckpointManager
    from maester_b200.trainer import Trainer
    tr = Trainer(cfg)
    state = TrainState()
    ck = CheckpointManager(model=tr.model, optimizer=tr.optimizers, lr_scheduler=tr.scheduler, dataloader=None,
                           states={"train_state": state}, cfg=cfg)
    return tr, state, ck


def _params(tr):
    return {sl.fqn: sl.param.data.clone() for u in tr.sharded.units for sl in u.slots}


def _run_save_resume(rank, world, cfg_kw, tmp, full, batches):
    """Train 2 steps, save, train 2 more; then a fresh trainer loads the checkpoint and trains the same 2."""
    cfg = _mk(tmp, **cfg_kw)
    tr, state, ck = _trainer_with_ckpt(cfg)
    _load_full(tr, full)
    mine = lambda b: {k: v[tr.dp_rank * 2:(tr.dp_rank + 1) * 2] for k, v in b.items()}
    for b in batches[:2]:
        tr.train_step(mine(b))
        state.step += 1
    ck.save(state.step)
    after_save = _params(tr)
    cont = [tr.train_step(mine(b)).item() for b in batches[2:]]
    want = _params(tr)
    tr2, state2, ck2 = _trainer_with_ckpt(cfg)
    assert ck2.load() and state2.step == 2
    restored = _params(tr2)
    for k in after_save:
        assert torch.equal(restored[k], after_save[k]), k
    tr2.step = state2.step
    resumed = [tr2.train_step(mine(b)).item() for b in batches[2:]]
    got = _params(tr2)
    assert resumed == pytest.approx(cont, abs=1e-6)
    for k in want:
        assert torch.allclose(got[k], want[k], atol=1e-6), k
    return True


def test_single_process_save_and_resume(tmp_path):
    cfg1 = _cfg()
    full = _full_weights(cfg1)
    os.environ.pop("WORLD_SIZE", None)
    assert _run_save_resume(0, 1, {}, tmp_path, full, _batches(4, 2, 64, 512))
    assert sorted(os.listdir(tmp_path / "job" / "checkpoints")) == ["step-2"]


def test_two_rank_fsdp_save_and_resume(tmp_path):
    full = _full_weights(_cfg())
    res = run_ranks(2, _run_save_resume, dict(data_parallel_shard_degree=2), str(tmp_path), full, _batches(4, 4, 64, 512))
    assert res == [True, True]


def test_two_rank_save_and_resume_with_the_default_muon_and_adamw_groups(tmp_path):
    """Muon's momentum (and the Adam moments of the other group) must come back from the checkpoint: the resumed run
    reproduces the continued one only if they do."""
    from maester_b200.config import Config
    full = _full_weights(_cfg(flavor="debugmodel"))
    kw = dict(data_parallel_shard_degree=2, flavor="debugmodel", optimizer_groups=Config().optimizer_groups)
    assert run_ranks(2, _run_save_resume, kw, str(tmp_path), full, _batches(4, 4, 64, 512)) == [True, True]


def _save_only(rank, world, cfg_kw, tmp, full, batches):
    cfg = _mk(tmp, **cfg_kw)
    tr, state, ck = _trainer_with_ckpt(cfg)
    _load_full(tr, full)
    for b in batches:
        tr.train_step({k: v[tr.dp_rank * 2:(tr.dp_rank + 1) * 2] for k, v in b.items()})
        state.step += 1
    ck.save(state.step)
    # unsharded view of the master weights for comparison
    return {sl.fqn: sl.param.data.clone() for u in tr.sharded.units for sl in u.slots}


def test_checkpoint_written_by_two_ranks_loads_in_one_process(tmp_path):
    """Resharding: the DTensor shard layout lets DCP load a 2-rank checkpoint into an unsharded model."""
    full = _full_weights(_cfg())
    res = run_ranks(2, _save_only, dict(data_parallel_shard_degree=2), str(tmp_path), full, _batches(2, 4, 64, 512))
    os.environ.pop("WORLD_SIZE", None)
    tr, state, ck = _trainer_with_ckpt(_mk(tmp_path))
    assert ck.load(model_only=True)
    got = _params(tr)
    for k, v in res[0].items():
        assert _close(got[k], v, tol=1e-2), k  # the 2-rank full view is bf16-free fp32 on CPU: equal up to rounding
    from maester_b200.convert.io import read_dcp_model
    flat = read_dcp_model(tmp_path / "job" / "checkpoints" / "step-2")
    assert set(flat) >= set(res[0]) and all(flat[k].shape == res[0][k].shape for k in res[0])


def test_final_export_is_weights_only_in_export_dtype(tmp_path):
    os.environ.pop("WORLD_SIZE", None)
    cfg = _mk(tmp_path, model_weights_only=True, export_dtype="bfloat16")
    tr, state, ck = _trainer_with_ckpt(cfg)
    tr.train_step(_batches(1, 2, 64, 512)[0])
    ck.save(7, force=True)
    from maester_b200.convert.io import read_dcp_model
    flat = read_dcp_model(tmp_path / "job" / "checkpoints" / "step-7")
    assert all(v.dtype == torch.bfloat16 for v in flat.values())
    import torch.distributed.checkpoint as dcp
    keys = dcp.FileSystemReader(str(tmp_path / "job" / "checkpoints" / "step-7")).read_metadata().state_dict_metadata
    assert not any(k.startswith(("optimizer", "lr_scheduler", "train_state")) for k in keys)


def test_seed_checkpoint_and_forced_load_path(tmp_path):
    os.environ.pop("WORLD_SIZE", None)
    cfg = _mk(tmp_path, model_weights_only=False)
    tr, state, ck = _trainer_with_ckpt(cfg)
    tr.train_step(_batches(1, 2, 64, 512)[0])
    state.step = 5
    ck.save(0, force=True)  # a step-0 ("seed") checkpoint: only the model is read back
    tr2, state2, ck2 = _trainer_with_ckpt(cfg)
    assert ck2.load(step=0) and state2.step == 0
    for k, v in _params(tr).items():
        assert torch.equal(_params(tr2)[k], v), k
    forced = tmp_path / "elsewhere"
    shutil.copytree(tmp_path / "job" / "checkpoints" / "step-0", forced)
    tr3, state3, ck3 = _trainer_with_ckpt(_mk(tmp_path / "other", forced_load_path=str(forced)))
    assert ck3.load() and state3.step == 0
    for k, v in _params(tr).items():
        assert torch.equal(_params(tr3)[k], v), k
    with pytest.raises(ValueError):
        _trainer_with_ckpt(_mk(tmp_path / "x", forced_load_path=str(tmp_path / "missing")))[2].load()


def test_corrupted_checkpoint_is_detected(tmp_path):
    os.environ.pop("WORLD_SIZE", None)
    cfg = _mk(tmp_path)
    tr, state, ck = _trainer_with_ckpt(cfg)
    tr.train_step(_batches(1, 2, 64, 512)[0])
    ck.save(2)
    meta = tmp_path / "job" / "checkpoints" / "step-2" / ".metadata"
    meta.write_bytes(meta.read_bytes()[:20])  # truncated metadata
    tr2, state2, ck2 = _trainer_with_ckpt(cfg)
    with pytest.raises(Exception):
        ck2.load()


def _ep_save_resume(rank, world, tmp, full, batches):
    from test_expert_parallel_cpu import _cfg as ep_cfg, _load
    from train import TrainState
    from maester_b200.checkpoint import CheckpointManager
    from maester_b200.trainer import Trainer
    cfg = ep_cfg(data_parallel_shard_degree=world, expert_parallel_degree=2, enable_checkpoint=True, dump_dir=str(tmp),
                 job_name="ep", checkpoint_interval=1)

    def make():
        tr = Trainer(cfg)
        st = TrainState()
        return tr, st, CheckpointManager(model=tr.model, optimizer=tr.optimizers, lr_scheduler=tr.scheduler,
                                         dataloader=None, states={"train_state": st}, cfg=cfg)

    tr, st, ck = make()
    _load(tr, full)
    mine = lambda b: {k: v[tr.dp_rank * 2:(tr.dp_rank + 1) * 2] for k, v in b.items()}
    tr.train_step(mine(batches[0]))
    st.step = 1
    ck.save(1)
    want_loss = tr.train_step(mine(batches[1])).item()
    tr2, st2, ck2 = make()
    assert ck2.load() and st2.step == 1
    got_loss = tr2.train_step(mine(batches[1])).item()
    assert got_loss == pytest.approx(want_loss, abs=1e-5)
    return sum(1 for m in tr2.model.layers.values() if getattr(m, "moe_enabled", False))


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_checkpoint_round_trip(tmp_path, world):
    from test_expert_parallel_cpu import _cfg as ep_cfg
    full = _full_weights(ep_cfg(train_batch_size=2 * world))
    res = run_ranks(world, _ep_save_resume, str(tmp_path), full, _batches(2, 2 * world, 32, 2000))
    assert all(r > 0 for r in res)
    from maester_b200.convert.io import read_dcp_model
    flat = read_dcp_model(tmp_path / "ep" / "checkpoints" / "step-1")
    w1 = next(v for k, v in flat.items() if k.endswith("moe.experts.w1"))
    assert w1.shape[0] == 8  # all experts, reassembled from the (ep x fsdp) shards


def _tp_save(rank, world, tmp, full, batches, dp, cp=1):
    from maester_b200.trainer import Trainer
    from train import TrainState
    from maester_b200.checkpoint import CheckpointManager
    cfg = _mk(tmp, tensor_parallel_degree=2, data_parallel_shard_degree=dp, context_parallel_degree=cp)
    tr = Trainer(cfg)
    import torch.distributed as dist
    g = tr.parallel_dims.mesh_group("tp")
    _load_full(tr, full, tp=(2, dist.get_rank(g)))
    st = TrainState()
    ck = CheckpointManager(model=tr.model, optimizer=tr.optimizers, lr_scheduler=tr.scheduler, dataloader=None,
                           states={"train_state": st}, cfg=cfg)
    ck.save(2, force=False)
    return True


@pytest.mark.parametrize("world,dp,cp", [(2, 1, 1), (4, 2, 1), (4, 1, 2)])
def test_tensor_parallel_checkpoint_reassembles_full_weights(tmp_path, world, dp, cp):
    """TP slices (x data-parallel shards, x context-parallel shards) are published as DTensors, so the checkpoint
    holds whole tensors."""
    full = _full_weights(_cfg())
    run_ranks(world, _tp_save, str(tmp_path), full, _batches(1, 2, 64, 512), dp, cp)
    from maester_b200.convert.io import read_dcp_model
    flat = read_dcp_model(tmp_path / "job" / "checkpoints" / "step-2")
    for k, v in full.items():
        if k in flat:
            assert flat[k].shape == v.shape, k
            assert torch.equal(flat[k], v.float()), k
    assert {"layers.0.attention.wq.weight", "layers.0.attention.wo.weight", "layers.0.feed_forward.w2.weight"} <= set(flat)


def _gemma_tp_save(rank, world, tmp, full, batches, dp):
    """Gemma under TP 2: one step, save, and a second trainer with the same layout loads the checkpoint back."""
    import torch.distributed as dist
    from test_parallel_cpu import GEMMA_HEADS
    cfg = _mk(tmp, model_name="gemma3", flavor="debug_gqa", tensor_parallel_degree=2, data_parallel_shard_degree=dp)
    tr, state, ck = _trainer_with_ckpt(cfg)
    g = tr.parallel_dims.mesh_group("tp")
    _load_full(tr, full, tp=(2, dist.get_rank(g), GEMMA_HEADS))
    mine = {k: v[tr.dp_rank * 2:(tr.dp_rank + 1) * 2] for k, v in batches[0].items()}
    tr.train_step(mine)
    state.step = 2
    ck.save(2)
    tr2, state2, ck2 = _trainer_with_ckpt(cfg)
    assert ck2.load() and state2.step == 2
    want, got = _params(tr), _params(tr2)
    for k in want:
        assert torch.equal(got[k], want[k]), k
    o1, o2 = tr.optimizers.optimizers[0], tr2.optimizers.optimizers[0]
    for key in ("m", "v"):
        assert o1._flat[key].abs().sum() > 0 and torch.equal(o1._flat[key], o2._flat[key]), key
    # the last checkpoint of a run: weights only, in the export dtype (the row pieces survive the conversion)
    ck.model_weights_only, ck.export_dtype = True, torch.bfloat16
    ck.save(4, force=True)
    return {k: v for k, v in want.items()} if tr.dp_rank == 0 or dp == 1 else None


@pytest.mark.parametrize("world,dp", [(2, 1), (4, 2)])
def test_gemma_tensor_parallel_checkpoint_holds_whole_tensors_in_the_reference_row_order(tmp_path, world, dp):
    """The fused qkv projection is split by head groups, so a rank's rows are three separate row ranges of the whole
    [q; k; v] matrix (more when a data-parallel shard boundary cuts one): the checkpoint must hold the whole matrix in
    that order, readable without knowing the parallel layout."""
    from maester_b200.parallel.tensor_parallel import tp_slice_state_dict
    from test_parallel_cpu import GEMMA_HEADS, _gemma_cfg
    full = _full_weights(_gemma_cfg())
    res = run_ranks(world, _gemma_tp_save, str(tmp_path), full, _batches(1, 2 * dp, 64, 512), dp)
    from maester_b200.convert.io import read_dcp_model
    flat = read_dcp_model(tmp_path / "job" / "checkpoints" / "step-2")
    assert set(full) <= set(flat)
    for k in full:
        assert flat[k].shape == full[k].shape, k
    export = read_dcp_model(tmp_path / "job" / "checkpoints" / "step-4")
    for k in full:
        assert export[k].dtype == torch.bfloat16 and torch.equal(export[k], flat[k].to(torch.bfloat16)), k
    # the trained slices of each TP rank are the head-group slices of the stored whole tensors
    for r in range(world):
        if res[r] is None:
            continue
        want = tp_slice_state_dict({k: flat[k] for k in full}, 2, r % 2, GEMMA_HEADS)
        for k, v in res[r].items():
            assert torch.equal(v.float(), want[k].float()), (r, k)


def _gemma_tp_load(rank, world, tmp, dp):
    import torch.distributed as dist
    cfg = _mk(tmp, model_name="gemma3", flavor="debug_gqa", tensor_parallel_degree=2, data_parallel_shard_degree=dp)
    tr, state, ck = _trainer_with_ckpt(cfg)
    assert ck.load() and state.step == 2
    return dist.get_rank(tr.parallel_dims.mesh_group("tp")), _params(tr)


@pytest.mark.parametrize("world,dp", [(2, 1), (4, 2)])
def test_unsharded_gemma_checkpoint_loads_into_tensor_parallel_ranks(tmp_path, world, dp):
    """A checkpoint written by one process (the layout of the reference and of converted HF weights) is read by
    tensor-parallel ranks: each takes its head groups out of the whole [q; k; v] matrix."""
    os.environ.pop("WORLD_SIZE", None)
    from maester_b200.parallel.tensor_parallel import tp_slice_state_dict
    from test_parallel_cpu import GEMMA_HEADS, _gemma_cfg
    full = _full_weights(_gemma_cfg())
    tr, state, ck = _trainer_with_ckpt(_mk(tmp_path, model_name="gemma3", flavor="debug_gqa"))
    _load_full(tr, full)
    tr.train_step(_batches(1, 2, 64, 512)[0])
    state.step = 2
    ck.save(2)
    want_full = _params(tr)
    for tp_rank, got in run_ranks(world, _gemma_tp_load, str(tmp_path), dp):
        want = tp_slice_state_dict(want_full, 2, tp_rank, GEMMA_HEADS)
        for k, v in got.items():
            assert torch.equal(v, want[k]), k


def _expert_tp_save(rank, world, tmp, full, cfg_kw):
    from test_expert_parallel_cpu import _cfg as ep_cfg, _load
    from train import TrainState
    from maester_b200.checkpoint import CheckpointManager
    from maester_b200.trainer import Trainer
    import torch.distributed as dist
    cfg = ep_cfg(enable_checkpoint=True, dump_dir=str(tmp), job_name="etp", checkpoint_interval=1, **cfg_kw)
    tr = Trainer(cfg)
    g = tr.parallel_dims.mesh_group("tp")
    _load(tr, full, (dist.get_rank(g), dist.get_world_size(g)))
    st = TrainState()
    ck = CheckpointManager(model=tr.model, optimizer=tr.optimizers, lr_scheduler=tr.scheduler, dataloader=None,
                           states={"train_state": st}, cfg=cfg)
    ck.save(1)
    # a fresh trainer restores exactly this rank's pieces
    before = {sl.fqn: sl.master.data.clone() for u in tr.sharded.units for sl in u.slots}
    tr2 = Trainer(cfg)
    st2 = TrainState()
    ck2 = CheckpointManager(model=tr2.model, optimizer=tr2.optimizers, lr_scheduler=tr2.scheduler, dataloader=None,
                            states={"train_state": st2}, cfg=cfg)
    assert ck2.load()
    for u in tr2.sharded.units:
        for sl in u.slots:
            assert torch.equal(sl.master.data, before[sl.fqn]), sl.fqn
    return True


@pytest.mark.parametrize("world,kw", [
    (2, dict(tensor_parallel_degree=2)),                                                          # TP-only experts
    (4, dict(tensor_parallel_degree=2, data_parallel_shard_degree=2, expert_parallel_degree=4)),  # EP x TP
])
def test_tensor_parallel_expert_checkpoint_holds_whole_tensors(tmp_path, world, kw):
    """Experts sliced over tp (alone or under expert parallelism) reassemble to the unsharded tensors."""
    from test_expert_parallel_cpu import _cfg as ep_cfg
    full = _full_weights(ep_cfg())
    run_ranks(world, _expert_tp_save, str(tmp_path), full, kw)
    from maester_b200.convert.io import read_dcp_model
    flat = read_dcp_model(tmp_path / "etp" / "checkpoints" / "step-1")
    checked = 0
    for k, v in full.items():
        if k in flat:
            assert flat[k].shape == v.shape, (k, flat[k].shape, v.shape)
            assert torch.equal(flat[k], v.float()), k
            checked += 1
    assert checked > 10 and any(k.endswith("moe.experts.w2") for k in flat)


def test_row_pieces_tile_the_owned_rows_and_point_at_the_right_global_rows():
    """Pure function behind the head-group-split checkpoints: for every split of a rank's local rows over data-parallel
    shards, the pieces cover exactly the owned rows, in order, without overlap, and each local row maps to the global
    row that the segment table says."""
    import itertools
    import types
    from maester_b200.checkpoint import row_pieces
    from maester_b200.parallel.tensor_parallel import qkv_segments
    for heads, kv, hd, tp in [(4, 2, 8, 2), (8, 4, 16, 4), (32, 16, 4, 2), (6, 3, 5, 3)]:
        for rank in range(tp):
            segs = qkv_segments(heads, kv, hd, tp, rank)
            local_rows = sum(n for _, n in segs)
            to_global = [g0 + i for g0, n in segs for i in range(n)]       # local row -> global row
            slot = types.SimpleNamespace(tp_segments=segs)
            for shards in (1, 2, 3, 5):
                per = -(-local_rows // shards)
                covered = []
                for s in range(shards):
                    lo, hi = min(s * per, local_rows), min((s + 1) * per, local_rows)
                    at = 0
                    for rel, g0, n in row_pieces(slot, lo, hi):
                        assert rel == at and n > 0                            # pieces follow one another
                        assert [g0 + i for i in range(n)] == to_global[lo + rel: lo + rel + n]
                        at += n
                    assert at == hi - lo
                    covered += list(range(lo, hi))
                assert covered == list(range(local_rows))
        # the ranks' segments partition the whole [q; k; v] matrix
        rows = sorted(itertools.chain.from_iterable(range(g0, g0 + n) for r in range(tp)
                                                    for g0, n in qkv_segments(heads, kv, hd, tp, r)))
        assert rows == list(range((heads + 2 * kv) * hd))
