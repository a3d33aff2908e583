"""Checkpoints from elsewhere: one whose keys went through a ``torch.compile`` wrapper (``_orig_mod`` components), and
one written by the reference's own ``CheckpointManager`` (maester/checkpoint.py:95-210) from the reference's model,
loaded into this repository's trainer by parameter name."""
import os
import sys
import types

import pytest
import torch
import torch.distributed.checkpoint as dcp

from test_checkpoint_cpu import _mk, _params, _trainer_with_ckpt
from maester_b200.config import Config
from test_parallel_cpu import _batches, _cfg, _full_weights, _load_full, run_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def test_keys_written_through_a_compile_wrapper_are_mapped(tmp_path):
    os.environ.pop("WORLD_SIZE", None)
    cfg = _mk(tmp_path)
    tr, state, ck = _trainer_with_ckpt(cfg)
    _load_full(tr, _full_weights(_cfg()))
    tr.train_step(_batches(1, 2, 64, 512)[0])
    want = _params(tr)
    sd = ck.states["model"].state_dict()

    def wrapped(k):   # layers.<i>.<rest> -> layers.<i>._orig_mod.<rest>, as torch.compile on each block names them
        parts = k.split(".")
        return ".".join(parts[:2] + ["_orig_mod"] + parts[2:]) if parts[0] == "layers" else k

    stored = {wrapped(k): v for k, v in sd.items()}
    assert any("_orig_mod" in k for k in stored)
    path = str(tmp_path / "compiled")
    dcp.save({"model": stored}, checkpoint_id=path, no_dist=True)

    cfg2 = _mk(tmp_path / "b", forced_load_path=path)
    tr2, _, ck2 = _trainer_with_ckpt(cfg2)
    before = _params(tr2)
    assert any(not torch.equal(before[k], want[k]) for k in want)
    assert ck2.load()
    got = _params(tr2)
    for k in want:
        assert torch.equal(got[k], want[k]), k


def _reference_writes_ours_reads(rank, world, tmp):
    sys.path.insert(0, os.path.join(ROOT, "baseline", "shims"))   # stand-ins for packages the reference imports
    sys.path.insert(0, REF)
    from maester.checkpoint import CheckpointManager as RefManager
    from maester.models import model_name_to_cls as ref_cls, models_config as ref_cfgs
    import copy
    args = copy.deepcopy(ref_cfgs["llama3"]["debugmodel"])
    args.vocab_size = 512
    torch.manual_seed(5)
    ref = ref_cls["llama3"].from_model_args(args)
    ref.init_weights()
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda s: 1.0)
    rcfg = types.SimpleNamespace(enable_checkpoint=True, forced_load_path=None, dump_dir=tmp, job_name="job",
                                 checkpoint_folder="checkpoints", checkpoint_interval=1, model_weights_only=False,
                                 export_dtype="float32")
    RefManager(model=ref, optimizer=opt, lr_scheduler=sched, dataloader=None,
               states={"train_state": _RefState()}, cfg=rcfg).save(3, force=True)
    want = {k: v.detach().clone() for k, v in ref.state_dict().items()}

    cfg = _mk(tmp, flavor="debugmodel")
    tr, state, ck = _trainer_with_ckpt(cfg)
    assert ck.load(step=3, model_only=True)
    got = _params(tr)
    missing = sorted(set(want) - set(got) - {k for k in want if k.endswith("freqs_cis")})
    assert not missing, missing
    for k, v in got.items():
        assert torch.equal(v.float(), want[k].float()), k
    # and the loaded weights compute the reference's function
    tok = torch.randint(0, 512, (2, 64), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        a = ref(tok).float()
        b = tr.model(tok).float()
    assert torch.allclose(a, b, atol=2e-3, rtol=2e-3), (a - b).abs().max()
    return True


class _RefState:
    """Minimal stand-in for the reference trainer's step counter (a Stateful)."""

    def __init__(self):
        self.step = 3

    def state_dict(self):
        return {"step": torch.tensor(self.step)}

    def load_state_dict(self, sd):
        self.step = int(sd["step"])


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "maester")), reason="the reference is not installed")
def test_checkpoint_written_by_the_reference_loads_by_name(tmp_path):
    assert run_ranks(1, _reference_writes_ours_reads, str(tmp_path)) == [True]


def _full_state_both_ways(rank, world, tmp):
    """The reference's whole stack on one gloo rank (its model under FSDP2, its default Muon + AdamW groups, its
    ``CheckpointManager``) and this repository's trainer exchange FULL checkpoints: weights, Muon momentum, Adam
    moments and step counts, group hyper-parameters, the schedule and the step counter, in both directions."""
    sys.path.insert(0, os.path.join(ROOT, "baseline", "shims"))
    sys.path.insert(0, REF)
    import copy
    import maester.models  # noqa: F401
    import maester.optimizers.muon as ref_muon
    from maester.checkpoint import CheckpointManager as RefManager
    from maester.config import Config as RefConfig
    from maester.lr_scheduling import get_lr_scheduler as ref_scheduler
    from maester.models import model_name_to_cls as ref_cls, models_config as ref_cfgs
    from maester.optimizers import build_optimizers as ref_build
    from torch.distributed.checkpoint.state_dict import get_optimizer_state_dict
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard
    gather, scatter = ref_muon.gather, ref_muon.scatter   # gloo does not order asynchronous collectives; NCCL's stream does
    ref_muon.gather = lambda *a, **k: gather(*a, **{**k, "async_op": False})
    ref_muon.scatter = lambda *a, **k: scatter(*a, **{**k, "async_op": False})

    def reference(job):
        args = copy.deepcopy(ref_cfgs["llama3"]["debugmodel"])
        args.vocab_size = 512
        torch.manual_seed(5)
        model = ref_cls["llama3"].from_model_args(args)
        model.init_weights()
        mesh = init_device_mesh("cpu", (1,))
        for layer in model.layers.values():
            fully_shard(layer, mesh=mesh)
        fully_shard(model, mesh=mesh)
        cfg = RefConfig(dump_dir=tmp, job_name=job, enable_checkpoint=True, checkpoint_interval=1, warmup_steps=4,
                        train_num_steps=20, scheduler="linear_warmup_cosine")
        opt = ref_build(model, cfg, types.SimpleNamespace(dp_enabled=False, world_mesh=None))
        sched = ref_scheduler(opt, cfg)
        state = _RefState()
        return model, opt, sched, state, RefManager(model=model, optimizer=opt, lr_scheduler=sched, dataloader=None,
                                                    states={"train_state": state}, cfg=cfg)

    def ours(job):
        cfg = _cfg(enable_checkpoint=True, dump_dir=tmp, job_name=job, checkpoint_interval=1, flavor="debugmodel",
                   optimizer_groups=Config().optimizer_groups, warmup_steps=4, train_num_steps=20,
                   scheduler="linear_warmup_cosine")
        return _trainer_with_ckpt(cfg)

    def ref_view(model, opt, sched, state):
        sd = get_optimizer_state_dict(model, opt.optimizers)
        local = lambda t: t.to_local() if hasattr(t, "to_local") else t
        flat = {f"{n}.{k}": local(v) for n, st in sd["state"].items() for k, v in st.items()}
        groups = [{k: v for k, v in g.items() if k != "params"} for g in sd["param_groups"]]
        return ({n: p.to_local().detach() for n, p in model.named_parameters()}, flat, groups, sched.last_epoch, state.step)

    def our_view(tr, state):
        c = tr.optimizers
        flat = {f"{c._names[id(p)]}.{k}": v for o in c.optimizers for g in o.param_groups for p in g["params"]
                for k, v in o.state.get(p, {}).items()}
        groups = [{k: v for k, v in g.items() if k != "params"} for o in c.optimizers for g in o.param_groups]
        return _params(tr), flat, groups, tr.scheduler.last_epoch, state.step

    def same(a, b, what):
        (pa, fa, ga, ea, sa), (pb, fb, gb, eb, sb) = a, b
        assert sorted(pa) == sorted(pb) and sorted(fa) == sorted(fb), (what, sorted(set(fa) ^ set(fb))[:8])
        for k in pa:
            assert torch.equal(pa[k].float(), pb[k].float().reshape(pa[k].shape)), (what, k)
        for k in fa:
            x, y = fa[k], fb[k]
            if torch.is_tensor(x):
                assert torch.equal(x.float().flatten(), torch.as_tensor(y).float().flatten()), (what, k)
            else:
                assert tuple(x) == tuple(y) if isinstance(x, (tuple, list)) else x == y, (what, k, x, y)
        assert len(ga) == len(gb)
        for x, y in zip(ga, gb):
            for k in set(x) & set(y):
                assert (tuple(x[k]) == tuple(y[k])) if isinstance(x[k], (tuple, list)) else x[k] == pytest.approx(y[k]), (what, k)
        assert (ea, sa) == (eb, sb), (what, ea, eb, sa, sb)

    tok = torch.randint(0, 512, (2, 64), generator=torch.Generator().manual_seed(0))
    # A: the reference trains two steps and saves; this trainer loads everything
    model, opt, sched, state, manager = reference("from_reference")
    for _ in range(2):
        model(tok).float().logsumexp(-1).mean().backward()
        opt.step()
        sched.step()
        opt.zero_grad()
    state.step = 2
    manager.save(2, force=False)
    tr, our_state, ck = ours("from_reference")
    assert ck.load() and our_state.step == 2
    same(ref_view(model, opt, sched, state), our_view(tr, our_state), "reference -> here")
    # B: this trainer trains on from there and saves; a fresh reference stack loads everything
    tr.step = 2
    tr.train_step({"input_ids": tok, "labels": tok.roll(-1, 1)})
    our_state.step = 3
    os.replace(os.path.join(tmp, "from_reference"), os.path.join(tmp, "from_here"))
    tr2, our_state2, ck2 = ours("from_here")
    assert ck2.load()
    tr2.step = 2
    tr2.train_step({"input_ids": tok, "labels": tok.roll(-1, 1)})
    our_state2.step = 3
    ck2.save(3, force=False)
    model2, opt2, sched2, state2, manager2 = reference("from_here")
    assert manager2.load() and state2.step == 3
    same(ref_view(model2, opt2, sched2, state2), our_view(tr2, our_state2), "here -> reference")
    return True


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "maester")), reason="the reference is not installed")
def test_full_checkpoints_go_both_ways_between_the_reference_and_this_trainer(tmp_path):
    os.environ["TORCHDYNAMO_DISABLE"] = "1"   # inherited by the spawned rank: no host compiler set-up for Inductor here
    try:
        assert run_ranks(1, _full_state_both_ways, str(tmp_path)) == [True]
    finally:
        os.environ.pop("TORCHDYNAMO_DISABLE", None)
