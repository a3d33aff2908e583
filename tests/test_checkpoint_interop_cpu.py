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
