"""Optimizer container, parameter grouping, Muon and Newton–Schulz (CPU), plus GPU NS check."""
import copy
import os
import sys

import pytest
import torch
import torch.nn as nn

from maester_b200.config import Config
from maester_b200.models import model_name_to_cls, model_name_to_optimizers_builder, models_config
from maester_b200.ops import reference as ref
from maester_b200.optimizers import FusedAdamW, Muon, OptimizersContainer, build_optimizers
from maester_b200.optimizers.muon import newton_schulz, syrk


def _tiny_llama():
    args = copy.deepcopy(models_config["llama3"]["tiny"])
    args.vocab_size, args.max_seq_len = 500, 64
    return model_name_to_cls["llama3"].from_model_args(args)


def test_default_groups_split_muon_and_adamw():
    model = _tiny_llama()
    opt = build_optimizers(model, Config(), None)
    assert len(opt.optimizers) == 2 and isinstance(opt.optimizers[0], Muon)
    muon_names = {opt._names[id(p)] for g in opt.optimizers[0].param_groups for p in g["params"]}
    adam_names = {opt._names[id(p)] for g in opt.optimizers[1].param_groups for p in g["params"]}
    assert "tok_embeddings.weight" in adam_names and "norm.weight" in adam_names
    assert "layers.0.attention.wq.weight" in muon_names and not (muon_names & adam_names)
    # one scheduler drives all groups
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda s: 0.5)
    assert opt.optimizers[0].param_groups[0]["lr"] == pytest.approx(0.01)
    assert opt.optimizers[1].param_groups[0]["lr"] == pytest.approx(1.5e-4)
    keys = opt.state_dict().keys()
    assert any(k.startswith("opt0_") for k in keys) and any(k.startswith("opt1_") for k in keys)


def test_class_paths_of_the_reference_package_name_this_package():
    from maester_b200.optimizers import Muon, MuonDDP
    from maester_b200.optimizers.container import _import
    assert _import("maester.optimizers.Muon") is Muon and _import("maester.optimizers.MuonDDP") is MuonDDP
    assert _import("torch.optim.AdamW") is torch.optim.AdamW


def test_unassigned_parameter_is_an_error():
    model = _tiny_llama()
    cfg = Config(optimizer_groups=[{"opt_class": "torch.optim.AdamW", "opt_cfg": {"lr": 1e-3}, "min_dim": 2}])
    with pytest.raises(ValueError):
        build_optimizers(model, cfg, None)


def test_mup_three_groups():
    model = _tiny_llama()
    cfg = Config(enable_mup=True, model_width=1024, base_model_width=256,
                 optimizer_groups=[{"opt_class": "torch.optim.AdamW", "opt_cfg": {"lr": 1e-2, "weight_decay": 0.1}}])
    opt = build_optimizers(model, cfg, None)
    groups = opt.param_groups
    assert len(groups) == 3
    assert groups[0]["lr"] == pytest.approx(1e-2 / 4) and groups[0]["weight_decay"] == 0.1
    assert groups[1]["lr"] == pytest.approx(1e-2) and groups[2]["weight_decay"] == 0.0


def test_newton_schulz_orthogonalises():
    torch.manual_seed(0)
    g = torch.randn(64, 160)
    o = newton_schulz(g).float()
    s = torch.linalg.svdvals(o)
    assert s.max() < 1.3 and s.min() > 0.5          # singular values pulled towards 1
    u, _, vh = torch.linalg.svd(g, full_matrices=False)
    assert ((o - u @ vh).norm() / (u @ vh).norm()) < 0.45
    assert newton_schulz(g.t().contiguous()).shape == (160, 64)
    a = torch.randn(8, 16)
    assert torch.allclose(syrk(a, alpha=2.0), 2 * a @ a.T, atol=1e-5)


def test_muon_step_matches_formula_and_trains():
    torch.manual_seed(0)
    w = nn.Parameter(torch.randn(32, 16))
    w0 = w.detach().clone()
    opt = Muon([w], lr=0.1, momentum=0.9, wd=0.01)
    w.grad = torch.randn(32, 16)
    g = w.grad.clone()
    opt.step()
    m = (1 - 0.9) * g
    u = g + 0.9 * (m - g)
    want = w0 * (1 - 0.1 * 0.01) - 0.1 * (32 / 16) ** 0.5 * ref.newton_schulz(u).float()
    assert torch.allclose(w.detach(), want, atol=2e-2)
    # a least-squares problem gets solved
    x, y = torch.randn(256, 16), torch.randn(256, 32)
    opt = Muon([w], lr=0.05, momentum=0.9, wd=0.0)
    first = None
    for _ in range(40):
        loss = ((x @ w.T - y) ** 2).mean()
        first = first or loss.item()
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert loss.item() < first


def test_fused_adamw_cpu_fallback_matches_torch():
    torch.manual_seed(0)
    p1, p2 = nn.Parameter(torch.randn(10, 4)), nn.Parameter(torch.randn(10, 4))
    p2.data.copy_(p1.data)
    a = FusedAdamW([p1], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    b = torch.optim.AdamW([p2], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for _ in range(3):
        g = torch.randn(10, 4)
        p1.grad, p2.grad = g.clone(), g.clone()
        a.step()
        b.step()
    assert torch.allclose(p1, p2, atol=1e-6)


@pytest.mark.gpu
def test_newton_schulz_native_matches_reference():
    torch.manual_seed(0)
    for shape in [(256, 1024), (1024, 256), (512, 512)]:
        g = torch.randn(*shape, device="cuda")
        got = newton_schulz(g).float()
        want = ref.newton_schulz(g).float()
        assert ((got - want).norm() / want.norm()) < 5e-2
    from maester_b200.ops import cuda as C
    C.check_status()


def test_moe_load_balance_hook_updates_biases_and_defers_its_statistics():
    """The optimizer pre-hook of the MoE families (reference: maester/models/deepseek/optimizer.py:14-222) moves the
    expert biases against the load and clears the counters; the balance statistics are only computed when read."""
    from maester_b200.config import Config
    from maester_b200.trainer import Trainer
    cfg = Config(model_name="deepseek", flavor="debug_flex", seq_len=64, train_batch_size=2, enable_checkpoint=False,
                 synthetic_vocab_size=512, scheduler="constant", ac_mode="none", data_parallel_shard_degree=1,
                 optimizer_groups=[{"opt_class": "torch.optim.AdamW", "opt_cfg": {"lr": 1e-3}, "min_dim": 0}])
    from maester_b200.models import models_config
    flavor = models_config["deepseek"]["debug_flex"]
    old = flavor.moe_args.load_balance_coeff
    flavor.moe_args.load_balance_coeff = 1e-3          # the debug flavors switch the bias update off
    try:
        tr = Trainer(cfg)
    finally:
        flavor.moe_args.load_balance_coeff = old
    moes = [l.moe for l in tr.model.layers.values() if getattr(l, "moe_enabled", False)]
    assert moes and all(m.expert_bias is not None for m in moes)
    before = [m.expert_bias.clone() for m in moes]
    g = torch.Generator().manual_seed(0)
    batch = {"input_ids": torch.randint(0, 512, (2, 64), generator=g), "labels": torch.randint(0, 512, (2, 64), generator=g)}
    tr.train_step(batch)
    stats = tr.optimizers._hook_stats
    assert stats._pending is not None and dict.__len__(stats) == 0        # nothing computed yet
    assert all(float(m.tokens_per_expert.abs().sum()) == 0 for m in moes)  # counters cleared by the hook
    assert any(not torch.equal(b, m.expert_bias) for b, m in zip(before, moes))
    assert all(abs(float(m.expert_bias.mean())) < 1e-6 for m in moes)      # re-centred
    assert bool(stats)
    out = dict(stats)                                                      # first read computes
    assert stats._pending is None
    assert out["expert_balance/batches"] == 1
    for key in ("maxvio_batch_avg", "cv_batch_min", "maxvio_global_max", "dead_frac_global_avg"):
        assert f"expert_balance/{key}" in out
    tr.train_step(batch)
    assert dict(tr.optimizers._hook_stats)["expert_balance/batches"] == 2


def test_muon_peer_exchange_layout_never_overlaps():
    """Offsets of the symmetric staging / result buffers of Muon's peer-memory exchange: every matrix has its own range
    in every rank's staging buffer, every owner's result ranges are disjoint, and all offsets keep 16-byte alignment
    when the chunks do."""
    from maester_b200.optimizers.muon import peer_exchange_layout
    import random
    rng = random.Random(0)
    for world in (2, 3, 4, 8):
        for _ in range(20):
            n = rng.randint(1, 40)
            chunks = [rng.choice([8, 64, 320, 1280, 2560]) for _ in range(n)]
            cols = [rng.choice([8, 256, 2560, 10240]) for _ in range(n)]
            sizes, in_off, out_off, fill = peer_exchange_layout(chunks, cols, world)
            assert in_off[0] == 0 and all(in_off[i + 1] - in_off[i] == sizes[i] for i in range(n))
            for owner in range(world):
                spans = sorted((out_off[i], out_off[i] + sizes[i] * world) for i in range(n) if i % world == owner)
                assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))
                assert (spans[-1][1] if spans else 0) == fill[owner]
            assert all(o % 8 == 0 for o in in_off + out_off)
            # the piece rank r pulls back from the owner lies inside the owner's range of that matrix
            for i in range(n):
                for r in range(world):
                    lo = out_off[i] + r * sizes[i]
                    assert out_off[i] <= lo and lo + sizes[i] <= out_off[i] + sizes[i] * world
