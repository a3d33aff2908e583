"""Optimizer-side parity with the reference's own code (installed copy of the reference package), on CPU as one gloo
rank: Muon with its built-in Adam groups step for step (bitwise: the Newton–Schulz iteration runs in bf16, so even the
grouping of a scalar factor matters), the learning-rate schedules, and the job configuration both ways.

Two process-wide adjustments, neither of which changes the reference's arithmetic: ``TORCHDYNAMO_DISABLE=1`` (no host
compiler set-up for Inductor here; ``torch.compile`` becomes the eager function) and the reference's asynchronous
``gather`` / ``scatter`` made blocking: on NCCL they are ordered by the stream, on gloo nothing orders them before the
next line reads their output."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "maester")), reason="the reference is not installed")


def _setup():
    sys.path.insert(0, os.path.join(ROOT, "baseline", "shims"))
    sys.path.insert(0, REF)
    sys.path.insert(0, ROOT)
    import maester.models  # noqa: F401  (the reference's packages import each other in a circle unless this one goes first)


def _muon():
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="29617")
    dist.init_process_group("gloo", rank=0, world_size=1)
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor
    import maester.optimizers.muon as ref_muon
    from maester_b200.optimizers import Muon
    gather, scatter = ref_muon.gather, ref_muon.scatter
    ref_muon.gather = lambda *a, **k: gather(*a, **{**k, "async_op": False})
    ref_muon.scatter = lambda *a, **k: scatter(*a, **{**k, "async_op": False})
    mesh = init_device_mesh("cpu", (1,))
    g = torch.Generator().manual_seed(0)
    shapes = [(64, 32), (32, 64), (48, 48), (40, 24)]
    adam_shapes = [(96, 16), (16,)]
    make = lambda ss: [torch.randn(s, generator=g) * 0.05 for s in ss]
    w, wa = make(shapes), make(adam_shapes)
    steps = [(make(shapes), make(adam_shapes)) for _ in range(4)]
    dt = lambda t: distribute_tensor(t.clone(), mesh, [Shard(0)])
    rp, ra = [torch.nn.Parameter(dt(t)) for t in w], [torch.nn.Parameter(dt(t)) for t in wa]
    op, oa = [torch.nn.Parameter(t.clone()) for t in w], [torch.nn.Parameter(t.clone()) for t in wa]
    adam = dict(use_muon=False, lr=3e-3, betas=(0.9, 0.95), eps=1e-8, wd=0.1)
    ref = ref_muon.Muon([dict(params=rp, use_muon=True, lr=0.02, wd=0.01, momentum=0.95, ns_steps=5), dict(params=ra, **adam)])
    ours = Muon([dict(params=op, use_muon=True, lr=0.02, wd=0.01, momentum=0.95, ns_steps=5), dict(params=oa, **adam)])
    for gm, ga in steps:
        for p, q, t in zip(rp + ra, op + oa, gm + ga):
            p.grad, q.grad = dt(t), t.clone()
        ref.step()
        ours.step()
        for p, q in zip(rp, op):
            assert torch.equal(p.data.to_local(), q.data), tuple(q.shape)       # Muon matrices: bitwise
        for p, q in zip(ra, oa):
            assert torch.allclose(p.data.to_local(), q.data, rtol=1e-6, atol=1e-8), tuple(q.shape)
    moved = ((op[0].data - w[0]).norm() / w[0].norm()).item()
    assert moved > 0.05, moved
    dist.destroy_process_group()
    print(f"muon: 4 steps bitwise equal on {shapes}; first matrix moved by {moved:.3f} of its norm")


def _schedules_and_config():
    import torch
    from maester.config import Config as RefConfig
    from maester.lr_scheduling import get_lr_scheduler as ref_sched
    from maester_b200.config import Config
    from maester_b200.lr_scheduling import get_lr_scheduler
    for kw in (dict(scheduler="linear_warmup_cosine", warmup_steps=7, train_num_steps=60),
               dict(scheduler="linear_warmup_constant_sqrt_decay", warmup_steps=5, train_num_steps=50, cooldown_steps=12)):
        lrs = []
        for cfg, build in ((RefConfig(**kw), ref_sched), (Config(**kw), get_lr_scheduler)):
            opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=0.5)
            sched, seq = build(opt, cfg), []
            for _ in range(kw["train_num_steps"]):
                seq.append(opt.param_groups[0]["lr"])
                opt.step()
                sched.step()
            lrs.append(seq)
        assert lrs[0] == pytest.approx(lrs[1], rel=1e-12), kw
    # a job configuration written by the reference's tooling is a valid configuration here, field for field
    ref = RefConfig(model_name="gemma3", flavor="4B", job_name="from-reference")
    dumped = json.loads(ref.model_dump_json())
    cfg = Config(**dumped)
    for k, v in dumped.items():
        assert json.loads(cfg.model_dump_json())[k] == v, k
    from maester_b200.optimizers.container import _import
    for group in cfg.optimizer_groups:   # "maester.optimizers.Muon" and "torch.optim.AdamW" both resolve
        assert _import(group["opt_class"]).__name__ == group["opt_class"].rpartition(".")[2]
    print("schedules equal; the reference's config.json loads field for field")


def _load_balance():
    """The auxiliary-loss-free balancing hook: same counters in, same biases and the same 18 statistics out, under the
    same metric names, step after step (running totals included)."""
    import copy
    import types
    import torch
    from maester.config import Config as RefConfig
    from maester.models import model_name_to_cls as ref_cls, models_config as ref_cfgs
    from maester.models.deepseek.optimizer import build_deepseek_optimizers as ref_build
    from maester_b200.config import Config
    from maester_b200.models import model_name_to_cls as our_cls, models_config as our_cfgs
    from maester_b200.models.deepseek.optimizer import build_deepseek_optimizers
    ra, oa = copy.deepcopy(ref_cfgs["deepseek"]["debug"]), copy.deepcopy(our_cfgs["deepseek"]["debug"])
    for a in (ra, oa):
        a.vocab_size, a.max_seq_len, a.n_layers, a.moe_args.load_balance_coeff = 512, 96, 4, 1e-2
    ref, ours = ref_cls["deepseek"].from_model_args(ra), our_cls["deepseek"].from_model_args(oa)
    ref.init_weights()
    ours.init_weights()
    groups = [{"opt_class": "torch.optim.AdamW", "opt_cfg": {"lr": 1e-3}, "min_dim": 0}]
    dims = types.SimpleNamespace(dp_enabled=False, world_mesh=None)
    ref_opt = ref_build(ref, RefConfig(optimizer_groups=groups, enable_wandb=False), dims)
    our_opt = build_deepseek_optimizers(ours, Config(optimizer_groups=groups, enable_wandb=False), dims)
    ref_moes = [l.moe for l in ref.layers.values() if l.moe_enabled]
    our_moes = ours.moe_layers()
    assert len(ref_moes) == len(our_moes) == 3
    g = torch.Generator().manual_seed(0)
    for step in range(4):
        for a, b in zip(ref_moes, our_moes):
            counts = torch.randint(0, 200, a.tokens_per_expert.shape, generator=g)
            if step == 2:
                counts[:3] = 0   # dead experts
            a.tokens_per_expert.copy_(counts)
            b.tokens_per_expert.copy_(counts)
        for p in list(ref.parameters()) + list(ours.parameters()):
            p.grad = torch.zeros_like(p)
        ref_opt.step()
        our_opt.step()
        for a, b in zip(ref_moes, our_moes):
            assert torch.equal(a.expert_bias, b.expert_bias) and a.expert_bias.abs().max() > 0
            assert not a.tokens_per_expert.any() and not b.tokens_per_expert.any()
        want, got = dict(ref_opt._hook_stats), dict(our_opt._hook_stats)
        assert len(want) == 18 and set(want) <= set(got), sorted(set(want) - set(got))
        for k, v in want.items():
            assert got[k] == pytest.approx(v, rel=1e-5, abs=1e-7), (step, k, v, got[k])
    print("load balance: biases equal and 18 statistics equal over 4 steps")


def _groups():
    """Which optimizer, learning rate and weight decay every parameter gets: the muP three-group rule and the
    first-match-wins ``optimizer_groups`` (``min_dim``, ``exclude_names``); and the container's state-dict keys."""
    import copy
    import types
    import torch
    from maester.config import Config as RefConfig
    from maester.models import model_name_to_cls as ref_cls, models_config as ref_cfgs
    from maester.optimizers import build_optimizers as ref_build
    from maester_b200.config import Config
    from maester_b200.models import model_name_to_cls as our_cls, models_config as our_cfgs
    from maester_b200.optimizers import build_optimizers

    def assignment(model, opt):
        names = {id(p): n for n, p in model.named_parameters()}
        return {names[id(p)]: (type(o).__name__, g.get("lr"), g.get("weight_decay"), g.get("momentum"))
                for o in opt.optimizers for g in o.param_groups for p in g["params"]}

    dims = types.SimpleNamespace(dp_enabled=False, world_mesh=None)
    adamw = {"opt_class": "torch.optim.AdamW", "opt_cfg": {"lr": 1e-3, "weight_decay": 0.1}, "min_dim": 0}
    cases = {
        "mup": dict(enable_mup=True, base_model_width=256, model_width=1024, optimizer_groups=[adamw]),
        "first match wins": dict(optimizer_groups=[
            {"opt_class": "torch.optim.SGD", "opt_cfg": {"lr": 0.02, "momentum": 0.9}, "min_dim": 2,
             "exclude_names": ["tok_embeddings", "output"]}, adamw]),
    }
    for name, kw in cases.items():
        ra, oa = copy.deepcopy(ref_cfgs["llama3"]["debugmodel"]), copy.deepcopy(our_cfgs["llama3"]["debugmodel"])
        for a in (ra, oa):
            a.vocab_size = 512
            if name == "mup":
                a.enable_mup, a.mup_width_mul = True, 4.0
        ref, ours = ref_cls["llama3"].from_model_args(ra), our_cls["llama3"].from_model_args(oa)
        ref_opt, our_opt = ref_build(ref, RefConfig(**kw), dims), build_optimizers(ours, Config(**kw), dims)
        want, got = assignment(ref, ref_opt), assignment(ours, our_opt)
        assert want == got, {k: (want[k], got.get(k)) for k in want if want[k] != got.get(k)}
        assert len({v for v in want.values()}) >= 2, name          # the rule did split the parameters
        for m, o in ((ref, ref_opt), (ours, our_opt)):             # one step, so that there is state to name
            for p in m.parameters():
                p.grad = torch.ones_like(p)
            o.step()
        # the reference's container returns nested dictionaries, this one flat dotted keys; a checkpoint stores the
        # dotted paths, which is where the two have to agree
        def dotted(d, prefix=""):
            out = set()
            for k, v in (d.items() if isinstance(d, dict) else enumerate(d)):
                key = f"{prefix}{k}"
                out |= dotted(v, key + ".") if isinstance(v, (dict, list)) and k != "params" and len(v) else {key}
            return out
        ref_keys, our_keys = dotted(ref_opt.state_dict()), dotted(our_opt.state_dict())
        assert ref_keys == our_keys, sorted(ref_keys ^ our_keys)[:10]
    print("optimizer groups: same assignment under muP and under first-match-wins; same state-dict keys")


def _utilities():
    """Peak-FLOPs table (the MFU denominator), metric names derived from parameter names, gradient clipping, the weight
    scale monitor."""
    import copy
    import torch
    import maester.metrics as ref_metrics
    import maester.utils as ref_utils
    import maester_b200.metrics as metrics
    import maester_b200.utils as utils
    from maester_b200.models import model_name_to_cls, models_config
    for device in ("NVIDIA A100-SXM4-80GB", "NVIDIA H100 80GB HBM3", "NVIDIA H100 NVL", "NVIDIA H100 PCIe", "NVIDIA H200",
                   "NVIDIA B200", "AMD Instinct MI250X", "AMD Instinct MI300X", "something else"):
        assert ref_utils.get_peak_flops(device) == utils.get_peak_flops(device), device
    for name, flavor in (("llama3", "debugmodel"), ("gemma3", "debug"), ("glm4", "debug"), ("deepseek", "debug")):
        args = copy.deepcopy(models_config[name][flavor])
        args.vocab_size = 512
        with torch.device("meta"):
            model = model_name_to_cls[name].from_model_args(args)
        for n, _ in model.named_parameters():
            for wrapped in (n, n.replace("layers.", "layers._checkpoint_wrapped_module.", 1), "_orig_mod." + n):
                assert ref_utils.clean_param_name(wrapped) == utils.clean_param_name(wrapped), wrapped
    g = torch.Generator().manual_seed(0)
    for kw in (dict(max_norm=1.0), dict(max_norm=0.5, norm_type=float("inf")), dict(max_norm=2.0, norm_type=1.0)):
        ps = [torch.nn.Parameter(torch.randn(5, 7, generator=g)) for _ in range(3)]
        qs = [torch.nn.Parameter(p.detach().clone()) for p in ps]
        for p, q in zip(ps, qs):
            p.grad = 3 * torch.randn(5, 7, generator=g)
            q.grad = p.grad.clone()
        ref_utils.clip_grad_norm(ps, **kw)
        utils.clip_grad_norm(qs, **kw)
        assert all(torch.allclose(p.grad, q.grad, rtol=1e-6) for p, q in zip(ps, qs)), kw
    net = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.Linear(3, 2))
    want, got = ref_metrics.WeightScaleMonitor(net, log_freq=1).step_monitor(), metrics.WeightScaleMonitor(net, log_freq=1).step_monitor()
    assert sorted(want) == sorted(got) and all(got[k] == pytest.approx(v, rel=1e-6) for k, v in want.items())
    print("utilities: peak FLOPs, metric names, clipping and the weight scale monitor agree")


@pytest.mark.parametrize("what", ["muon", "schedules_and_config", "load_balance", "groups", "utilities"])
def test_optimizer_side_parity_with_the_reference(what):
    r = subprocess.run([sys.executable, os.path.abspath(__file__), what], capture_output=True, text=True,
                       env=dict(os.environ, TORCHDYNAMO_DISABLE="1"), timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    print(r.stdout.strip().splitlines()[-1])


if __name__ == "__main__":
    _setup()
    {"muon": _muon, "schedules_and_config": _schedules_and_config, "load_balance": _load_balance,
     "groups": _groups, "utilities": _utilities}[sys.argv[1]]()
