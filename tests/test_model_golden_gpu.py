"""Whole models on the native bf16 kernels against the same models on the plain-PyTorch fp32 path (the oracle):
per-step losses of a short training run, and logits / hidden states of one forward pass.  The reference checks its
models layer by layer against transformers (tests/test_model_gemma.py:30-190, tests/test_model_llama.py:62-256); the
CPU suite of this repository does that comparison for the reference-math path (tests/test_convert.py), and this
file ties the GPU kernels to that path."""
import pytest
import torch

pytestmark = pytest.mark.gpu

ADAMW = [{"opt_class": "torch.optim.AdamW", "opt_cfg": {"lr": 2e-4, "betas": (0.9, 0.95), "weight_decay": 0.0},
          "min_dim": 0}]


def _pair(name, flavor, seq, **kw):
    """(native bf16 trainer, fp32 oracle trainer) with identical fp32 master weights."""
    from maester_b200.config import Config
    from maester_b200.trainer import Trainer
    base = dict(model_name=name, flavor=flavor, seq_len=seq, train_batch_size=2, data_parallel_shard_degree=1,
                ac_mode="selective", enable_checkpoint=False, synthetic_vocab_size=2000, scheduler="constant",
                optimizer_groups=ADAMW, **kw)
    torch.manual_seed(0)
    nat = Trainer(Config(**base))
    torch.manual_seed(0)
    ora = Trainer(Config(**base, mixed_precision_param="float32"))
    assert nat.sharded.full.dtype == torch.bfloat16 and ora.sharded.full.dtype == torch.float32
    with torch.no_grad():
        ora.sharded.master.copy_(nat.sharded.master)
        ora.sharded.full.copy_(nat.sharded.master)      # one rank: the shard is the whole model
    return nat, ora


@pytest.mark.parametrize("name,flavor", [("gemma3", "debug"), ("llama3", "tiny")])
def test_twenty_step_loss_curve_matches_the_fp32_oracle(name, flavor):
    from maester_b200.datasets.synthetic import SyntheticLoader
    from maester_b200.ops import cuda as C
    nat, ora = _pair(name, flavor, 512)
    before = C.launch_count
    vocab = min(nat.model_args.vocab_size, 2000)
    loader = SyntheticLoader(2, 512, vocab, "uniform:16:200", seed=1, with_position_ids=(name == "gemma3"))
    batches = [next(loader) for _ in range(4)]
    ln, lo = [], []
    for i in range(20):
        b = batches[i % 4]
        ln.append(nat.train_step(b).item())
        lo.append(ora.train_step(b).item())
    C.check_status()
    assert C.launch_count - before > 500, "the native kernels did not run"
    assert lo[-1] < lo[0] - 0.05, ("the oracle did not learn", lo)
    # bf16 rounding perturbs the trajectory in proportion to how far it has moved: 2e-2 absolute plus 5 % of the
    # oracle's loss decrease so far
    for i, (a, b) in enumerate(zip(ln, lo)):
        assert abs(a - b) < 2e-2 + 0.05 * (lo[0] - min(lo[:i + 1])), (i, a, b, ln, lo)
    assert ln[-1] < ln[0] - 0.05                                # and so does the native path


def test_gemma_hidden_states_and_logits_match_the_fp32_oracle_layer_by_layer():
    from maester_b200.datasets.synthetic import SyntheticLoader
    nat, ora = _pair("gemma3", "debug", 384)
    batch = next(SyntheticLoader(2, 384, 2000, "uniform:16:150", seed=2, with_position_ids=True))
    b = nat.to_device(batch)
    hs = {}

    def grab(tag):
        def hook(mod, inp, out):
            hs.setdefault(tag, []).append(out.detach().float())
        return hook

    handles = []
    for tag, tr in (("nat", nat), ("ora", ora)):
        inner = getattr(tr.model, "language_model", tr.model)
        layers = inner.model.layers
        for layer in (layers.values() if hasattr(layers, "values") else layers):
            handles.append(layer.register_forward_hook(grab(tag)))
    with torch.no_grad():
        nat.model.eval()
        ora.model.eval()
        logits_n = nat.model(b["input_ids"], position_ids=b.get("position_ids"), document_ids=b.get("document_ids"))
        logits_o = ora.model(b["input_ids"], position_ids=b.get("position_ids"), document_ids=b.get("document_ids"))
    for h in handles:
        h.remove()
    assert len(hs["nat"]) == len(hs["ora"]) > 0
    for i, (a, o) in enumerate(zip(hs["nat"], hs["ora"])):
        rel = ((a - o).norm() / o.norm()).item()
        assert rel < 2e-2, (i, rel)
    ln, lo = logits_n.float(), logits_o.float()
    assert ((ln - lo).norm() / lo.norm()).item() < 2e-2
    agree = (ln.argmax(-1) == lo.argmax(-1)).float().mean().item()
    assert agree > 0.9, agree   # a freshly initialised model has near-ties between its top logits


@pytest.mark.parametrize("name,flavor", [("gemma3", "debug"), ("llama3", "tiny")])
def test_every_parameter_gradient_matches_the_fp32_oracle(name, flavor):
    """One forward + backward on the same batch: the reduced gradient of every parameter, native against oracle."""
    from maester_b200.datasets.synthetic import SyntheticLoader
    nat, ora = _pair(name, flavor, 512)
    vocab = min(nat.model_args.vocab_size, 2000)
    batch = next(SyntheticLoader(2, 512, vocab, "uniform:16:200", seed=3, with_position_ids=(name == "gemma3")))
    grads = []
    for tr in (nat, ora):
        tr.optimizers.zero_grad()
        loss = tr.forward_backward(batch, True)
        tr.sharded.pre_optimizer_step()
        torch.cuda.synchronize()
        grads.append(({sl.fqn: tr.sharded.shard_grad[sl.shard_off: sl.shard_off + sl.padded_numel].clone()
                       for u in tr.sharded.units for sl in u.slots}, loss.item()))
    (gn, ln), (go, lo) = grads
    assert abs(ln - lo) < 5e-3
    report = {k: ((gn[k] - go[k]).norm() / go[k].norm().clamp_min(1e-20)).item() for k in go}
    bad = {k: round(v, 4) for k, v in report.items() if not v < 5e-2}
    assert not bad, bad


def test_the_optimizer_kernel_clears_the_gradients_it_consumed():
    """One rank: AdamW reads the accumulation buffer itself and clears it, so zero_grad() skips its pass over the
    buffer; the training trajectory is the same as with the separate clearing pass."""
    from maester_b200.config import Config
    from maester_b200.datasets.synthetic import SyntheticLoader
    from maester_b200.trainer import Trainer
    base = dict(model_name="llama3", flavor="tiny", seq_len=256, train_batch_size=2, data_parallel_shard_degree=1,
                ac_mode="none", enable_checkpoint=False, synthetic_vocab_size=512, scheduler="constant",
                optimizer_groups=ADAMW)
    curves = []
    for fused_clear in (True, False):
        torch.manual_seed(0)
        tr = Trainer(Config(**base))
        if not fused_clear:
            tr.sharded.grad_cleared_by_optimizer = None      # switches the kernel's clearing off
        loader = SyntheticLoader(2, 256, 512, "uniform:16:100", seed=4)
        losses = []
        for _ in range(4):
            losses.append(tr.train_step(next(loader)).item())
            if fused_clear:
                assert tr.sharded.grad_cleared_by_optimizer is True
                assert float(tr.sharded.shard_grad.abs().max()) == 0.0
        curves.append(losses)
    assert curves[0] == pytest.approx(curves[1], abs=2e-3)   # (row losses are summed with atomics: not bitwise)
