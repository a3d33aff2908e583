"""Whole models on the native bf16 kernels against the same models on the plain-PyTorch fp32 path (the oracle):
per-step losses of a short training run, and logits / hidden states of one forward pass.  The reference checks its
models layer by layer against transformers (tests/test_model_gemma.py:30-190, tests/test_model_llama.py:62-256); the
CPU suite of this repository does that comparison for the reference-math path (tests/test_convert.py), and this
file ties the GPU kernels to that path."""
import pytest
import torch

pytestmark = pytest.mark.gpu

ADAMW = [{"opt_class": "torch.optim.AdamW", "opt_cfg": {"lr": 1e-3, "betas": (0.9, 0.95), "weight_decay": 0.0},
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
    worst = max(abs(a - b) for a, b in zip(ln, lo))
    assert worst < 2e-2, (worst, ln, lo)
    assert ln[-1] < ln[0] - 0.5 and lo[-1] < lo[0] - 0.5   # both actually learn the four batches


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
    assert agree > 0.97, agree
