"""Grouped tcgen05 GEMM and the MoE block on the GPU against plain-PyTorch fp32 references."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("E,K,N,counts", [
    (4, 128, 256, [100, 0, 300, 17]),
    (8, 256, 1408, [1, 127, 128, 129, 0, 500, 64, 333]),
    (3, 2048, 704, [1000, 2000, 50]),
])
def test_grouped_gemm_forward_dgrad_wgrad(E, K, N, counts):
    from maester_b200.ops import cuda as C
    from maester_b200.ops.functional import padded_group_offsets
    torch.manual_seed(0)
    cnt = torch.tensor(counts, device="cuda")
    offs = padded_group_offsets(cnt)
    rows_cap = int(offs[-1].item()) + 256  # capacity may exceed what is used
    x = torch.zeros(rows_cap, K, device="cuda", dtype=torch.bfloat16)
    dy = torch.zeros(rows_cap, N, device="cuda", dtype=torch.bfloat16)
    o = offs.tolist()
    for e in range(E):
        x[o[e]:o[e] + counts[e]] = torch.randn(counts[e], K, device="cuda").to(torch.bfloat16)
        dy[o[e]:o[e] + counts[e]] = torch.randn(counts[e], N, device="cuda").to(torch.bfloat16)
    w = (torch.randn(E, K, N, device="cuda") * 0.05).to(torch.bfloat16)
    y = C.gemm_grouped_rows(x, w, offs, b_mn=True)
    dx = C.gemm_grouped_rows(dy, w, offs, b_mn=False)
    dw = torch.zeros(E, K, N, device="cuda")
    C.gemm_grouped_contr(x, dy, offs, dw)
    C.check_status()
    for e in range(E):
        sl = slice(o[e], o[e] + counts[e])
        if counts[e]:
            assert _rel(y[sl], x[sl].float() @ w[e].float()) < 6e-3
            assert _rel(dx[sl], dy[sl].float() @ w[e].float().T) < 6e-3
            assert _rel(dw[e], x[sl].float().T @ dy[sl].float()) < 6e-3
        else:
            assert dw[e].abs().max().item() == 0
        assert y[o[e] + counts[e]:o[e + 1]].abs().max().item() == 0 if o[e + 1] > o[e] + counts[e] else True


@pytest.mark.parametrize("score_func,before", [("softmax", True), ("sigmoid", False)])
def test_moe_block_native_matches_reference(score_func, before):
    from maester_b200.models.moe import MoE, MoEArgs
    torch.manual_seed(1)
    args = MoEArgs(num_experts=8, num_shared_experts=2, top_k=3, score_func=score_func, route_norm=True,
                   score_before_experts=before, load_balance_coeff=None)
    ref = MoE(args, 256, 128).cuda()
    ref.init_weights(0.05)
    nat = copy.deepcopy(ref).to(torch.bfloat16)
    for (n, p), (_, q) in zip(ref.named_parameters(), nat.named_parameters()):
        p.data.copy_(q.data.float())  # same (bf16-representable) weights on both sides
    x = (torch.randn(2, 300, 256, device="cuda") * 0.5).to(torch.bfloat16)
    xn = x.clone().requires_grad_()
    xr = x.float().requires_grad_()
    yn = nat(xn)
    yr = ref(xr)
    assert _rel(yn, yr) < 2e-2
    g = torch.randn_like(yn)
    yn.backward(g)
    yr.backward(g.float())
    assert _rel(xn.grad, xr.grad) < 3e-2
    for (n, p), (_, q) in zip(ref.named_parameters(), nat.named_parameters()):
        assert _rel(q.grad, p.grad) < 4e-2, n
    from maester_b200.ops import cuda as C
    C.check_status()


@pytest.mark.parametrize("name,flavor", [("deepseek", "debug_flex"), ("glm4", "debug"), ("llama3", "tiny")])
def test_model_families_train_on_gpu(name, flavor):
    from maester_b200.config import Config
    from maester_b200.datasets.synthetic import SyntheticLoader
    from maester_b200.ops import cuda as C
    from maester_b200.trainer import Trainer
    cfg = Config(model_name=name, flavor=flavor, seq_len=256, train_batch_size=2, data_parallel_shard_degree=1,
                 ac_mode="selective", enable_checkpoint=False, synthetic_vocab_size=2000, scheduler="constant",
                 optimizer_groups=[{"opt_class": "torch.optim.AdamW",
                                    "opt_cfg": {"lr": 2e-3, "betas": (0.9, 0.95), "weight_decay": 0.0}, "min_dim": 0}])
    tr = Trainer(cfg)
    batch = next(SyntheticLoader(2, 256, min(tr.model_args.vocab_size, 2000), "uniform:16:100"))
    losses = [tr.train_step(batch).item() for _ in range(6)]
    C.check_status()
    assert all(l == l for l in losses) and losses[-1] < losses[0], losses
