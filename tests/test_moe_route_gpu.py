"""Native MoE routing plan and row kernels (csrc/moe_route.cu) against plain PyTorch on the GPU."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _ref_route(logits, bias, k, softmax, norm, scale):
    scores = torch.softmax(logits, 1) if softmax else torch.sigmoid(logits)
    sel = scores + bias if bias is not None else scores
    _, idx = torch.topk(sel, k, dim=1)
    top = scores.gather(1, idx)
    if norm:
        top = top / (top.sum(-1, keepdim=True) + 1e-20)
    return scores, top * scale, idx


@pytest.mark.parametrize("T,E,k,softmax,norm,use_bias", [
    (1000, 64, 6, False, True, True),
    (4096, 160, 8, True, False, False),
    (77, 8, 2, False, False, False),
    (130, 256, 1, True, True, True),
])
def test_routing_plan_matches_torch(T, E, k, softmax, norm, use_bias):
    from maester_b200.ops import cuda as C
    logits = torch.randn(T, E, device="cuda") * 2
    bias = torch.randn(E, device="cuda") * 0.1 if use_bias else None
    p = C.moe_route(logits, bias, k, softmax, norm, 2.5, False, 128)
    scores, top, idx = _ref_route(logits, bias, k, softmax, norm, 2.5)
    assert torch.allclose(p.scores, scores, atol=1e-6, rtol=1e-5)
    # same expert set per token, same gate value per chosen expert
    a, ai = torch.sort(p.idx.long(), dim=1)
    b, bi = torch.sort(idx, dim=1)
    assert torch.equal(a, b)
    assert torch.allclose(p.top.gather(1, ai), top.gather(1, bi), atol=1e-6, rtol=1e-5)
    flat = p.idx.long().reshape(-1)
    counts = torch.bincount(flat, minlength=E)
    assert torch.equal(p.counts.long(), counts) and torch.equal(p.counts_f, counts.float())
    order = torch.argsort(flat, stable=True)
    assert torch.equal(p.order.long(), order)
    assert torch.equal(p.inv.long()[order], torch.arange(T * k, device="cuda"))
    assert torch.equal(p.token_idx.long(), order // k)
    assert torch.equal(p.sorted_experts.long(), flat[order])
    assert torch.equal(p.sorted_scores, p.top.reshape(-1)[order])
    padded = (counts + 127) // 128 * 128
    offs = torch.cat([padded.new_zeros(1), padded.cumsum(0)])
    assert torch.equal(p.offs.long(), offs)
    assert p.rows_cap % 128 == 0 and p.rows_cap >= int(offs[-1])
    start = counts.cumsum(0) - counts
    row = offs[:-1][flat[order]] + torch.arange(T * k, device="cuda") - start[flat[order]]
    assert torch.equal(p.slot_row.long()[order], row)
    want = torch.full((p.rows_cap,), -1, device="cuda", dtype=torch.long)
    want[row] = order
    assert torch.equal(p.row_slot.long(), want)
    C.check_status()


def test_forced_balance_routing():
    from maester_b200.ops import cuda as C
    logits = torch.randn(100, 16, device="cuda")
    p = C.moe_route(logits, None, 4, False, False, 1.0, True, 128)
    want = (torch.arange(400, device="cuda") % 16).view(100, 4)
    assert torch.equal(p.idx.long(), want)
    assert torch.allclose(p.top, torch.sigmoid(logits).gather(1, want), atol=1e-6)


@pytest.mark.parametrize("softmax,norm", [(False, True), (True, False), (True, True), (False, False)])
def test_routing_backward_matches_autograd(softmax, norm):
    from maester_b200.ops import cuda as C
    T, E, k = 300, 64, 6
    logits = (torch.randn(T, E, device="cuda") * 2).requires_grad_()
    scores, top, idx = _ref_route(logits, None, k, softmax, norm, 1.7)
    d_top, d_scores = torch.randn(T, k, device="cuda"), torch.randn(T, E, device="cuda") * 0.1
    (top * d_top).sum().backward(retain_graph=True)
    g_top_only = logits.grad.clone()
    logits.grad = None
    ((top * d_top).sum() + (scores * d_scores).sum()).backward()
    p = C.moe_route(logits.detach(), None, k, softmax, norm, 1.7, False, 128)
    # align d_top with the kernel's own order of the chosen experts
    pos = (p.idx.long()[:, :, None] == idx[:, None, :]).float().argmax(-1)
    got = C.moe_route_bwd(d_top.gather(1, pos), None, p.scores, p.idx, softmax, norm, 1.7)
    assert torch.allclose(got, g_top_only, atol=2e-5, rtol=1e-4)
    got = C.moe_route_bwd(d_top.gather(1, pos), d_scores, p.scores, p.idx, softmax, norm, 1.7)
    assert torch.allclose(got, logits.grad, atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("scaled", [False, True])
def test_row_kernels(scaled):
    from maester_b200.ops import cuda as C
    T, E, k, D = 500, 16, 4, 264
    logits = torch.randn(T, E, device="cuda")
    p = C.moe_route(logits, None, k, False, True, 1.0, False, 128)
    x = torch.randn(T, D, device="cuda").to(torch.bfloat16)
    gate = p.top if scaled else None
    buf = C.moe_rows_gather(x, p.row_slot, gate, k)
    rs = p.row_slot.long()
    want = torch.zeros(p.rows_cap, D, device="cuda")
    live = rs >= 0
    w = p.top.reshape(-1)[rs[live]][:, None] if scaled else 1.0
    want[live] = x.float()[rs[live] // k] * w
    assert torch.allclose(buf.float(), want.to(torch.bfloat16).float())
    y = torch.randn(p.rows_cap, D, device="cuda").to(torch.bfloat16)
    out = C.moe_rows_combine(y, p.slot_row, gate, k)
    rows = y.float()[p.slot_row.long()].view(T, k, D)
    if scaled:
        rows = rows * p.top[:, :, None]
    assert _rel(out, rows.sum(1)) < 4e-3
    g = torch.randn(T, D, device="cuda").to(torch.bfloat16)
    dots = C.moe_slot_dot(y, p.slot_row, g, k)
    wantd = (y.float()[p.slot_row.long()].view(T, k, D) * g.float()[:, None, :]).sum(-1).reshape(-1)
    assert torch.allclose(dots, wantd, atol=1e-3, rtol=1e-4)
    C.check_status()


@pytest.mark.parametrize("score_func,before,bias", [("sigmoid", True, True), ("softmax", False, False),
                                                     ("sigmoid", False, True)])
def test_fused_block_matches_aten_chain(score_func, before, bias, monkeypatch):
    """The same bf16 block with and without the native routing kernels."""
    import maester_b200.models.moe.moe as M
    torch.manual_seed(3)
    args = M.MoEArgs(num_experts=16, num_shared_experts=1, top_k=4, score_func=score_func, route_norm=True,
                     route_scale=1.5, score_before_experts=before, load_balance_coeff=1e-3 if bias else None,
                     aux_loss_coeff=0.01)
    a = M.MoE(args, 256, 128).cuda()
    a.init_weights(0.05)
    a = a.to(torch.bfloat16)
    if bias:
        a.expert_bias = torch.randn(16, device="cuda") * 0.05
    b = copy.deepcopy(a)
    x = (torch.randn(2, 333, 256, device="cuda") * 0.5).to(torch.bfloat16)
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    g = torch.randn_like(x)
    monkeypatch.setattr(M, "FUSED_ROUTING", True)
    ya = a(xa)
    (ya.float() * g.float()).sum().add(a.aux_loss).backward()
    monkeypatch.setattr(M, "FUSED_ROUTING", False)
    yb = b(xb)
    (yb.float() * g.float()).sum().add(b.aux_loss).backward()
    assert _rel(ya, yb) < 1e-2
    assert torch.equal(a.tokens_per_expert, b.tokens_per_expert)
    assert abs(a.aux_loss.item() - b.aux_loss.item()) < 1e-5
    assert _rel(xa.grad, xb.grad) < 2e-2
    for (n, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
        assert _rel(p.grad, q.grad) < 3e-2, n
    from maester_b200.ops import cuda as C
    C.check_status()
