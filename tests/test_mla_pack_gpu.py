"""Latent-attention packing kernel (csrc/mla_pack.cu) against the eager slicing / RoPE / cat path."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("H,nope,rope,vdim,P", [(16, 128, 64, 128, 256), (4, 64, 32, 64, 128), (3, 32, 16, 40, 64)])
def test_pack_forward_backward_match_eager(H, nope, rope, vdim, P):
    from maester_b200.ops import cuda as C
    from maester_b200.ops import reference as ref
    B, S, lat = 2, 333, 96
    T = B * S
    q = torch.randn(T, H * (nope + rope), device="cuda").to(torch.bfloat16)
    kvb = torch.randn(T, H * (nope + vdim), device="cuda").to(torch.bfloat16)
    kv_a = torch.randn(T, lat + rope, device="cuda").to(torch.bfloat16)
    kpe = kv_a[:, lat:]
    pos = torch.randint(0, 5000, (B, S), device="cuda")
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, rope, 2, device="cuda", dtype=torch.float32) / rope))
    out = C.mla_pack_fwd(q, kvb, kpe, pos.reshape(-1), inv_freq, H, nope, rope, vdim, P).view(T, 3, H, P)

    def eager(q, kvb, kpe):
        q4 = q.view(B, S, H, nope + rope)
        qn, qp = q4.split([nope, rope], dim=-1)
        qp = ref.apply_rope(qp, pos, inv_freq, "interleaved")
        kp = ref.apply_rope(kpe.reshape(B, S, 1, rope), pos, inv_freq, "interleaved").expand(-1, -1, H, -1)
        kn, v = kvb.view(B, S, H, nope + vdim).split([nope, vdim], dim=-1)
        z = lambda n: q.new_zeros(B, S, H, n)
        return torch.stack([torch.cat([qn, qp, z(P - nope - rope)], -1), torch.cat([kn, kp, z(P - nope - rope)], -1),
                            torch.cat([v, z(P - vdim)], -1)], dim=2).reshape(T, 3, H, P)

    qe, kvbe, kpee = (t.clone().float().requires_grad_() for t in (q, kvb, kpe))
    want = eager(qe, kvbe, kpee)
    assert torch.allclose(out.float(), want.to(torch.bfloat16).float(), atol=2e-2, rtol=2e-2)
    assert _rel(out, want) < 4e-3
    g = torch.randn(T, 3 * H * P, device="cuda").to(torch.bfloat16)
    (want * g.float().view(T, 3, H, P)).sum().backward()
    dq, dkvb, dkpe = C.mla_pack_bwd(g, pos.reshape(-1), inv_freq, H, nope, rope, vdim, P)
    assert _rel(dq, qe.grad) < 4e-3
    assert _rel(dkvb, kvbe.grad) < 4e-3
    assert _rel(dkpe, kpee.grad) < 6e-3
    C.check_status()


def test_attention_module_with_and_without_packing_kernel(monkeypatch):
    import maester_b200.models.deepseek.model as M
    from maester_b200.models.deepseek import deepseek_configs
    args = deepseek_configs["debug_flex"]
    a = M.Attention(args).cuda()
    a.init_weights(0.02)
    a = a.to(torch.bfloat16)
    b = copy.deepcopy(a)
    B, S = 2, 256
    x = (torch.randn(B, S, args.dim, device="cuda") * 0.5).to(torch.bfloat16)
    pos = torch.arange(S, device="cuda")[None].expand(B, S).contiguous()
    inv_freq = M.yarn_inv_freq(args, device="cuda")
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    g = torch.randn_like(x)
    monkeypatch.setattr(M, "FUSED_MLA_PACK", True)
    ya = a(xa, pos, inv_freq, None)
    ya.backward(g)
    monkeypatch.setattr(M, "FUSED_MLA_PACK", False)
    yb = b(xb, pos, inv_freq, None)
    yb.backward(g)
    assert _rel(ya, yb) < 1e-2
    assert _rel(xa.grad, xb.grad) < 2e-2
    for (n, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
        assert _rel(p.grad, q.grad) < 2e-2, n
