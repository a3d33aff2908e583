"""Tensor-parallel fused kernels on ONE GPU: the peer table points at local tensors (one per emulated rank), so the
all-gather GEMM's copying CTA pairs and the pull-and-sum kernel run as over NVLink.  Each launch is self-contained
(the copying and the computing CTAs belong to the same kernel), so nothing waits on another launch."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


class _Blocks:
    def __init__(self, tensors):
        self.world = len(tensors)
        self.tensors = tensors
        self.ptr_array = (ctypes.c_void_p * self.world)(*[t.data_ptr() for t in tensors])
        self.tensor = tensors[0]


@pytest.mark.parametrize("world,Ml,K,N,b_mn,copiers", [(2, 256, 512, 384, False, 1), (2, 1024, 1024, 640, True, 4),
                                                       (4, 512, 264, 136, False, 8), (2, 2048, 4096, 1024, False, 2)])
def test_all_gather_gemm_with_local_peer_table(world, Ml, K, N, b_mn, copiers):
    from maester_b200.ops import cuda as C
    blocks = [torch.randn(Ml, K, device="cuda").to(torch.bfloat16) for _ in range(world)]
    peers = _Blocks(blocks)
    w = (torch.randn((K, N) if b_mn else (N, K), device="cuda") * 0.05).to(torch.bfloat16)
    full = torch.cat(blocks)
    want = full.float() @ (w.float() if b_mn else w.float().t())
    flags = torch.zeros(world * Ml // 256, dtype=torch.int32, device="cuda")
    for rank in range(world):
        a = torch.full((world * Ml, K), float("nan"), device="cuda", dtype=torch.bfloat16)
        a[rank * Ml:(rank + 1) * Ml].copy_(blocks[rank])  # only the local block is in place
        y = C.gemm_ag(a, peers, rank, w, flags, b_mn=b_mn, copiers=copiers)
        assert torch.equal(a, full), "the gathered operand is left behind for the backward pass"
        assert ((y.float() - want).norm() / want.norm()).item() < 1e-2
    C.check_status()


@pytest.mark.parametrize("world,M,N,with_res", [(2, 512, 256, True), (4, 1024, 520, False), (8, 1024, 128, True)])
def test_pull_sum_with_local_peer_table(world, M, N, with_res):
    from maester_b200.ops import cuda as C
    parts = [torch.randn(M, N, device="cuda").to(torch.bfloat16) for _ in range(world)]
    peers = _Blocks(parts)
    rows = M // world
    total = torch.stack([p.float() for p in parts]).sum(0)
    for rank in range(world):
        res = torch.randn(rows, N, device="cuda").to(torch.bfloat16) if with_res else None
        out = torch.empty(rows, N, device="cuda", dtype=torch.bfloat16)
        C.pull_sum(peers, rank, res, out)
        want = total[rank * rows:(rank + 1) * rows] + (res.float() if with_res else 0)
        assert ((out.float() - want).norm() / want.norm()).item() < 6e-3
    C.check_status()


@pytest.mark.parametrize("world,Ml,K,F,act", [(2, 256, 512, 384, 1), (2, 512, 1024, 1024, 0), (4, 256, 256, 128, 1)])
def test_all_gather_gemm_with_gated_unit_epilogues(world, Ml, K, F, act):
    """Forward (gate|up GEMM + activation) and backward (down-projection dgrad + activation derivative) of the
    tensor-parallel gated MLP, with the gather of the row blocks inside the same kernel (local peer table)."""
    from maester_b200.ops import cuda as C
    from maester_b200.ops import reference as ref
    torch.manual_seed(7)
    blocks = [torch.randn(Ml, K, device="cuda").to(torch.bfloat16) for _ in range(world)]
    peers = _Blocks(blocks)
    w_gu = (torch.randn(2 * F, K, device="cuda") * K ** -0.5).to(torch.bfloat16)
    full = torch.cat(blocks)
    glu = ref.swiglu if act == 1 else ref.geglu
    want_gu = (full.float() @ w_gu.float().t())
    flags = torch.zeros(world * Ml // 256, dtype=torch.int32, device="cuda")
    for rank in range(world):
        a = torch.full((world * Ml, K), float("nan"), device="cuda", dtype=torch.bfloat16)
        a[rank * Ml:(rank + 1) * Ml].copy_(blocks[rank])
        gu, out = C.gemm_ag_glu(a, peers, rank, w_gu, flags, mode=1, act=act, copiers=2)
        assert torch.equal(a, full)
        assert ((gu.float() - want_gu).norm() / want_gu.norm()).item() < 1e-2
        want_out = glu(gu.float())                    # the activation sees the rounded [gate | up] that is stored
        assert ((out.float() - want_out).norm() / want_out.norm()).item() < 1e-2
    # backward: the gathered operand is dy [M, D]; weight [D, F]; epilogue applies act'
    D = K
    dys = [torch.randn(Ml, D, device="cuda").to(torch.bfloat16) for _ in range(world)]
    dpeers = _Blocks(dys)
    w_down = (torch.randn(D, F, device="cuda") * D ** -0.5).to(torch.bfloat16)
    dy_full = torch.cat(dys)
    guf = gu.float().requires_grad_()
    glu(guf).backward(dy_full.float() @ w_down.float())
    for rank in range(world):
        a = torch.full((world * Ml, D), float("nan"), device="cuda", dtype=torch.bfloat16)
        a[rank * Ml:(rank + 1) * Ml].copy_(dys[rank])
        d_gu = C.gemm_ag_glu(a, dpeers, rank, w_down, flags, mode=2, act=act, gate_up=gu, copiers=2)
        assert torch.equal(a, dy_full)
        assert ((d_gu.float() - guf.grad).norm() / guf.grad.norm()).item() < 1.5e-2
    C.check_status()
