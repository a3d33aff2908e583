"""Collective-fused kernels on ONE GPU with a local peer table (one buffer per emulated rank): the reduce-scatter +
AdamW + all-gather kernel on its peer-loop path, the shard push, and the GEMM whose epilogue routes rows to their
owners followed by the partial-sum kernel.  None of these kernels waits on another launch."""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


class _Peers:
    multicast_ptr = 0

    def __init__(self, tensors):
        self.world = len(tensors)
        self.tensors = tensors
        self.ptr_array = (ctypes.c_void_p * self.world)(*[t.data_ptr() for t in tensors])
        self.tensor = tensors[0]


def _fused_chunks(recs):
    arr = np.zeros(len(recs), dtype=np.dtype([("s", "<i8"), ("f", "<i8"), ("len", "<i4"), ("t", "<i4")]))
    for i, r in enumerate(recs):
        arr[i] = r
    return torch.from_numpy(arr.view(np.uint8).copy()).cuda()


@pytest.mark.parametrize("world", [2, 4])
def test_reduce_scatter_adamw_all_gather_kernel(world):
    from maester_b200.ops import cuda as C
    n0, n1 = 40000, 1024                      # two tensors per shard: (lr x1, decay 0.1) and (lr x0.5, no decay)
    n = n0 + n1
    grads = [torch.randn(world * n, device="cuda") for _ in range(world)]            # param-major full gradients
    fulls = [torch.zeros(world * n, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    pg, pf = _Peers(grads), _Peers(fulls)
    tensors = torch.tensor([[1.0, 0.1], [0.5, 0.0]], device="cuda")
    lr_t = torch.tensor([3e-3], device="cuda")
    b1, b2, eps, step, divide = 0.9, 0.95, 1e-8, 3, float(world)
    gsum = torch.stack(grads).sum(0) / divide
    for rank in range(world):
        master, m, v = torch.randn(n, device="cuda"), torch.randn(n, device="cuda") * 0.1, torch.rand(n, device="cuda") * 0.01
        p0, m0, v0 = master.clone(), m.clone(), v.clone()
        gout = torch.empty(n, device="cuda")
        # tensor 0 occupies full rows [world*0 .. ) rank-major: rank r's rows of tensor t start at base_t + r * n_t
        recs, full_of = [], {}
        for t, (off, cnt, base) in enumerate([(0, n0, 0), (n0, n1, world * n0)]):
            for c0 in range(0, cnt, 32768):
                recs.append((off + c0, base + rank * cnt + c0, min(32768, cnt - c0), t))
        chunks = _fused_chunks(recs)
        C.fused_rs_adamw_ag(pg, pf, master, m, v, gout, chunks, tensors, len(recs), lr_t, b1, b2, eps, step, divide)
        torch.cuda.synchronize()
        for t, (off, cnt, base, lrm, wd) in enumerate([(0, n0, 0, 1.0, 0.1), (n0, n1, world * n0, 0.5, 0.0)]):
            g = gsum[base + rank * cnt: base + (rank + 1) * cnt]
            sl = slice(off, off + cnt)
            wm = b1 * m0[sl] + (1 - b1) * g
            wv = b2 * v0[sl] + (1 - b2) * g * g
            lr = 3e-3 * lrm
            wp = p0[sl] * (1 - lr * wd) - lr / (1 - b1 ** step) * wm / (wv.sqrt() / math.sqrt(1 - b2 ** step) + eps)
            assert torch.allclose(gout[sl], g, atol=1e-6, rtol=1e-5)
            assert torch.allclose(m[sl], wm, atol=1e-6, rtol=1e-5) and torch.allclose(v[sl], wv, atol=1e-7, rtol=1e-5)
            assert torch.allclose(master[sl], wp, atol=1e-5, rtol=1e-5)
            for f in fulls:  # every rank's parameter buffer received the bf16 copy
                assert torch.equal(f[base + rank * cnt: base + (rank + 1) * cnt], master[sl].to(torch.bfloat16))
    C.check_status()


def test_routed_gemm_epilogue_and_partial_sum():
    from maester_b200.ops import cuda as C
    world, M, N, K = 2, 1024, 384, 512
    rows = M // world
    outs = [torch.full((world * rows * N,), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    peers = _Peers(outs)
    a = [torch.randn(M, K, device="cuda").to(torch.bfloat16) for _ in range(world)]
    b = [(torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16) for _ in range(world)]
    for rank in range(world):
        C.gemm_rs(a[rank], b[rank], peers, rank)
    total = sum(a[r].float() @ b[r].float().t() for r in range(world))
    for owner in range(world):
        res = torch.randn(rows, N, device="cuda").to(torch.bfloat16)
        out = torch.empty(rows, N, device="cuda", dtype=torch.bfloat16)
        C.sum_partials(outs[owner], res, out, world)
        want = total[owner * rows:(owner + 1) * rows] + res.float()
        assert ((out.float() - want).norm() / want.norm()).item() < 1e-2
    C.check_status()
