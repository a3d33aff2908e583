"""Run-to-run bitwise equality of the kernels that have a fixed summation order (everything except the GEMMs that cut
their contraction into atomically reduced parts), on fresh output buffers poisoned with NaN: a kernel that reads its
own output, leaves part of it unwritten, or races shows up as a difference or a NaN."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _twice(fn):
    a = fn()
    b = fn()
    a = a if isinstance(a, (tuple, list)) else (a,)
    b = b if isinstance(b, (tuple, list)) else (b,)
    for x, y in zip(a, b):
        assert not torch.isnan(x.float()).any(), "poison left in the output"
        assert torch.equal(x, y)


def _poison(*shape, dtype=torch.bfloat16):
    return torch.full(shape, float("nan"), device="cuda", dtype=dtype)


def test_gemm_forms_repeat_bitwise():
    from maester_b200.ops import cuda as C
    torch.manual_seed(0)
    M, N, K = 1024, 768, 1536
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    for two in (False, True):
        _twice(lambda: C.gemm(x, w, out=_poison(M, N), two_cta=two))
        _twice(lambda: C.gemm(dy, w, b_mn=True, out=_poison(M, K), two_cta=two))
        _twice(lambda: C.gemm(dy, x, a_mn=True, b_mn=True, out=_poison(N, K, dtype=torch.float32), epi=C.EPI_F32,
                              two_cta=two))
    _twice(lambda: C.syrk(x))
    C.check_status()


def test_glu_epilogues_and_cross_entropy_repeat_bitwise():
    from maester_b200.ops import cuda as C
    torch.manual_seed(1)
    M, D, F, V = 512, 256, 1024, 5000
    x = torch.randn(M, D, device="cuda", dtype=torch.bfloat16)
    wgu = torch.randn(2 * F, D, device="cuda", dtype=torch.bfloat16) * 0.05
    wd = torch.randn(D, F, device="cuda", dtype=torch.bfloat16) * 0.05
    dy = torch.randn(M, D, device="cuda", dtype=torch.bfloat16)
    _twice(lambda: C.gemm_glu_fwd(x, wgu, 0))
    gu, _ = C.gemm_glu_fwd(x, wgu, 0)
    _twice(lambda: C.gemm_glu_bwd(dy, wd, gu, 0))
    wv = torch.randn(V, D, device="cuda", dtype=torch.bfloat16) * 0.05
    labels = torch.randint(0, V, (M,), device="cuda")
    gs = torch.full((1,), 1.0 / M, device="cuda")

    def ce():
        logits, stats, tgt = C.gemm_ce(x, wv, labels, logits=_poison(M, V))
        rec = _poison(M, 4, dtype=torch.float32)
        C.ce_merge(stats, tgt, rec)
        C.ce_grad(logits, labels, [rec.data_ptr()], None, gs)
        return logits, rec
    _twice(ce)
    C.check_status()


@pytest.mark.parametrize("hd,window,docs", [(256, 0, False), (256, 128, True), (128, 0, True)])
def test_attention_forward_and_backward_repeat_bitwise(hd, window, docs):
    from maester_b200.ops import cuda as C
    from maester_b200.ops.functional import attention_plan
    torch.manual_seed(2)
    B, S, H, KV = 2, 1024, 4, 2
    q = torch.randn(B, S, H, hd, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, S, KV, hd, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(B, S, KV, hd, device="cuda", dtype=torch.bfloat16)
    do = torch.randn(B, S, H, hd, device="cuda", dtype=torch.bfloat16)
    doc = None
    if docs:
        doc = torch.zeros(B, S, dtype=torch.int32, device="cuda")
        doc[:, 300:] = 1
        doc[:, 777:] = 2
    plan = attention_plan(S, window, doc, q.device, B)
    scale = hd ** -0.5
    _twice(lambda: C.attn_fwd(q, k, v, scale, True, window, plan))
    out, lse = C.attn_fwd(q, k, v, scale, True, window, plan)

    def bwd():
        dqkv = _poison(B * S, (H + 2 * KV) * hd)
        C.attn_bwd(q, k, v, out, do, lse, dqkv, scale, True, window, plan)
        return dqkv
    _twice(bwd)
    C.check_status()


def test_norms_rope_and_optimizer_repeat_bitwise():
    from maester_b200.ops import cuda as C
    torch.manual_seed(3)
    M, D = 2048, 2560
    x = torch.randn(M, D, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(D, device="cuda", dtype=torch.bfloat16) * 0.1
    res = torch.randn(M, D, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(M, D, device="cuda", dtype=torch.bfloat16)
    _twice(lambda: C.rmsnorm_fwd(x, w, 1e-6, True, res))
    y, rstd = C.rmsnorm_fwd(x, w, 1e-6, True, None)

    def nb():
        dw = torch.zeros(D, device="cuda")
        return C.rmsnorm_bwd(dy, x, w, rstd, True, dw)   # dw is summed with atomics across blocks: not checked
    _twice(nb)
    C.check_status()


def test_checked_build_runs_the_kernels_without_a_report():
    """The checked build (index checks in front of the kernels' global stores, a failing check skips the store and
    records a status code) runs in a process of its own, selected by MB_CHECKED_KERNELS=1: same results within
    tolerance, status word clean."""
    import os
    import subprocess
    import sys
    code = r'''
import torch
from maester_b200.ops import _lib, cuda as C
assert _lib.CHECKED and _lib.LIB_PATH.name.endswith("_checked.so")
torch.manual_seed(0)
x = torch.randn(1000, 328, device="cuda", dtype=torch.bfloat16)
w = torch.randn(520, 328, device="cuda", dtype=torch.bfloat16) * 0.05
y = C.gemm(x, w)
want = x.float() @ w.float().T
assert ((y.float() - want).norm() / want.norm()).item() < 1e-2
wgu = torch.randn(512, 328, device="cuda", dtype=torch.bfloat16) * 0.05
gu, a = C.gemm_glu_fwd(x, wgu, 1)
labels = torch.randint(0, 520, (1000,), device="cuda")
logits, stats, tgt = C.gemm_ce(x, w, labels)
rec = torch.empty(1000, 4, device="cuda")
C.ce_merge(stats, tgt, rec)
lse = torch.logsumexp(logits.float(), dim=1)
assert ((rec[:, 0] + rec[:, 1].log()) - lse).abs().max().item() < 2e-4
q = torch.randn(1, 512, 4, 128, device="cuda", dtype=torch.bfloat16)
k = torch.randn(1, 512, 2, 128, device="cuda", dtype=torch.bfloat16)
out, l = C.attn_fwd(q, k, k, 128 ** -0.5, True, None, None)
assert torch.isfinite(out.float()).all()
C.set_norm_pipeline(True)
xn = torch.randn(4099, 2560, device="cuda", dtype=torch.bfloat16)
yn, rstd = C.rmsnorm_fwd(xn, torch.zeros(2560, device="cuda", dtype=torch.bfloat16), 1e-6, True)
assert torch.isfinite(yn.float()).all()
C.check_status()
print("checked build ok")
'''
    env = dict(os.environ, MB_CHECKED_KERNELS="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "checked build ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
