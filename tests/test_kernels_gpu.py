"""CUDA kernels against the plain-PyTorch fp32 oracle (maester_b200/ops/reference.py)."""
import math

import pytest
import torch

from maester_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _status():
    from maester_b200.ops import cuda as C
    yield
    C.check_status()


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (300, 520, 136), (1024, 2560, 4096), (77, 40, 72)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    from maester_b200.ops import cuda as C
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a pitch that is a multiple of 8")
    torch.manual_seed(0)
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    want = A.float() @ B.float().T
    a = A.T.contiguous() if a_mn else A
    b = B.T.contiguous() if b_mn else B
    got = C.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    C.check_status()
    assert _rel(got, want) < 5e-3
    got32 = C.gemm(a, b, a_mn=a_mn, b_mn=b_mn, epi=C.EPI_F32)
    assert _rel(got32, want) < 1e-5 * math.sqrt(K) + 1e-4
    acc = torch.ones(M, N, device="cuda")
    C.gemm(a, b, a_mn=a_mn, b_mn=b_mn, epi=C.EPI_F32_ACC, out=acc, alpha=0.5)
    assert _rel(acc, 1 + 0.5 * want) < 1e-4


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 320), (1000, 520, 136), (2048, 2560, 4096), (300, 40, 72)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_two_cta(M, N, K, a_mn, b_mn):
    from maester_b200.ops import cuda as C
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a pitch that is a multiple of 8")
    torch.manual_seed(0)
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    want = A.float() @ B.float().T
    a = A.T.contiguous() if a_mn else A
    b = B.T.contiguous() if b_mn else B
    got = C.gemm(a, b, a_mn=a_mn, b_mn=b_mn, two_cta=True)
    C.check_status()
    assert _rel(got, want) < 5e-3
    acc = torch.ones(M, N, device="cuda")
    C.gemm(a, b, a_mn=a_mn, b_mn=b_mn, epi=C.EPI_F32_ACC, out=acc, alpha=0.5, two_cta=True)
    assert _rel(acc, 1 + 0.5 * want) < 1e-4
    one = C.gemm(a, b, a_mn=a_mn, b_mn=b_mn, two_cta=False)
    assert torch.equal(one, got)


def test_gemm_residual_epilogue():
    from maester_b200.ops import cuda as C
    A = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(768, 512, device="cuda", dtype=torch.bfloat16)
    R = torch.randn(256, 768, device="cuda", dtype=torch.bfloat16)
    got = C.gemm(A, B, epi=C.EPI_BF16_ADD, aux=R)
    assert _rel(got, A.float() @ B.float().T + R.float()) < 5e-3


@pytest.mark.parametrize("M,D", [(64, 256), (1000, 2560), (33, 4096), (16, 5376)])
@pytest.mark.parametrize("unit", [False, True])
def test_rmsnorm(M, D, unit):
    from maester_b200.ops import cuda as C
    x = torch.randn(M, D, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(D, device="cuda") * 0.1).to(torch.bfloat16)
    res = torch.randn(M, D, device="cuda", dtype=torch.bfloat16)
    y, rstd = C.rmsnorm_fwd(x, w, 1e-6, unit)
    assert _rel(y, ref.rmsnorm(x.float(), w.float(), 1e-6, unit)) < 4e-3
    y2, _ = C.rmsnorm_fwd(x, w, 1e-6, unit, residual=res)
    assert _rel(y2, ref.rmsnorm(x, w, 1e-6, unit, residual=res)) < 4e-3
    # backward
    dy = torch.randn(M, D, device="cuda", dtype=torch.bfloat16)
    xf = x.float().requires_grad_()
    wf = w.float().requires_grad_()
    ref.rmsnorm(xf, wf, 1e-6, unit).backward(dy.float())
    dw = torch.zeros(D, device="cuda")
    dx = C.rmsnorm_bwd(dy, x, w, rstd, unit, dw)
    assert _rel(dx, xf.grad) < 5e-3
    assert _rel(dw, wf.grad) < 5e-3


@pytest.mark.parametrize("M,D", [(1185, 256), (4099, 2560), (2400, 1024), (3000, 2048), (1300, 3072), (16384, 2560)])
@pytest.mark.parametrize("unit", [False, True])
@pytest.mark.parametrize("pipeline", [True, False])
def test_rmsnorm_on_tall_inputs(M, D, unit, pipeline):
    """Inputs tall enough for the pipelined kernels (a ring of shared-memory stages filled by bulk copies): ragged last
    tile, every vector width, residual / gradient-accumulate streams, and the same results as the row-per-warp form."""
    from maester_b200.ops import cuda as C
    C.set_norm_pipeline(pipeline)
    try:
        _check_tall_rmsnorm(C, M, D, unit)
    finally:
        C.set_norm_pipeline(False)


def _check_tall_rmsnorm(C, M, D, unit):
    torch.manual_seed(M + D)
    x = torch.randn(M, D, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(D, device="cuda") * 0.1).to(torch.bfloat16)
    res = torch.randn(M, D, device="cuda", dtype=torch.bfloat16)
    y, rstd = C.rmsnorm_fwd(x, w, 1e-6, unit)
    want = ref.rmsnorm(x.float(), w.float(), 1e-6, unit)
    assert _rel(y, want) < 4e-3
    assert (y.float() - want).abs().max().item() < 0.05 * want.abs().max().item()
    assert _rel(rstd, torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)) < 1e-5
    y2, _ = C.rmsnorm_fwd(x, w, 1e-6, unit, residual=res)
    assert _rel(y2, ref.rmsnorm(x, w, 1e-6, unit, residual=res)) < 4e-3
    dy = torch.randn(M, D, device="cuda", dtype=torch.bfloat16)
    xf = x.float().requires_grad_()
    wf = w.float().requires_grad_()
    ref.rmsnorm(xf, wf, 1e-6, unit).backward(dy.float())
    dw = torch.zeros(D, device="cuda")
    dx = C.rmsnorm_bwd(dy, x, w, rstd, unit, dw)
    assert _rel(dx, xf.grad) < 5e-3
    assert _rel(dw, wf.grad) < 5e-3
    add = torch.randn(M, D, device="cuda", dtype=torch.bfloat16)
    dw2 = torch.zeros(D, device="cuda")
    dx2 = C.rmsnorm_bwd(dy, x, w, rstd, unit, dw2, dres_add=add)
    assert _rel(dx2, xf.grad + add.float()) < 5e-3
    assert _rel(dw2, wf.grad) < 5e-3
    dx3 = C.rmsnorm_bwd(dy, x, w, rstd, unit, None)          # no weight gradient wanted
    assert torch.equal(dx3, dx)
    C.check_status()


@pytest.mark.parametrize("hd,rot,layout", [(256, 256, "half"), (128, 128, "interleaved"), (128, 64, "half"), (64, 64, "interleaved")])
@pytest.mark.parametrize("norm", [True, False])
def test_qknorm_rope(hd, rot, layout, norm):
    from maester_b200.ops import cuda as C
    torch.manual_seed(1)
    B, S, H, KV = 2, 96, 4, 2
    T = B * S
    qkv = torch.randn(T, (H + 2 * KV) * hd, device="cuda", dtype=torch.bfloat16)
    qw = (torch.randn(hd, device="cuda") * 0.1).to(torch.bfloat16) if norm else None
    kw = (torch.randn(hd, device="cuda") * 0.1).to(torch.bfloat16) if norm else None
    pos = torch.randint(0, 500, (B, S), device="cuda")
    inv = ref.rope_inv_freq(rot, 10000.0, device="cuda")
    ang = torch.arange(512, device="cuda").float()[:, None] * inv[None]
    cs = torch.stack([ang.cos(), ang.sin()], dim=-1).contiguous()
    lay = 0 if layout == "half" else 1
    out = C.qknorm_rope_fwd(qkv, qw, kw, pos.reshape(-1).int(), cs, H, KV, hd, lay, 1e-6, True)
    q = qkv[:, : H * hd].view(B, S, H, hd)
    k = qkv[:, H * hd:(H + KV) * hd].view(B, S, KV, hd)
    qf, kf = q.float().requires_grad_(), k.float().requires_grad_()
    qwf = qw.float().requires_grad_() if norm else None
    kwf = kw.float().requires_grad_() if norm else None
    rq, rk = ref.qk_norm_rope(qf, kf, qwf, kwf, pos, inv, layout, 1e-6, True)
    want = torch.cat([rq.reshape(T, -1), rk.reshape(T, -1)], dim=1)
    assert _rel(out, want) < 6e-3
    g = torch.randn_like(out)
    want.backward(g.float())
    dqk = g.clone()
    dqw = torch.zeros(hd, device="cuda") if norm else None
    dkw = torch.zeros(hd, device="cuda") if norm else None
    C.qknorm_rope_bwd(dqk, qkv, qw, kw, pos.reshape(-1).int(), cs, dqw, dkw, H, KV, hd, lay, 1e-6, True)
    wantg = torch.cat([qf.grad.reshape(T, -1), kf.grad.reshape(T, -1)], dim=1)
    assert _rel(dqk, wantg) < 8e-3
    if norm:
        assert _rel(dqw, qwf.grad) < 8e-3
        assert _rel(dkw, kwf.grad) < 8e-3


@pytest.mark.parametrize("act", [0, 1])
def test_glu(act):
    from maester_b200.ops import cuda as C
    x = torch.randn(300, 2 * 640, device="cuda", dtype=torch.bfloat16)
    f = ref.geglu if act == 0 else ref.swiglu
    assert _rel(C.glu_fwd(x, act), f(x.float())) < 4e-3
    xf = x.float().requires_grad_()
    d = torch.randn(300, 640, device="cuda", dtype=torch.bfloat16)
    f(xf).backward(d.float())
    assert _rel(C.glu_bwd(x, d, act), xf.grad) < 5e-3


@pytest.mark.parametrize("act,name", [(0, "gelu_tanh"), (1, "silu")])
@pytest.mark.parametrize("M,K,F,D", [(256, 128, 128, 64), (1000, 320, 384, 136), (2048, 2560, 1024, 2560)])
def test_glu_mlp_fused_epilogues(act, name, M, K, F, D):
    """Gate|up GEMM with the activation in its epilogue, and the down projection's input-gradient GEMM with the
    activation's derivative in its epilogue, against the fp32 definition (values and all gradients)."""
    from maester_b200.ops import cuda as C
    from maester_b200.ops.functional import glu_mlp
    torch.manual_seed(4)
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    w_gu = (torch.randn(2 * F, K, device="cuda") * K ** -0.5).to(torch.bfloat16).requires_grad_(True)
    w_d = (torch.randn(D, F, device="cuda") * F ** -0.5).to(torch.bfloat16).requires_grad_(True)
    res = torch.randn(M, D, device="cuda", dtype=torch.bfloat16)
    gate_up, a = C.gemm_glu_fwd(x.detach(), w_gu.detach(), act)
    gu_ref = x.detach().float() @ w_gu.detach().float().T
    assert _rel(gate_up, gu_ref) < 5e-3
    g, u = gate_up.float().chunk(2, dim=-1)
    a_ref = (torch.nn.functional.gelu(g, approximate="tanh") if act == 0 else torch.nn.functional.silu(g)) * u
    assert _rel(a, a_ref) < 6e-3
    assert (a.float() - a_ref).abs().max().item() < 2e-2 * a_ref.abs().max().item() + 1e-2
    y = glu_mlp(x, w_gu, w_d, name, residual=res)
    dy = torch.randn_like(y)
    y.backward(dy)
    xf, wf, df = (t.detach().float().requires_grad_(True) for t in (x, w_gu, w_d))
    gf, uf = (xf @ wf.T).chunk(2, dim=-1)
    af = (torch.nn.functional.gelu(gf, approximate="tanh") if act == 0 else torch.nn.functional.silu(gf)) * uf
    yf = af @ df.T + res.float()
    yf.backward(dy.float())
    assert _rel(y, yf) < 8e-3
    for name_, got, want in (("dx", x.grad, xf.grad), ("dw_gu", w_gu.grad, wf.grad), ("dw_down", w_d.grad, df.grad)):
        assert _rel(got, want) < 1.5e-2, (name_, _rel(got, want))


def test_embedding():
    from maester_b200.ops import cuda as C
    w = torch.randn(1000, 256, device="cuda", dtype=torch.bfloat16)
    tok = torch.randint(0, 1000, (4, 50), device="cuda")
    out = C.embedding_fwd(tok, w, 16.0)
    assert torch.equal(out, ref.embedding(tok, w, 16.0))
    d = torch.randn(4, 50, 256, device="cuda", dtype=torch.bfloat16)
    dw = torch.zeros(1000, 256, device="cuda")
    C.embedding_bwd(tok, d, dw, 16.0)
    want = torch.zeros(1000, 256, device="cuda").index_add_(0, tok.reshape(-1), d.reshape(-1, 256).float() * 16.0)
    assert _rel(dw, want) < 1e-5


@pytest.mark.parametrize("V", [1000, 32003, 262208])
def test_cross_entropy(V):
    from maester_b200.ops import cuda as C
    R = 64
    pitch = (V + 7) // 8 * 8  # the kernel needs a row pitch that is a multiple of 8 elements
    logits = (torch.randn(R, pitch, device="cuda") * 3).to(torch.bfloat16)[:, :V]
    labels = torch.randint(0, V, (R,), device="cuda")
    labels[::7] = -100
    lf = logits.float().requires_grad_()
    want = torch.nn.functional.cross_entropy(lf, labels, ignore_index=-100, reduction="sum")
    nvalid = (labels != -100).sum()
    (want / nvalid).backward()
    loss = torch.zeros(1, device="cuda")
    gs = (1.0 / nvalid.float()).reshape(1)
    lg = torch.empty(R, pitch, device="cuda", dtype=torch.bfloat16)[:, :V]
    lg.copy_(logits)
    C.ce_fwd_bwd(lg, labels, loss, gs)
    assert abs(loss.item() - want.item()) / want.item() < 1e-4
    assert _rel(lg, lf.grad) < 1e-2  # bf16 output of the gradient


def test_adamw_flat():
    from maester_b200.ops import cuda as C
    from maester_b200.optimizers.adamw import build_chunk_table
    n = 100_000
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    lp = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    segs = [(0, 60_000, 1.0, 0.1), (60_000, 40_000, 0.5, 0.0)]
    chunks, tensors, nch = build_chunk_table(segs, "cuda")
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    lr = torch.tensor([1e-2], device="cuda")
    for step in (1, 2):
        C.adamw(p, g, m, v, lp, chunks, tensors, nch, lr, 0.9, 0.95, 1e-8, step)
        for off, ln, lrm, wd in segs:
            sl = slice(off, off + ln)
            ref.adamw_step(pr[sl], g[sl], mr[sl], vr[sl], step, 1e-2 * lrm, 0.9, 0.95, 1e-8, wd)
    assert _rel(p, pr) < 1e-5
    assert _rel(lp, pr) < 4e-3


def _attn_case(B, S, H, KV, hd, causal, window, docs):
    from maester_b200.ops import cuda as C
    from maester_b200.ops.functional import attention_plan
    torch.manual_seed(2)
    qkv = torch.randn(B, S, (H + 2 * KV) * hd, device="cuda", dtype=torch.bfloat16)
    q = qkv[..., : H * hd].view(B, S, H, hd)
    k = qkv[..., H * hd:(H + KV) * hd].view(B, S, KV, hd)
    v = qkv[..., (H + KV) * hd:].view(B, S, KV, hd)
    doc = None
    if docs:
        doc = torch.zeros(B, S, dtype=torch.int32, device="cuda")
        for b in range(B):
            cuts = sorted(torch.randint(1, max(2, S), (3,)).tolist())
            for c in cuts:
                doc[b, c:] += 1
    scale = hd ** -0.5
    plan = attention_plan(S, window, doc, "cuda", batch=B, causal=causal)
    out, lse = C.attn_fwd(q, k, v, scale, causal, window, plan)
    C.check_status()
    want, wlse = ref.attention(q, k, v, scale, causal, window, doc, return_lse=True)
    assert _rel(out, want) < 1e-2, _rel(out, want)
    assert (out.float() - want.float()).abs().max().item() < 6e-2  # no wrong row hides in a norm
    assert (lse - wlse).abs().max().item() < 2e-2


@pytest.mark.parametrize("hd", [64, 128, 256])
@pytest.mark.parametrize("causal,window,docs", [(True, None, False), (True, 100, False), (True, None, True), (True, 64, True), (False, None, False),
                                                (False, None, True)])
def test_attention_fwd(hd, causal, window, docs):
    _attn_case(2, 384, 4, 2, hd, causal, window, docs)


def test_attention_fwd_ragged_len():
    _attn_case(1, 200, 2, 1, 128, True, None, False)
    _attn_case(1, 333, 2, 2, 256, True, 50, True)
    _attn_case(1, 64, 2, 2, 256, True, None, False)      # a single kv block: the second softmax set stays idle
    _attn_case(1, 1, 2, 1, 128, True, None, True)        # one token
    _attn_case(2, 1100, 4, 2, 256, True, 300, True)      # many blocks, window wider than a document


def _packed_docs(B, S, mean, seed):
    import numpy as np
    rng = np.random.default_rng(seed)
    doc = torch.zeros(B, S, dtype=torch.int32)
    for b in range(B):
        i = d = 0
        while i < S:
            j = min(S, i + max(1, int(rng.geometric(1.0 / mean))))
            doc[b, i:j] = d
            i, d = j, d + 1
    return doc.cuda()


@pytest.mark.parametrize("window", [None, 1024])
def test_attention_benchmark_shape_fwd_bwd(window):
    """The shape of the headline benchmark (sequence 8192, 8 query / 4 kv heads of 256, window 1024 or global,
    geometric documents) against the fp32 definition, element by element: a wrong row or a mask slip at a tile
    boundary of a long sequence cannot hide in a norm.  The oracle runs one head group at a time to bound memory."""
    from maester_b200.ops import cuda as C
    from maester_b200.ops.functional import attention_plan
    B, S, H, KV, hd = 1, 8192, 8, 4, 256
    torch.manual_seed(7)
    doc = _packed_docs(B, S, 700.0, 3)
    qkv = (torch.randn(B, S, (H + 2 * KV) * hd, device="cuda") * 0.7).to(torch.bfloat16)
    q = qkv[..., : H * hd].view(B, S, H, hd)
    k = qkv[..., H * hd:(H + KV) * hd].view(B, S, KV, hd)
    v = qkv[..., (H + KV) * hd:].view(B, S, KV, hd)
    scale = hd ** -0.5
    plan = attention_plan(S, window, doc, "cuda", batch=B)
    out, lse = C.attn_fwd(q, k, v, scale, True, window, plan)
    dout = (torch.randn_like(out) * 0.5)
    dqkv = torch.zeros(B * S, (H + 2 * KV) * hd, device="cuda", dtype=torch.bfloat16)
    C.attn_bwd(q, k, v, out, dout, lse, dqkv, scale, True, window, plan)
    C.check_status()
    G = H // KV
    for g in range(KV):  # oracle per kv head (its G query heads), fp32, dense mask
        qf = q[:, :, g * G:(g + 1) * G].float().detach().requires_grad_(True)
        kf = k[:, :, g:g + 1].float().detach().requires_grad_(True)
        vf = v[:, :, g:g + 1].float().detach().requires_grad_(True)
        want, wlse = ref.attention(qf, kf, vf, scale, True, window, doc, return_lse=True)
        want.backward(dout[:, :, g * G:(g + 1) * G].float())
        got = out[:, :, g * G:(g + 1) * G].float()
        assert (got - want).abs().max().item() < 4e-2, (g, (got - want).abs().max().item())
        assert _rel(got, want) < 1e-2
        assert (lse[:, g * G:(g + 1) * G] - wlse).abs().max().item() < 2e-2
        d = dqkv.view(B, S, -1).float()
        dq = d[..., g * G * hd:(g + 1) * G * hd].view(B, S, G, hd)
        dk = d[..., (H + g) * hd:(H + g + 1) * hd].view(B, S, 1, hd)
        dv = d[..., (H + KV + g) * hd:(H + KV + g + 1) * hd].view(B, S, 1, hd)
        for name, a, w in (("dq", dq, qf.grad), ("dk", dk, kf.grad), ("dv", dv, vf.grad)):
            assert _rel(a, w) < 2e-2, (name, g, _rel(a, w))
            assert (a - w).abs().max().item() < 0.05 * w.abs().max().item() + 2e-2, (name, g)
        del qf, kf, vf, want


def _attn_bwd_case(B, S, H, KV, hd, causal, window, docs):
    from maester_b200.ops.functional import attention_block
    torch.manual_seed(3)
    qkv = (torch.randn(B, S, (H + 2 * KV) * hd, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    doc = None
    if docs:
        doc = torch.zeros(B, S, dtype=torch.int32, device="cuda")
        for b in range(B):
            for c in sorted(torch.randint(1, S, (3,)).tolist()):
                doc[b, c:] += 1
    scale = hd ** -0.5
    out = attention_block(qkv, None, None, None, None, None, doc, H, KV, hd, scale=scale, causal=causal, window=window)
    g = torch.randn_like(out)
    out.backward(g)
    qf = qkv.detach().float().requires_grad_()
    want = attention_block(qf, None, None, None, None, None, doc, H, KV, hd, scale=scale, causal=causal, window=window)
    want.backward(g.float())
    assert _rel(out, want) < 1e-2
    for name, sl in (("dq", slice(0, H * hd)), ("dk", slice(H * hd, (H + KV) * hd)), ("dv", slice((H + KV) * hd, None))):
        r = _rel(qkv.grad[..., sl], qf.grad[..., sl])
        assert r < 2e-2, (name, r)


@pytest.mark.parametrize("hd", [64, 128, 256])
@pytest.mark.parametrize("causal,window,docs", [(True, None, False), (True, 100, False), (True, 64, True), (False, None, False)])
def test_attention_bwd(hd, causal, window, docs):
    _attn_bwd_case(2, 384, 4, 2, hd, causal, window, docs)


def test_attention_bwd_ragged():
    _attn_bwd_case(1, 200, 4, 1, 128, True, None, True)
    _attn_bwd_case(1, 333, 2, 2, 256, True, 50, True)


def test_attention_block_norm_rope_grads():
    from maester_b200.ops.functional import attention_block, rope_table
    torch.manual_seed(4)
    B, S, H, KV, hd = 2, 256, 4, 2, 256
    qkv = (torch.randn(B, S, (H + 2 * KV) * hd, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    qw = (torch.randn(hd, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_()
    kw = (torch.randn(hd, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_()
    inv = ref.rope_inv_freq(hd, 10000.0, device="cuda")
    cs = rope_table(inv, 1024)
    pos = torch.arange(S, device="cuda")[None].expand(B, S).contiguous()
    out = attention_block(qkv, qw, kw, pos, inv, cs, None, H, KV, hd, unit_offset=True, window=64)
    g = torch.randn_like(out)
    out.backward(g)
    qf, qwf, kwf = (t.detach().float().requires_grad_() for t in (qkv, qw, kw))
    want = attention_block(qf, qwf, kwf, pos, inv, None, None, H, KV, hd, unit_offset=True, window=64)
    want.backward(g.float())
    assert _rel(out, want) < 1.5e-2
    assert _rel(qkv.grad, qf.grad) < 3e-2
    assert _rel(qw.grad, qwf.grad) < 3e-2
    assert _rel(kw.grad, kwf.grad) < 3e-2


def test_linear_autograd_and_main_grad():
    from maester_b200.ops.functional import linear
    x = torch.randn(4, 100, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(384, 256, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    y = linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    (xf @ wf.T).backward(g.float())
    assert _rel(y, xf @ wf.T) < 5e-3
    assert _rel(x.grad, xf.grad) < 5e-3
    assert _rel(w.grad, wf.grad) < 5e-3
    w2 = w.detach().clone().requires_grad_()
    w2.main_grad = torch.zeros(384, 256, device="cuda")
    for _ in range(2):
        linear(x.detach(), w2).backward(g)
    assert w2.grad is None
    assert _rel(w2.main_grad, 2 * wf.grad) < 5e-3


def test_linear_cross_entropy_fused():
    from maester_b200.ops.functional import linear_cross_entropy
    import maester_b200.ops.functional as Fm
    torch.manual_seed(5)
    M, D, V = 700, 256, 5000
    h = torch.randn(M, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(V, D, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    labels = torch.randint(0, V, (M,), device="cuda")
    labels[::5] = -100
    old = Fm.CE_CHUNK_ROWS
    Fm.CE_CHUNK_ROWS = 256
    try:
        loss = linear_cross_entropy(h, w, labels)
        (loss * 0.5).backward()
    finally:
        Fm.CE_CHUNK_ROWS = old
    hf, wf = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    want = ref.linear_cross_entropy(hf, wf, labels)
    (want * 0.5).backward()
    assert abs(loss.item() - want.item()) < 2e-2
    assert _rel(h.grad, hf.grad) < 2e-2
    assert _rel(w.grad, wf.grad) < 2e-2


@pytest.mark.parametrize("M,D,V,scale", [(300, 256, 5000, 1.0), (512, 640, 262208, 1.0), (130, 128, 1000, 0.5)])
def test_logits_gemm_leaves_online_lse_records(M, D, V, scale):
    """The logits GEMM's epilogue statistics (per 256-column tile) merge to the exact row log-sum-exp and target."""
    from maester_b200.ops import cuda as C
    torch.manual_seed(2)
    h = torch.randn(M, D, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(V, D, device="cuda") * 0.2).to(torch.bfloat16)
    labels = torch.randint(0, V, (M,), device="cuda")
    labels[::9] = -100
    logits, stats, tgt = C.gemm_ce(h, w, labels, 0, scale)
    want = (h.float() @ w.float().T) * scale
    assert (logits.float() - want).abs().max().item() < 0.02 * want.abs().max().item() + 1e-2
    rec = torch.empty(M, 4, device="cuda")
    C.ce_merge(stats, tgt, rec)
    lf = logits.float()                      # the records describe the stored (rounded) logits exactly
    lse = torch.logsumexp(lf, dim=1)
    got = rec[:, 0] + rec[:, 1].log()
    assert (got - lse).abs().max().item() < 2e-4
    valid = labels != -100
    pick = lf.gather(1, labels.clamp_min(0)[:, None]).squeeze(1)
    assert torch.equal(rec[valid, 2], pick[valid]) and bool((rec[~valid, 2] == 0).all())
    # without storing logits the records are the same
    none, stats2, tgt2 = C.gemm_ce(h, w, labels, 0, scale, store_logits=False)
    assert none is None and torch.equal(stats2, stats) and torch.equal(tgt2, tgt)
    # loss and gradient from the records
    loss = torch.zeros(1, device="cuda")
    gs = (1.0 / valid.sum().float()).reshape(1)
    C.ce_grad(logits, labels, [rec.data_ptr()], loss, gs)
    lr = lf.clone().requires_grad_()
    ref_loss = torch.nn.functional.cross_entropy(lr, labels, ignore_index=-100, reduction="sum")
    (ref_loss * gs).backward()
    assert abs(loss.item() - ref_loss.item()) / ref_loss.item() < 1e-4
    assert _rel(logits, lr.grad) < 1e-2
    C.check_status()


def test_vocabulary_slices_combine_through_their_records():
    """Two slices of the vocabulary, each with its own records: the combined loss and gradients equal the whole."""
    from maester_b200.ops import cuda as C
    torch.manual_seed(3)
    M, D, V = 200, 256, 3216
    h = torch.randn(M, D, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(V, D, device="cuda") * 0.2).to(torch.bfloat16)
    labels = torch.randint(0, V, (M,), device="cuda")
    labels[::4] = -100
    halves, recs = [], []
    for r in range(2):
        v0 = r * (V // 2)
        lg, st, tg = C.gemm_ce(h, w[v0:v0 + V // 2], labels, v0)
        rec = torch.empty(M, 4, device="cuda")
        C.ce_merge(st, tg, rec)
        halves.append(lg)
        recs.append(rec)
    full = torch.cat([x.float() for x in halves], dim=1).requires_grad_()
    ref_loss = torch.nn.functional.cross_entropy(full, labels, ignore_index=-100, reduction="sum")
    gs = (1.0 / (labels != -100).sum().float()).reshape(1)
    (ref_loss * gs).backward()
    for r in range(2):
        loss = torch.zeros(1, device="cuda")
        C.ce_grad(halves[r], labels, [x.data_ptr() for x in recs], loss, gs, v0=r * (V // 2))
        assert abs(loss.item() - ref_loss.item()) / ref_loss.item() < 1e-4
        assert _rel(halves[r], full.grad[:, r * (V // 2):(r + 1) * (V // 2)]) < 1e-2


@pytest.mark.parametrize("mode", ["stored", "recomputed", "ahead"])
def test_linear_cross_entropy_modes_agree_with_the_oracle(mode):
    from maester_b200 import ops
    from maester_b200.ops import cuda as C
    import maester_b200.ops.functional as Fm
    torch.manual_seed(6)
    M, D, V = 900, 256, 6008
    h = torch.randn(M, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(V, D, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    labels = torch.randint(0, V, (M,), device="cuda")
    labels[::5] = -100
    old = Fm.CE_CHUNK_ROWS, Fm.CE_STORE_LIMIT_BYTES
    Fm.CE_CHUNK_ROWS = 256
    if mode == "recomputed":
        Fm.CE_STORE_LIMIT_BYTES = 0
    try:
        with ops.loss_backward_scale(0.25 if mode == "ahead" else None):
            loss = ops.linear_cross_entropy(h, w, labels, 0.5)
        (loss * 0.25).backward()
    finally:
        Fm.CE_CHUNK_ROWS, Fm.CE_STORE_LIMIT_BYTES = old
    hf, wf = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    want = ref.linear_cross_entropy(hf, wf, labels, 0.5)
    (want * 0.25).backward()
    assert abs(loss.item() - want.item()) < 2e-2
    assert _rel(h.grad, hf.grad) < 2e-2
    assert _rel(w.grad, wf.grad) < 2e-2
    C.check_status()


def test_a_broken_gradient_promise_is_reported_not_ignored():
    from maester_b200 import ops
    from maester_b200.ops import cuda as C
    h = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(512, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    labels = torch.randint(0, 512, (256,), device="cuda")
    with ops.loss_backward_scale(1.0):
        loss = ops.linear_cross_entropy(h, w, labels)
    (loss * 3.0).backward()
    with pytest.raises(RuntimeError, match="different output gradient"):
        C.check_status()
    C.check_status()   # the status word was cleared: later work is unaffected


@pytest.mark.parametrize("Mo,No,K", [(4096, 2560, 4096), (2560, 2048, 8192), (5120, 2560, 1024), (1024, 512, 4096),
                                      (4104, 2568, 2048), (4104, 2312, 4096)])
def test_accumulating_gemm_splits_only_the_tail_wave(Mo, No, K):
    """C += A^T B (the weight-gradient form, fp32 accumulate) over shapes whose tiles fill whole waves plus a tail
    (whole tiles read-modify-write, tail tiles cut and merged with atomics), exactly whole waves, fewer tiles than
    CTA pairs (every tile cut), and ragged edges; repeated calls keep accumulating."""
    from maester_b200.ops import cuda as C
    torch.manual_seed(Mo + No)
    dy = (torch.randn(K, Mo, device="cuda") * 0.1).to(torch.bfloat16)
    x = (torch.randn(K, No, device="cuda") * 0.1).to(torch.bfloat16)
    buf = torch.randn(Mo, No, device="cuda")
    want = buf.clone()
    for _ in range(2):
        C.gemm(dy, x, a_mn=True, b_mn=True, out=buf, epi=C.EPI_F32_ACC)
        want += dy.float().T @ x.float()
    assert _rel(buf, want) < 2e-3
    assert (buf - want).abs().max().item() < 2e-2 * want.abs().max().item()
    C.check_status()


def test_attention_block_with_recomputed_qk_matches_the_kept_form():
    """The per-op recomputation plan (rotated q / k rebuilt in backward) changes no number."""
    from maester_b200 import ops
    torch.manual_seed(4)
    B, S, H, KV, hd = 2, 512, 4, 2, 128
    qkv0 = torch.randn(B, S, (H + 2 * KV) * hd, device="cuda", dtype=torch.bfloat16)
    qw = (torch.randn(hd, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_()
    kw = (torch.randn(hd, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_()
    pos = torch.arange(S, device="cuda", dtype=torch.int32)[None].expand(B, S)
    cs = ops.rope_table(ref.rope_inv_freq(hd, 10000.0, device="cuda"), 1024)
    do = torch.randn(B, S, H * hd, device="cuda", dtype=torch.bfloat16)
    res = []
    for rc in (False, True):
        qkv = qkv0.clone().requires_grad_()
        qw.grad = kw.grad = None
        out = ops.attention_block(qkv, qw, kw, pos, None, cs, None, H, KV, hd, eps=1e-6, unit_offset=True,
                                  recompute_qk=rc)
        out.backward(do)
        res.append((out.detach(), qkv.grad, qw.grad.clone(), kw.grad.clone()))
    for a, b in zip(*res):
        assert torch.equal(a, b)


@pytest.mark.parametrize("M,K", [(256, 64), (1000, 328), (2560, 2560)])
def test_syrk_triangular_schedule(M, K):
    """A A^T (+ beta C) computed on the tiles below the diagonal and mirrored equals the full product."""
    from maester_b200.ops import cuda as C
    torch.manual_seed(1)
    a = (torch.randn(M, K, device="cuda") * K ** -0.5).to(torch.bfloat16)
    want = a.float() @ a.float().T
    got = C.syrk(a)
    assert _rel(got, want) < 5e-3
    assert torch.equal(got, got.T.contiguous())          # exactly symmetric: the mirror is a copy
    aux = torch.randn(M, M, device="cuda", dtype=torch.bfloat16)
    got2 = C.syrk(a, aux, alpha=-2.0, beta=0.5)
    assert _rel(got2, -2.0 * want + 0.5 * aux.float()) < 5e-3


def test_newton_schulz_on_triangular_syrk():
    from maester_b200.optimizers.muon import newton_schulz
    torch.manual_seed(2)
    g = torch.randn(512, 1280, device="cuda")
    got = newton_schulz(g.to(torch.bfloat16), steps=5).float()
    want = ref.newton_schulz(g, 5, 1e-7).float()
    assert _rel(got, want) < 6e-2
    s = torch.linalg.svdvals(got)
    assert 0.5 < s.min().item() and s.max().item() < 1.3  # close to an orthogonal factor


def test_multi_tensor_sqnorm_and_scale():
    from maester_b200.ops import cuda as C
    from maester_b200.optimizers.adamw import build_chunk_table
    torch.manual_seed(3)
    sizes = [5, 32768, 70001, 1, 123457]
    flat = torch.randn(sum(sizes) + 64, device="cuda")
    segs, off = [], 3   # an odd start: unaligned chunks take the scalar path
    for n in sizes:
        segs.append((off, n, 1.0, 0.0))
        off += n
    chunks, _, nch = build_chunk_table(segs, "cuda")
    out = torch.zeros(len(sizes), device="cuda")
    C.multi_sqnorm(flat, chunks, nch, out)
    want = torch.stack([flat[o:o + n].double().pow(2).sum() for o, n, _, _ in segs]).float()
    assert torch.allclose(out, want, rtol=1e-5)
    before = flat.clone()
    C.multi_sqnorm(flat, chunks, nch, None, torch.tensor([0.25], device="cuda"))
    for o, n, _, _ in segs:
        assert torch.equal(flat[o:o + n], before[o:o + n] * 0.25)
    assert torch.equal(flat[:3], before[:3])
