"""Kernel micro-benchmarks: ``python -m benchmarks.kernel_bench <op> [--iters N] [--small]``.

``op``: ``gemm`` (forward / dgrad / wgrad layouts of the Gemma-3 4B projections, 1-CTA and CTA-pair
kernels next to ``torch.matmul``), ``attention`` (forward and backward for head sizes 256 and 128,
causal and sliding-window), ``elementwise`` (RMSNorm, GeGLU, AdamW), ``grouped`` (MoE grouped GEMM).
Timing is by CUDA events after warm-up; every iteration's operands exceed the L2 capacity.
``--small`` runs one launch per kernel on a case of a few hundred MB, the size meant for a
profiler capture.  Fractions are of the peaks in ``MEASURED_PEAKS.json`` at the repository root
when that file exists (copy bandwidth and dense bf16 GEMM rate measured on the same machines).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from maester_b200.ops import cuda as C
from maester_b200.ops.functional import attention_plan


def _peaks() -> tuple[float, float]:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        return 1590.0, 6650.0


def timeit(fn, iters: int, warm: int = 3) -> float:
    """Mean milliseconds per call."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def bench_gemm(iters: int, small: bool) -> None:
    tf_peak, _ = _peaks()
    M = 8192 if small else 16384
    shapes = {"qkv": (4096, 2560)} if small else {"qkv": (4096, 2560), "o": (2560, 2048), "gate_up": (20480, 2560),
                                                  "down": (2560, 10240)}
    warm = 0 if small else 3
    for name, (N, K) in shapes.items():
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
        dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
        g32 = torch.zeros(N, K, device="cuda")
        fl = 2 * M * N * K
        cases = {
            "fwd  ": (lambda two: C.gemm(x, w, two_cta=two), lambda: x @ w.T),
            "dgrad": (lambda two: C.gemm(dy, w, b_mn=True, two_cta=two), lambda: dy @ w),
            "wgrad": (lambda two: C.gemm(dy, x, a_mn=True, b_mn=True, out=g32, epi=C.EPI_F32_ACC, two_cta=two),
                      lambda: dy.T @ x),
        }
        for cname, (ours, lib) in cases.items():
            t1 = timeit(lambda: ours(False), iters, warm)
            t2 = timeit(lambda: ours(True), iters, warm)
            tl = timeit(lib, iters, warm)
            print(f"gemm {name:8s} {cname} M{M} N{N} K{K}: 1cta {t1:.3f} ms {fl / t1 / 1e9:6.0f} TF | pair {t2:.3f} ms "
                  f"{fl / t2 / 1e9:6.0f} TF ({fl / t2 / 1e9 / tf_peak:.2f} of measured) | torch {tl:.3f} ms {fl / tl / 1e9:6.0f} TF")
    C.check_status()


def bench_attention(iters: int, small: bool) -> None:
    tf_peak, _ = _peaks()
    B, S = (1, 4096) if small else (2, 8192)
    cfgs = [(8, 4, 256, None)] if small else [(8, 4, 256, None), (8, 4, 256, 1024), (32, 8, 128, None), (16, 16, 64, None)]
    warm = 0 if small else 3
    for H, KV, hd, window in cfgs:
        qkv = torch.randn(B, S, (H + 2 * KV) * hd, device="cuda", dtype=torch.bfloat16)
        q = qkv[..., :H * hd].view(B, S, H, hd)
        k = qkv[..., H * hd:(H + KV) * hd].view(B, S, KV, hd)
        v = qkv[..., (H + KV) * hd:].view(B, S, KV, hd)
        plan = attention_plan(S, window, None, "cuda", batch=B)
        out, lse = C.attn_fwd(q, k, v, hd ** -0.5, True, window, plan)
        dout = torch.randn_like(out)
        dqkv = torch.empty_like(qkv).view(B * S, -1)
        fl = 4 * B * H * hd * S * (S / 2 if window is None else window)
        tf = timeit(lambda: C.attn_fwd(q, k, v, hd ** -0.5, True, window, plan), iters, warm)
        tb = timeit(lambda: C.attn_bwd(q, k, v, out, dout, lse, dqkv, hd ** -0.5, True, window, plan), iters, warm)
        print(f"attention H{H} KV{KV} hd{hd} window={window} B{B} S{S}: fwd {tf:.3f} ms {fl / tf / 1e9:5.0f} TF "
              f"({fl / tf / 1e9 / tf_peak:.2f} of measured) | bwd {tb:.3f} ms {2.5 * fl / tb / 1e9:5.0f} TF "
              f"({2.5 * fl / tb / 1e9 / tf_peak:.2f} of measured)")
    C.check_status()


def bench_elementwise(iters: int, small: bool) -> None:
    _, gbs_peak = _peaks()
    M, D, F = (16384, 2560, 10240)
    warm = 0 if small else 3

    def report(name: str, ms: float, nbytes: int) -> None:
        gbs = nbytes / ms / 1e6
        print(f"{name:22s} {ms * 1e3:8.1f} us {gbs:6.0f} GB/s ({gbs / gbs_peak:.2f} of measured)")

    x = torch.randn(M, D, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(D, device="cuda", dtype=torch.bfloat16)
    report("rmsnorm fwd", timeit(lambda: C.rmsnorm_fwd(x, w, 1e-6, True), iters, warm), 2 * x.numel() * 2)
    _, rstd = C.rmsnorm_fwd(x, w, 1e-6, True)
    dw = torch.zeros(D, device="cuda")
    report("rmsnorm bwd", timeit(lambda: C.rmsnorm_bwd(x, x, w, rstd, True, dw), iters, warm), 3 * x.numel() * 2)
    gu = torch.randn(M, 2 * F, device="cuda", dtype=torch.bfloat16)
    report("geglu fwd", timeit(lambda: C.glu_fwd(gu, 0), iters, warm), gu.numel() * 3)
    do = torch.randn(M, F, device="cuda", dtype=torch.bfloat16)
    report("geglu bwd", timeit(lambda: C.glu_bwd(gu, do, 0), iters, warm), gu.numel() * 2 * 2 + do.numel() * 2)
    H, KV, hd = 8, 4, 256
    qkv = torch.randn(M, (H + 2 * KV) * hd, device="cuda", dtype=torch.bfloat16)
    qw = torch.zeros(hd, device="cuda", dtype=torch.bfloat16)
    pos = (torch.arange(M, device="cuda", dtype=torch.int32) % 8192).contiguous()
    cs = torch.randn(8192, hd // 2, 2, device="cuda")
    nbytes = M * ((H + KV) * hd * 2) * 2
    report("qknorm+rope fwd", timeit(lambda: C.qknorm_rope_fwd(qkv, qw, qw, pos, cs, H, KV, hd, 0, 1e-6, True), iters, warm),
           nbytes)
    dqk = torch.randn(M, (H + 2 * KV) * hd, device="cuda", dtype=torch.bfloat16)
    dqw, dkw = torch.zeros(hd, device="cuda"), torch.zeros(hd, device="cuda")
    report("qknorm+rope bwd", timeit(lambda: C.qknorm_rope_bwd(dqk, qkv, qw, qw, pos, cs, dqw, dkw, H, KV, hd, 0, 1e-6, True),
                                     iters, warm), M * ((H + KV) * hd * 2) * 3)
    if small:
        return
    from maester_b200.optimizers.adamw import FusedAdamW
    n = 512 * 2 ** 20
    p = torch.nn.Parameter(torch.zeros(n, device="cuda"))
    p.grad = torch.randn(n, device="cuda")
    lowp = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    opt = FusedAdamW([p], lr=1e-3)
    opt.attach_flat(p.data, p.grad, lowp, {p: (0, n)}, torch.zeros_like(p.data), torch.zeros_like(p.data))
    report("adamw (512M params)", timeit(opt.step, iters, warm), n * (4 * 4 + 3 * 4 + 2))
    C.check_status()


def bench_grouped(iters: int, small: bool) -> None:
    tf_peak, _ = _peaks()
    from maester_b200.ops.functional import padded_group_offsets
    E, dim, hidden = (8, 2048, 1408) if small else (64, 2048, 1408)
    T = 16384 if small else 6 * 16384
    counts = torch.full((E,), T // E, device="cuda", dtype=torch.int64)
    offs = padded_group_offsets(counts)
    rows = int(offs[-1].item())
    x = torch.randn(rows, dim, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(E, dim, hidden, device="cuda", dtype=torch.bfloat16) * 0.02
    fl = 2 * rows * dim * hidden
    t = timeit(lambda: C.gemm_grouped_rows(x, w, offs, b_mn=True), iters, 0 if small else 3)
    print(f"grouped gemm E{E} rows{rows} {dim}x{hidden}: {t:.3f} ms {fl / t / 1e9:.0f} TF ({fl / t / 1e9 / tf_peak:.2f} of measured)")
    C.check_status()


def bench_moe(iters: int, small: bool) -> None:
    """Routing plan and row kernels of the MoE block (DeepSeek-style: 64 experts, top-6, dim 2048)."""
    _, bw_peak = _peaks()
    T, E, k, D = (4096, 64, 6, 2048) if small else (16384, 64, 6, 2048)
    logits = torch.randn(T, E, device="cuda")
    warm = 0 if small else 3
    t = timeit(lambda: C.moe_route(logits, None, k, True, False, 1.0, False, 128), iters, warm)
    print(f"moe route T{T} E{E} top{k} (score + top-k + stable sort + offsets, 3 kernels + allocations): {t * 1e3:.1f} us")
    p = C.moe_route(logits, None, k, True, False, 1.0, False, 128)
    x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16)
    t = timeit(lambda: C.moe_rows_gather(x, p.row_slot, p.top, k), iters, warm)
    nb = (T * D + p.rows_cap * D) * 2
    print(f"moe rows gather -> [{p.rows_cap}, {D}]: {t * 1e3:.1f} us {nb / t / 1e6:.0f} GB/s ({nb / t / 1e6 / bw_peak:.2f} of measured)")
    buf = torch.randn(p.rows_cap, D, device="cuda", dtype=torch.bfloat16)
    t = timeit(lambda: C.moe_rows_combine(buf, p.slot_row, p.top, k), iters, warm)
    nb = (T * k * D + T * D) * 2
    print(f"moe rows combine -> [{T}, {D}]: {t * 1e3:.1f} us {nb / t / 1e6:.0f} GB/s ({nb / t / 1e6 / bw_peak:.2f} of measured)")
    t = timeit(lambda: C.moe_slot_dot(buf, p.slot_row, x, k), iters, warm)
    print(f"moe slot dot: {t * 1e3:.1f} us {nb / t / 1e6:.0f} GB/s ({nb / t / 1e6 / bw_peak:.2f} of measured)")
    C.check_status()


def bench_ce(iters: int, small: bool) -> None:
    """LM head + cross-entropy of the Gemma-3 4B step (16384 tokens, hidden 2560, vocabulary 262144): the pieces of
    a row chunk, and forward + backward of the whole loss in its modes."""
    from maester_b200 import ops
    import maester_b200.ops.functional as Fm
    tf_peak, bw_peak = _peaks()
    M, D, V = (4096, 2560, 32768) if small else (16384, 2560, 262144)
    Fm.CE_CHUNK_ROWS = int(os.environ.get("MB_CE_CHUNK_ROWS", Fm.CE_CHUNK_ROWS))
    R = min(M, Fm.CE_CHUNK_ROWS)
    warm = 0 if small else 3
    h = (torch.randn(M, D, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(V, D, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_()
    w.main_grad = torch.zeros(V, D, device="cuda")
    labels = torch.randint(0, V, (M,), device="cuda")
    gs = torch.full((1,), 1.0 / M, device="cuda")
    fl = 2 * R * V * D
    buf = torch.empty(R, V, device="cuda", dtype=torch.bfloat16)
    rec = torch.empty(R, 4, device="cuda")
    loss = torch.zeros(1, device="cuda")
    hd, wd = h.detach(), w.detach()
    t = timeit(lambda: C.gemm(hd[:R], wd, out=buf), iters, warm)
    print(f"ce logits GEMM plain          [{R} x {V}]: {t:.3f} ms {fl / t / 1e9:6.0f} TF ({fl / t / 1e9 / tf_peak:.2f} of measured)")
    t = timeit(lambda: C.gemm_ce(hd[:R], wd, labels[:R], logits=buf), iters, warm)
    print(f"ce logits GEMM + LSE records  [{R} x {V}]: {t:.3f} ms {fl / t / 1e9:6.0f} TF ({fl / t / 1e9 / tf_peak:.2f} of measured)")
    t = timeit(lambda: C.gemm_ce(hd[:R], wd, labels[:R], store_logits=False), iters, warm)
    print(f"ce LSE records only (no logits stored)       : {t:.3f} ms {fl / t / 1e9:6.0f} TF")
    _, stats, tgt = C.gemm_ce(hd[:R], wd, labels[:R], logits=buf)
    t = timeit(lambda: C.ce_merge(stats, tgt, rec), iters, warm)
    print(f"ce merge records: {t * 1e3:.1f} us")
    by = 2 * R * V * 2
    t = timeit(lambda: C.ce_grad(buf, labels[:R], [rec.data_ptr()], loss, gs), iters, warm)
    print(f"ce gradient in place (1 read + 1 write): {t * 1e3:.1f} us {by / t / 1e6:.0f} GB/s ({by / t / 1e6 / bw_peak:.2f} of measured)")
    t = timeit(lambda: C.ce_fwd_bwd(buf, labels[:R], loss, gs), iters, warm)
    print(f"ce two-pass kernel (row max/sum, then gradient): {t * 1e3:.1f} us {by / t / 1e6:.0f} GB/s")
    dh32 = torch.zeros(R, D, device="cuda")
    dhb = torch.empty(R, D, device="cuda", dtype=torch.bfloat16)
    fl2 = 2 * R * V * D
    t = timeit(lambda: C.gemm(buf, wd, b_mn=True, out=dhb), iters, warm)
    print(f"ce dH GEMM, bf16 out (one unit per tile)   : {t:.3f} ms {fl2 / t / 1e9:6.0f} TF")
    t = timeit(lambda: C.gemm(buf, wd, b_mn=True, out=dh32, epi=C.EPI_F32_ACC), iters, warm)
    print(f"ce dH GEMM, fp32 accumulate (contraction cut): {t:.3f} ms {fl2 / t / 1e9:6.0f} TF")
    t = timeit(lambda: C.gemm(buf, hd[:R], a_mn=True, b_mn=True, out=w.main_grad, epi=C.EPI_F32_ACC), iters, warm)
    print(f"ce dW GEMM, fp32 accumulate                  : {t:.3f} ms {fl2 / t / 1e9:6.0f} TF")
    for mode in ("stored", "ahead"):
        def step():
            with ops.loss_backward_scale(1.0 if mode == "ahead" else None):
                l = ops.linear_cross_entropy(h, w, labels)
            l.backward()
            h.grad = None
        torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        t = timeit(step, max(1, iters // 2), 1 if small else 2)
        peak = (torch.cuda.max_memory_allocated() - base) / 2 ** 30
        print(f"ce loss fwd+bwd, gradients {mode:6s}: {t:.2f} ms ({3 * 2 * M * V * D / t / 1e9:.0f} TF), "
              f"{peak:.1f} GiB above the inputs")
    C.check_status()


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("op", choices=["gemm", "attention", "elementwise", "grouped", "moe", "ce", "all"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--small", action="store_true", help="one cold launch per kernel on a small case")
    a = ap.parse_args()
    iters = 1 if a.small else a.iters
    table = {"gemm": bench_gemm, "attention": bench_attention, "elementwise": bench_elementwise, "grouped": bench_grouped,
             "moe": bench_moe, "ce": bench_ce}
    for name, fn in table.items():
        if a.op in (name, "all"):
            fn(iters, a.small)


if __name__ == "__main__":
    main()
