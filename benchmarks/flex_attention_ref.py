"""Time the reference's attention call next to this library's kernels on the same GPU and inputs.

    python -m benchmarks.flex_attention_ref [--iters 10] [--batch 2] [--seq 8192]

The reference attends with ``torch.compile(flex_attention)`` under a ``BlockMask`` built from its own
mask functions (maester/models/gemma/model.py:203-256 mask functions, :388-396 the call, :694-739 the
two masks per forward).  This script imports those mask functions from the installed reference
(``baseline/_ref``), builds the same masks for the Gemma-3 4B attention shape (8 query / 4 KV heads of
256, window 1024) on packed documents, and times forward and forward+backward with CUDA events after
warm-up, beside ``attn_fwd`` / ``attn_bwd`` of this library on identical tensors.  The outputs are
compared as a sanity check.  One JSON line per case.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def timeit(fn, iters: int, warm: int = 3) -> float:
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


def packed_docs(B: int, S: int, mean: float, seed: int = 0) -> torch.Tensor:
    rng = np.random.default_rng(seed)
    docs = np.zeros((B, S), dtype=np.int32)
    for b in range(B):
        i = d = 0
        while i < S:
            j = min(S, i + max(1, int(rng.geometric(1.0 / mean))))
            docs[b, i:j] = d
            i, d = j, d + 1
    return torch.from_numpy(docs)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--no-reference", action="store_true", help="time only this library's kernels")
    a = ap.parse_args()
    B, S, H, KV, hd, W = a.batch, a.seq, 8, 4, 256, 1024
    dev = torch.device("cuda")
    torch.manual_seed(0)

    from maester_b200.ops import cuda as C
    from maester_b200.ops.functional import attention_plan

    have_ref = False
    if not a.no_reference:
        sys.path.insert(0, os.path.join(ROOT, "baseline", "shims"))
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        try:
            from maester.models.gemma.model import (causal_mask, make_document_mask_wrapper,
                                                    make_sliding_window_mask_fn)
            from torch.nn.attention.flex_attention import create_block_mask, flex_attention
            flex = torch.compile(flex_attention, fullgraph=True)
            have_ref = True
        except Exception as e:  # noqa: BLE001
            print(json.dumps({"reference": "unavailable", "why": repr(e)[:200]}))

    qkv = torch.randn(B, S, (H + 2 * KV) * hd, device=dev, dtype=torch.bfloat16)
    q = qkv[..., :H * hd].view(B, S, H, hd)
    k = qkv[..., H * hd:(H + KV) * hd].view(B, S, KV, hd)
    v = qkv[..., (H + KV) * hd:].view(B, S, KV, hd)
    scale = hd ** -0.5

    cases = [("causal", None, None), ("window1024", W, None), ("causal+docs1500", None, 1500.0),
             ("window1024+docs1500", W, 1500.0)]
    for name, window, doc_mean in cases:
        doc = packed_docs(B, S, doc_mean).to(dev) if doc_mean else None
        plan = attention_plan(S, window, doc, dev, batch=B)
        out, lse = C.attn_fwd(q, k, v, scale, True, window, plan)
        dout = torch.randn_like(out)
        dqkv = torch.empty(B * S, (H + 2 * KV) * hd, device=dev, dtype=torch.bfloat16)
        t_f = timeit(lambda: C.attn_fwd(q, k, v, scale, True, window, plan), a.iters)
        t_b = timeit(lambda: C.attn_bwd(q, k, v, out, dout, lse, dqkv, scale, True, window, plan), a.iters)
        C.check_status()
        rec = {"case": name, "B": B, "S": S, "H": H, "KV": KV, "hd": hd, "ours_fwd_ms": round(t_f, 4),
               "ours_bwd_ms": round(t_b, 4)}
        if have_ref:
            base = causal_mask if window is None else make_sliding_window_mask_fn(window)
            fn = make_document_mask_wrapper(base, doc) if doc is not None else base
            bm = create_block_mask(fn, B, None, S, S, device=dev)
            qt = q.transpose(1, 2).detach().clone().requires_grad_(True)
            kt = k.transpose(1, 2).detach().clone().requires_grad_(True)
            vt = v.transpose(1, 2).detach().clone().requires_grad_(True)
            dot = dout.transpose(1, 2)

            def ref_fwd():
                return flex(qt, kt, vt, block_mask=bm, scale=scale, enable_gqa=True)

            def ref_fwd_bwd():
                o = ref_fwd()
                torch.autograd.grad(o, (qt, kt, vt), dot)

            with torch.no_grad():
                o_ref = ref_fwd()
                t_rf = timeit(ref_fwd, a.iters)
            t_rfb = timeit(ref_fwd_bwd, a.iters)
            err = (o_ref.transpose(1, 2).float() - out.float()).abs().max().item()
            rec.update({"flex_fwd_ms": round(t_rf, 4), "flex_fwd_bwd_ms": round(t_rfb, 4),
                        "flex_bwd_ms": round(t_rfb - t_rf, 4), "max_abs_diff_out": round(err, 5),
                        "speedup_fwd": round(t_rf / t_f, 2), "speedup_bwd": round((t_rfb - t_rf) / t_b, 2)})
        print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
