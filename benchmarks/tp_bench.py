"""Micro-benchmark of the tensor-parallel linears: collective fused into the GEMM kernel vs NCCL + GEMM.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29560 \
        -m benchmarks.tp_bench [--tokens 16384] [--dim 4096] [--iters 20] [--copiers 1,2,4,8]

Shapes default to Llama-3 8B with TP = world size (sequence-sharded activations ``[tokens / tp, dim]``): the
column-parallel ``wq|wk|wv`` and ``w1|w3`` (all-gather -> GEMM) and the row-parallel ``wo`` and ``w2``
(GEMM -> reduce-scatter).  Every number is the maximum over ranks of the CUDA-event time per call, after
warm-up; inputs rotate over buffers larger than L2.  Rank 0 prints one JSON line per case.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _time(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--dim", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--qkv", type=int, default=6144)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--copiers", default="1,2,4,8")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from maester_b200.ops import cuda as C
    from maester_b200.parallel.fused_tp import FusedTP, _all_gather_rows
    from maester_b200.parallel.tensor_parallel import TPInfo

    tp = TPInfo(dist.group.WORLD, world, rank)
    M, K = a.tokens, a.dim
    Ml = M // world
    g = torch.Generator(device="cuda").manual_seed(1 + rank)
    xs = [torch.randn(Ml, K, device="cuda", generator=g).to(torch.bfloat16) for _ in range(4)]
    out = []
    for name, n_full in (("wqkv", a.qkv), ("w13", 2 * a.ffn)):
        N = n_full // world
        w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
        i = [0]

        def nccl():
            i[0] += 1
            return C.gemm(_all_gather_rows(xs[i[0] % 4], tp), w)

        t_nccl = _time(nccl, a.iters)
        t_gemm = _time(lambda: C.gemm(torch.empty(M, K, device="cuda", dtype=torch.bfloat16), w), a.iters)
        rec = {"case": f"all-gather -> {name}", "M": M, "N": N, "K": K, "tp": world, "nccl_ag_plus_gemm_ms": round(t_nccl, 4),
               "gemm_alone_ms": round(t_gemm, 4), "fused_ms": {}}
        for c in [int(v) for v in a.copiers.split(",")]:
            f = FusedTP(tp)
            f.ag_mode, f.ag_copiers = "fused", c

            def fused():
                i[0] += 1
                return f.ag_gemm(xs[i[0] % 4], w, b_mn=False)[1]

            rec["fused_ms"][str(c)] = round(_time(fused, a.iters), 4)
            want = C.gemm(_all_gather_rows(xs[0], tp), w)
            got = f.ag_gemm(xs[0], w, b_mn=False)[1]
            rec.setdefault("max_abs_diff", 0.0)
            rec["max_abs_diff"] = max(rec["max_abs_diff"], float((want.float() - got.float()).abs().max().item()))
            C.check_status()
            del f
        out.append(rec)
    for name, k_full in (("wo", a.dim), ("w2", a.ffn)):
        Kl = k_full // world
        x = torch.randn(M, Kl, device="cuda", generator=g).to(torch.bfloat16)
        w = (torch.randn(K, Kl, device="cuda", generator=g) * 0.02).to(torch.bfloat16)

        def nccl_rs():
            y = C.gemm(x, w)
            o = torch.empty(Ml, K, device="cuda", dtype=torch.bfloat16)
            dist.reduce_scatter_tensor(o, y, group=tp.group)
            return o

        rec = {"case": f"{name} -> reduce-scatter", "M": M, "N": K, "K": Kl, "tp": world,
               "gemm_plus_nccl_rs_ms": round(_time(nccl_rs, a.iters), 4)}
        for mode in ("pull", "push"):
            f = FusedTP(tp, mode)
            rec[f"fused_{mode}_ms"] = round(_time(lambda: f.gemm_rs(x, w, b_mn=False), a.iters), 4)
            C.check_status()
            del f
        out.append(rec)
    if rank == 0:
        for rec in out:
            print(json.dumps(rec), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
