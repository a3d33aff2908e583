"""Collective health and bandwidth check, run before training when ``RUN_NCCL_PREFLIGHT=1``.

For every dtype in ``NCCL_PREFLIGHT_DTYPES`` (default fp32,fp16,bf16) and message size from 1 KiB
up to ``NCCL_PREFLIGHT_MAX_MB`` (default 256, powers of 4): a value-checked ``all_reduce(SUM)``, an
``all_gather_into_tensor`` (halving the size on out-of-memory) and, unless
``NCCL_PREFLIGHT_TRY_REDUCE_SCATTER=0``, a ``reduce_scatter_tensor``.  Each is timed over
``NCCL_PREFLIGHT_ITERS`` iterations after ``NCCL_PREFLIGHT_WARMUP`` warm-ups — on the device with CUDA
events when the backend is NCCL — and rank 0 writes ``nccl_preflight_report.json`` into
``NCCL_PREFLIGHT_REPORT_DIR`` with p50/p99 latency and bus bandwidth per rank.  A wrong value raises.
Reference tool: nccl_preflight.py:74-473.  Also runnable stand-alone under torchrun.
"""
from __future__ import annotations

import json
import os
import time

import torch
import torch.distributed as dist

DTYPES = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


def _env_int(name: str, default: int) -> int:
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def _device() -> torch.device:
    if dist.get_backend() == "nccl":
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def _time_op(fn, iters: int, warmup: int, dev: torch.device) -> list[float]:
    """Per-iteration milliseconds."""
    for _ in range(warmup):
        fn()
    out = []
    if dev.type == "cuda":
        torch.cuda.synchronize()
        for _ in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            out.append(e0.elapsed_time(e1))
    else:
        for _ in range(iters):
            t = time.perf_counter()
            fn()
            out.append((time.perf_counter() - t) * 1e3)
    return out


def _stats(ms: list[float], bus_bytes: float) -> dict:
    s = sorted(ms)
    p50 = s[len(s) // 2]
    p99 = s[min(len(s) - 1, int(len(s) * 0.99))]
    return {"p50_us": p50 * 1e3, "p99_us": p99 * 1e3, "busbw_GBps": bus_bytes / (p50 * 1e-3) / 1e9 if p50 > 0 else 0.0}


def _sizes(max_mb: int) -> list[int]:
    out, n = [], 1024
    while n <= max_mb * 2**20:
        out.append(n)
        n *= 4
    return out


def run_nccl_preflight() -> dict:
    assert dist.is_initialized(), "run_nccl_preflight needs an initialised process group"
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = _device()
    iters, warmup = _env_int("NCCL_PREFLIGHT_ITERS", 10), _env_int("NCCL_PREFLIGHT_WARMUP", 3)
    max_mb = _env_int("NCCL_PREFLIGHT_MAX_MB", 256)
    names = [d.strip() for d in os.environ.get("NCCL_PREFLIGHT_DTYPES", "fp32,fp16,bf16").split(",") if d.strip()]
    try_rs = os.environ.get("NCCL_PREFLIGHT_TRY_REDUCE_SCATTER", "1") not in {"0", "false", "no"}
    results = []
    for name in names:
        dtype = DTYPES[name]
        if dev.type == "cpu" and dtype == torch.float16:
            continue  # gloo reductions on fp16 are not supported everywhere
        esize = torch.empty((), dtype=dtype).element_size()
        for nbytes in _sizes(max_mb):
            n = max(world, nbytes // esize // world * world)
            rec = {"dtype": name, "bytes": n * esize}
            # ---- all_reduce with a value check: sum of (rank+1) over ranks
            x = torch.full((n,), float(rank + 1), dtype=dtype, device=dev)
            dist.all_reduce(x)
            want = world * (world + 1) / 2
            if not torch.allclose(x.float(), torch.full_like(x, want, dtype=torch.float32), rtol=1e-2):
                raise RuntimeError(f"all_reduce value check failed on rank {rank}: {x[0].item()} != {want} "
                                   f"({name}, {n * esize} bytes)")
            buf = torch.ones(n, dtype=dtype, device=dev)
            ms = _time_op(lambda: dist.all_reduce(buf), iters, warmup, dev)
            rec["all_reduce"] = _stats(ms, 2 * (world - 1) / world * n * esize)
            # ---- all_gather (shard -> full), back off on OOM
            shard = n // world
            while True:
                try:
                    src = torch.full((shard,), float(rank), dtype=dtype, device=dev)
                    dst = torch.empty(shard * world, dtype=dtype, device=dev)
                    break
                except torch.OutOfMemoryError:
                    shard //= 2
                    if shard == 0:
                        raise
            dist.all_gather_into_tensor(dst, src)
            got = dst.view(world, shard)[:, 0].float().cpu().tolist()
            if got != [float(r) for r in range(world)]:
                raise RuntimeError(f"all_gather value check failed on rank {rank}: {got}")
            ms = _time_op(lambda: dist.all_gather_into_tensor(dst, src), iters, warmup, dev)
            rec["all_gather"] = _stats(ms, (world - 1) * shard * esize)
            # ---- reduce_scatter
            if try_rs:
                try:
                    full = torch.ones(shard * world, dtype=dtype, device=dev)
                    out = torch.empty(shard, dtype=dtype, device=dev)
                    dist.reduce_scatter_tensor(out, full)
                    if abs(out[0].item() - world) > 1e-2 * world:
                        raise RuntimeError(f"reduce_scatter value check failed on rank {rank}: {out[0].item()}")
                    ms = _time_op(lambda: dist.reduce_scatter_tensor(out, full), iters, warmup, dev)
                    rec["reduce_scatter"] = _stats(ms, (world - 1) * shard * esize)
                except (RuntimeError, NotImplementedError) as e:
                    if "value check" in str(e):
                        raise
                    rec["reduce_scatter"] = {"unsupported": str(e)[:100]}
            results.append(rec)
    gathered: list = [None] * world
    dist.all_gather_object(gathered, {"rank": rank, "host": os.uname().nodename, "results": results})
    report = {"world_size": world, "backend": dist.get_backend(), "ranks": gathered}
    if rank == 0:
        out_dir = os.environ.get("NCCL_PREFLIGHT_REPORT_DIR", ".")
        os.makedirs(out_dir, exist_ok=True)
        path = os.path.join(out_dir, "nccl_preflight_report.json")
        with open(path, "w") as f:
            json.dump(report, f, indent=1)
        big = [r for r in results if "all_reduce" in r][-1]
        print(f"[preflight] ok: world={world}, largest all_reduce {big['bytes'] / 2**20:.0f} MiB "
              f"p50 {big['all_reduce']['p50_us']:.0f} us, {big['all_reduce']['busbw_GBps']:.1f} GB/s bus; report {path}")
    dist.barrier()
    return report


if __name__ == "__main__":
    backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group(backend)
    run_nccl_preflight()
    dist.destroy_process_group()
