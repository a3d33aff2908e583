"""Profiler and memory-snapshot context managers (reference: maester/profiling.py:25-133).

``maybe_enable_profiling`` yields a ``torch.profiler`` stepping object: schedule wait =
``profile_freq - 4``, warm-up 3, active 1, repeated 3 times; chrome traces go to
``<dump_dir>/<job>/<traces_folder>/iteration_<N>/rank<r>_trace.json`` and all ranks meet at a
barrier after an export.  ``maybe_enable_memory_snapshot`` records CUDA allocator history and
pickles a snapshot every ``profile_freq`` steps and when an out-of-memory error escapes.
Native kernels appear in the traces under their own names; NVTX ranges can be added around steps
with ``nvtx_range``.
"""
from __future__ import annotations

import contextlib
import os
import pickle
import time

import torch
import torch.distributed as dist

from maester_b200.log_utils import logger

WARMUP = 3
MEMORY_SNAPSHOT_MAX_ENTRIES = 100_000


@contextlib.contextmanager
def nvtx_range(name: str):
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


@contextlib.contextmanager
def maybe_enable_profiling(cfg, *, global_step: int = 0):
    if not cfg.enable_profiling:
        yield None
        return
    trace_dir = os.path.join(cfg.dump_dir, cfg.job_name, cfg.traces_folder)
    rank = dist.get_rank() if dist.is_initialized() else 0
    freq = cfg.profile_freq

    def on_trace(prof):
        cur = os.path.join(trace_dir, f"iteration_{prof.step_num}")
        os.makedirs(cur, exist_ok=True)
        begin = time.monotonic()
        prof.export_chrome_trace(f"{cur}/rank{rank}_trace.json")
        logger.info(f"Finished dumping traces in {time.monotonic() - begin:.2f} seconds")
        if dist.is_initialized():
            dist.barrier()  # keep ranks aligned: a slow dump must not trip the collective timeout

    logger.info(f"Profiling active. Traces will be saved at {trace_dir}")
    os.makedirs(trace_dir, exist_ok=True)
    wait = max(freq - (1 + WARMUP), 0)
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    with torch.profiler.profile(
        activities=acts,
        schedule=torch.profiler.schedule(wait=wait, warmup=WARMUP, active=1, repeat=3),
        on_trace_ready=on_trace,
        record_shapes=True,
    ) as prof:
        prof.step_num = global_step
        yield prof


@contextlib.contextmanager
def maybe_enable_memory_snapshot(cfg, *, global_step: int = 0):
    if not cfg.enable_memory_snapshot or not torch.cuda.is_available():
        yield None
        return
    snap_dir = os.path.join(cfg.dump_dir, cfg.job_name, cfg.memory_snapshot_folder)
    os.makedirs(snap_dir, exist_ok=True)
    rank = dist.get_rank() if dist.is_initialized() else 0

    class MemoryProfiler:
        def __init__(self, step_num: int, freq: int):
            torch.cuda.memory._record_memory_history(max_entries=MEMORY_SNAPSHOT_MAX_ENTRIES)
            self.step_num, self.freq = step_num, freq

        def step(self, exit_ctx: bool = False) -> None:
            self.step_num += 1
            if not exit_ctx and self.step_num % self.freq != 0:
                return
            name = f"iteration_{self.step_num}" + ("_exit" if exit_ctx else "")
            cur = os.path.join(snap_dir, name)
            os.makedirs(cur, exist_ok=True)
            logger.info(f"Dumping memory snapshot at step {self.step_num}")
            begin = time.monotonic()
            with open(f"{cur}/rank{rank}_memory_snapshot.pickle", "wb") as f:
                pickle.dump(torch.cuda.memory._snapshot(), f)
            logger.info(f"Finished dumping memory snapshot in {time.monotonic() - begin:.2f} seconds")
            if dist.is_initialized():
                dist.barrier()

    logger.info(f"Memory profiler active. Snapshot will be saved at {snap_dir}")
    profiler = MemoryProfiler(global_step, cfg.profile_freq)
    try:
        yield profiler
    except torch.OutOfMemoryError:
        profiler.step(exit_ctx=True)
        raise
