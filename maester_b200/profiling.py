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


class KernelTimers:
    """NVTX ranges and CUDA-event timers around every native launcher of ``maester_b200.ops.cuda``.

    ``with KernelTimers() as kt: trainer.train_step(batch)`` wraps the module's launcher functions for the duration
    of the block: each call is bracketed by an NVTX range named after the launcher and by two CUDA events on the
    launching stream.  ``kt.report()`` synchronises once and returns ``{launcher: (calls, device milliseconds)}``
    sorted by time; ``kt.report(group=...)`` additionally takes the maximum over the ranks of a process group, the way
    multi-GPU numbers are quoted.  The wrappers add two event records per call, so use it for attribution, not for
    headline numbers.  ``module`` and ``names`` exist for tests (any module with callables works, also without CUDA).
    """

    def __init__(self, module=None, names: list[str] | None = None):
        if module is None:
            from maester_b200.ops import cuda as module
        self.module = module
        self.names = names or [n for n, f in vars(module).items()
                               if callable(f) and not n.startswith("_") and getattr(f, "__module__", None) == module.__name__
                               and not isinstance(f, type) and n not in ("check_status",)]
        self._saved: dict = {}
        self._events: dict[str, list] = {}
        self.calls: dict[str, int] = {}
        self._cuda = torch.cuda.is_available()

    def _wrap(self, name: str, fn):
        def timed(*a, **kw):
            self.calls[name] = self.calls.get(name, 0) + 1
            if not self._cuda:
                return fn(*a, **kw)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.nvtx.range_push(f"mb::{name}")
            e0.record()
            try:
                return fn(*a, **kw)
            finally:
                e1.record()
                torch.cuda.nvtx.range_pop()
                self._events.setdefault(name, []).append((e0, e1))
        timed.__wrapped__ = fn
        return timed

    def __enter__(self):
        for n in self.names:
            self._saved[n] = getattr(self.module, n)
            setattr(self.module, n, self._wrap(n, self._saved[n]))
        return self

    def __exit__(self, *exc):
        for n, f in self._saved.items():
            setattr(self.module, n, f)
        self._saved.clear()
        return False

    def report(self, group=None) -> dict[str, tuple[int, float]]:
        if self._cuda:
            torch.cuda.synchronize()
        names = sorted(self.calls)
        ms = [sum(a.elapsed_time(b) for a, b in self._events.get(n, [])) for n in names]
        if group is not None and dist.is_initialized() and names:
            t = torch.tensor(ms, dtype=torch.float64, device="cuda" if self._cuda else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
            ms = t.tolist()
        out = {n: (self.calls[n], float(m)) for n, m in zip(names, ms)}
        return dict(sorted(out.items(), key=lambda kv: -kv[1][1]))


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
