"""Symmetric (peer-mapped) device buffers for kernels that read and write other GPUs' memory.

A ``SymmBuffer`` is the same-sized allocation on every rank of a process group, mapped into every
peer's address space (CUDA VMM handles exchanged by ``torch.distributed._symmetric_memory``) and,
where the fabric supports it, bound to an NVLink multicast object whose address lets one instruction
reduce over (``multimem.ld_reduce``) or store to (``multimem.st``) all ranks through NVSwitch.
Kernels receive ``peer_ptrs`` (one device pointer per rank) and ``multicast_ptr`` (0 if unavailable).
``barrier()`` is a stream-ordered cross-rank barrier on a signal pad that lives at the end of the same
allocation.  It is this library's own kernel (``csrc/flag_wait.cu``): plain peer stores and acquire loads with a
deadline, after which the kernel records "timed out waiting on a peer" in the status word and returns, so a rank
that died or raised cannot leave the others spinning inside a kernel (``ops.cuda.check_status`` then raises on the
host).  PyTorch's own symmetric-memory barrier spins without a limit by default and traps when given one.

Rules for kernels using these buffers: plain loads/stores, ``red`` and ``multimem`` only; no TMA load
with cluster multicast may ever target a peer pointer.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist


PAD_CHANNELS = 8      # independent barrier channels per buffer (one per stream that synchronises on it)
PAD_MAX_RANKS = 64
PAD_INTS = PAD_CHANNELS * PAD_MAX_RANKS


def barrier_timeout_ms() -> float:
    """Deadline of one cross-rank barrier.  Long enough for ordinary skew between ranks (a checkpoint write, a
    garbage collection, a slow first step), short enough that a dead peer ends the job instead of hanging it."""
    return float(os.environ.get("MB_BARRIER_TIMEOUT_MS", "120000"))


class SymmBuffer:
    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        self.pad_offset = (nbytes + 255) // 256 * 256
        self.raw = symm_mem.empty(self.pad_offset + PAD_INTS * 4, dtype=torch.uint8, device=device)
        self.tensor = self.raw[:nbytes].view(dtype)
        self.pad = self.raw[self.pad_offset:].view(torch.int32)
        self.pad.zero_()
        torch.cuda.synchronize(device)
        self.handle = symm_mem.rendezvous(self.raw, group)
        self.world = self.handle.world_size
        self.rank = self.handle.rank
        if self.world > PAD_MAX_RANKS:
            raise ValueError(f"symmetric buffers support at most {PAD_MAX_RANKS} ranks per group")
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.multicast_ptr = int(self.handle.multicast_ptr) if self.handle.has_multicast_support else 0
        self._ptr_array = (ctypes.c_void_p * self.world)(*self.peer_ptrs)
        self._pad_array = (ctypes.c_void_p * self.world)(*[p + self.pad_offset for p in self.peer_ptrs])
        self._epoch = [0] * PAD_CHANNELS
        # nobody may signal into a pad that its owner has not cleared yet
        dist.barrier(group=group)

    @property
    def ptr_array(self):
        """``void* [world]`` host array for the native launchers."""
        return self._ptr_array

    def barrier(self, channel: int = 0, timeout_ms: float | None = None) -> None:
        """All ranks reach this point on their current streams before any continues.

        Every rank must call it the same number of times per channel; barriers issued on different streams need
        different channels.  A peer that does not arrive within the deadline makes the kernel give up (status
        "timed out waiting on a peer GPU's flag"); it never spins without a limit and never traps."""
        from maester_b200.ops import cuda as C

        self._epoch[channel] += 1
        C.symm_barrier(self._pad_array, self.world, self.rank, channel * PAD_MAX_RANKS, self._epoch[channel],
                       barrier_timeout_ms() if timeout_ms is None else timeout_ms)


_PREFLIGHT: dict = {}


def preflight(group, device: torch.device | None = None, nbytes: int = 1 << 20) -> dict:
    """Start-up check of the peer-memory plane of ``group`` (cached per group): rendezvous of a small symmetric
    buffer, one bounded cross-rank barrier, and a pull of every peer's pattern through its mapped pointer.

    Returns ``{"ok", "reason", "world", "multicast", "pull_gbs"}``; all ranks agree on ``ok`` (it is all-reduced), so
    either every rank uses the peer-memory kernels or every rank uses NCCL.  Nothing here can hang: the barrier
    gives up after a few seconds and reports through the status word."""
    key = id(group)
    if key in _PREFLIGHT:
        return _PREFLIGHT[key]
    out = {"ok": False, "reason": "", "world": 1, "multicast": False, "pull_gbs": 0.0}
    try:
        import importlib

        importlib.import_module("torch.distributed._symmetric_memory")
        if not (torch.cuda.is_available() and dist.is_initialized()):
            raise RuntimeError("needs CUDA and an initialised process group")
        if dist.get_backend(group) != "nccl":
            raise RuntimeError(f"backend is {dist.get_backend(group)}, not nccl")
        from maester_b200.ops import cuda as C

        device = device or torch.device("cuda", torch.cuda.current_device())
        world = dist.get_world_size(group)
        out["world"] = world
        local_ok, reason = 1, ""
        try:
            buf = SymmBuffer(nbytes // 4, torch.int32, device, group)
            out["multicast"] = bool(buf.multicast_ptr)
            buf.tensor.fill_(buf.rank + 1)
            buf.barrier(channel=PAD_CHANNELS - 1, timeout_ms=5000.0)
            got = torch.empty(nbytes // 4, dtype=torch.int32, device=device)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for r in range(world):
                if r == buf.rank:
                    continue
                e0.record()
                C.peer_copy(got, buf.peer_ptrs[r], nbytes)
                e1.record()
                torch.cuda.synchronize(device)
                if not bool((got == r + 1).all()):
                    local_ok, reason = 0, f"rank {buf.rank} read a wrong pattern from rank {r}"
                out["pull_gbs"] = max(out["pull_gbs"], nbytes / max(e0.elapsed_time(e1), 1e-3) / 1e6)
            buf.barrier(channel=PAD_CHANNELS - 1, timeout_ms=5000.0)   # nobody frees the buffer while a peer reads it
            C.check_status()
        except Exception as e:  # noqa: BLE001  (no peer access, unsupported driver, an expired barrier, ...)
            local_ok, reason = 0, f"{type(e).__name__}: {e}"
        flag = torch.tensor([local_ok], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        out["ok"] = bool(flag.item())
        out["reason"] = reason if not out["ok"] else ""
        if not out["ok"] and not reason:
            out["reason"] = "another rank of the group failed the check"
    except Exception as e:  # noqa: BLE001
        out["reason"] = f"{type(e).__name__}: {e}"
    _PREFLIGHT[key] = out
    from maester_b200.log_utils import logger

    if out["ok"]:
        logger.info(f"peer-memory preflight: {out['world']} ranks, multicast={out['multicast']}, "
                    f"pull {out['pull_gbs']:.0f} GB/s at {nbytes >> 10} KiB")
    elif out["world"] > 1 or "nccl" not in out["reason"]:
        logger.info(f"peer-memory preflight failed, NCCL collectives are used instead: {out['reason']}")
    return out


def symmetric_memory_available(group) -> bool:
    """True when the peer-memory plane of ``group`` passed its start-up check (see ``preflight``)."""
    if not (torch.cuda.is_available() and dist.is_initialized()):
        return False
    return preflight(group)["ok"]
