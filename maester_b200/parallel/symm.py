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


def symmetric_memory_available(group) -> bool:
    """True on CUDA with an initialised NCCL group (the rendezvous itself is the final check)."""
    if not (torch.cuda.is_available() and dist.is_initialized()):
        return False
    try:
        import importlib
        importlib.import_module("torch.distributed._symmetric_memory")
    except ImportError:
        return False
    return dist.get_backend(group) == "nccl"
