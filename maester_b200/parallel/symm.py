"""Symmetric (peer-mapped) device buffers for kernels that read and write other GPUs' memory.

A ``SymmBuffer`` is the same-sized allocation on every rank of a process group, mapped into every
peer's address space (CUDA VMM handles exchanged by ``torch.distributed._symmetric_memory``) and,
where the fabric supports it, bound to an NVLink multicast object whose address lets one instruction
reduce over (``multimem.ld_reduce``) or store to (``multimem.st``) all ranks through NVSwitch.
Kernels receive ``peer_ptrs`` (one device pointer per rank) and ``multicast_ptr`` (0 if unavailable).
``barrier()`` is a stream-ordered cross-rank barrier on the buffer's signal pad.

Rules for kernels using these buffers: plain loads/stores, ``red`` and ``multimem`` only; no TMA load
with cluster multicast may ever target a peer pointer.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist


class SymmBuffer:
    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, group)
        self.world = self.handle.world_size
        self.rank = self.handle.rank
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.multicast_ptr = int(self.handle.multicast_ptr) if self.handle.has_multicast_support else 0
        self._ptr_array = (ctypes.c_void_p * self.world)(*self.peer_ptrs)

    @property
    def ptr_array(self):
        """``void* [world]`` host array for the native launchers."""
        return self._ptr_array

    def barrier(self, channel: int = 0) -> None:
        """All ranks reach this point on their current streams before any continues."""
        self.handle.barrier(channel=channel)


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
