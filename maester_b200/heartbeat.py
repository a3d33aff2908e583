"""Host-side liveness of the ranks of a job, through the rendezvous key-value store.

The reference detects failures only through process-group timeouts (300 s during start-up, 100 s in
steady state, train.py:539-543) and the scheduler-level babysitter.  Kernels of this framework that
talk to peers directly (symmetric-memory collectives) should never be launched towards a rank that
is gone, so the trainer can ask the store first: every rank posts the number of the step it is about
to run; ``check`` returns (or raises ``PeerLost``) without touching the GPU.  A rank that leaves on
purpose posts a tombstone, so its peers stop at the same step boundary instead of timing out.
"""
from __future__ import annotations

import time

import torch.distributed as dist


class PeerLost(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank} {reason}")
        self.rank, self.reason = rank, reason


class StepHeartbeat:
    def __init__(self, store=None, rank: int | None = None, world: int | None = None, prefix: str = "mb_heartbeat"):
        self.store = store if store is not None else dist.distributed_c10d._get_default_store()
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.prefix = prefix

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def beat(self, step: int) -> None:
        """Announce that this rank is about to run ``step``."""
        self.store.set(self._key(self.rank), f"{step}:{time.time():.3f}")

    def leave(self, step: int, reason: str = "left") -> None:
        """Announce a deliberate departure before ``step`` (call between steps, with nothing in flight)."""
        self.store.set(self._key(self.rank), f"gone@{step}:{reason}")

    def _read(self, rank: int):
        try:
            if not self.store.check([self._key(rank)]):
                return None
            return self.store.get(self._key(rank)).decode()
        except Exception:  # noqa: BLE001  (store gone: treat as silence)
            return None

    def check(self, step: int, timeout_s: float = 30.0, poll_s: float = 0.05) -> None:
        """Return once every rank has announced ``step`` (or a later one); raise ``PeerLost`` if a rank
        posted a tombstone or stays silent for ``timeout_s``."""
        deadline = time.monotonic() + timeout_s
        pending = set(range(self.world)) - {self.rank}
        while pending:
            for r in sorted(pending):
                v = self._read(r)
                if v is None:
                    continue
                if v.startswith("gone@"):
                    raise PeerLost(r, v.split(":", 1)[1] if ":" in v else "left")
                if int(v.split(":", 1)[0]) >= step:
                    pending.discard(r)
            if not pending:
                return
            if time.monotonic() > deadline:
                raise PeerLost(min(pending), f"did not reach step {step} within {timeout_s:.0f} s")
            time.sleep(poll_s)
