"""Failure detection without faulting a GPU: failures are made on the host (a rank that raises, never
joins or leaves), kernels' waits are bounded, and corrupted inputs are reported as exceptions."""
import os
import tempfile
import time
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from test_parallel_cpu import _free_port


def _spawn(world, fn, *args, timeout_s=120):
    with tempfile.TemporaryDirectory() as d:
        ctx = mp.spawn(_entry, args=(world, _free_port(), fn, args, d), nprocs=world, join=False)
        t0 = time.time()
        while not ctx.join(timeout=1.0):
            assert time.time() - t0 < timeout_s, "ranks did not finish: a failure was not detected"
        return [torch.load(os.path.join(d, f"r{r}.pt"), weights_only=False) for r in range(world)
                if os.path.exists(os.path.join(d, f"r{r}.pt"))]


def _entry(rank, world, port, fn, args, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    res = fn(rank, world, *args)
    torch.save(res, os.path.join(out_dir, f"r{rank}.pt"))


# ----------------------------------------------------------------------------- collective timeouts
def _rank_raises(rank, world):
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=4))
    x = torch.ones(4)
    dist.all_reduce(x)  # step 1 works
    try:
        if rank == 1:
            raise ValueError("rank 1 fails between steps")  # host-side failure, no collective in flight
        t0 = time.time()
        dist.all_reduce(x)  # the survivor's next collective must end with an error, not hang
        return ("no error", time.time() - t0)
    except ValueError as e:
        return ("raised", str(e))
    except RuntimeError as e:
        return ("collective error", time.time() - t0)


def test_survivor_gets_an_error_after_a_peer_failed():
    res = dict(enumerate(_spawn(2, _rank_raises)))
    assert res[1][0] == "raised"
    kind, waited = res[0]
    assert kind == "collective error" and waited < 30


def _never_joins(rank, world):
    if rank == 1:
        return "absent"  # never calls init_process_group
    t0 = time.time()
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=3))
        return "joined"
    except Exception as e:  # noqa: BLE001
        return ("rendezvous error", time.time() - t0, type(e).__name__)


def test_missing_rank_fails_the_rendezvous_within_the_timeout():
    res = _spawn(2, _never_joins)
    r0 = next(r for r in res if r != "absent")
    assert r0[0] == "rendezvous error" and r0[1] < 30


def _pg_timeout_tightening(rank, world):
    from maester_b200.utils import set_pg_timeouts
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=60))
    set_pg_timeouts(timedelta(seconds=3))  # what the trainer does after the first step
    x = torch.ones(1)
    dist.all_reduce(x)
    if rank == 1:
        time.sleep(8)
        return "slept"
    t0 = time.time()
    try:
        dist.all_reduce(x)
        return ("no error", time.time() - t0)
    except RuntimeError:
        return ("timeout", time.time() - t0)


def test_tightened_timeout_bounds_the_wait_for_a_straggler():
    res = _spawn(2, _pg_timeout_tightening)
    r0 = next(r for r in res if r != "slept")
    assert r0[0] == "timeout" and r0[1] < 7.5


# ----------------------------------------------------------------------------- heartbeat through the store
def _heartbeat(rank, world):
    from maester_b200.heartbeat import PeerLost, StepHeartbeat
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=30))
    hb = StepHeartbeat()
    log = []
    for step in range(1, 5):
        if rank == 2 and step == 3:
            hb.leave(step, "preempted")  # leaves between steps, nothing in flight
            return log + ["left"]
        hb.beat(step)
        try:
            hb.check(step, timeout_s=10)
        except PeerLost as e:
            return log + [f"lost rank {e.rank}: {e.reason}"]
        x = torch.ones(1)
        dist.all_reduce(x)  # the step's collectives only run once everybody is known to be there
        log.append(int(x.item()))
    return log


def test_ranks_learn_of_a_departure_before_their_next_launch():
    res = _spawn(3, _heartbeat)
    assert res[2] == [3, 3, "left"]
    for r in (0, 1):
        assert res[r] == [3, 3, "lost rank 2: preempted"]


def _silent_peer(rank, world):
    from maester_b200.heartbeat import PeerLost, StepHeartbeat
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=30))
    hb = StepHeartbeat()
    if rank == 1:
        time.sleep(4)
        return "silent"
    hb.beat(1)
    t0 = time.time()
    try:
        hb.check(1, timeout_s=1.5)
        return "ok"
    except PeerLost as e:
        return (e.rank, time.time() - t0)


def test_silent_peer_is_reported_after_the_deadline():
    res = _spawn(2, _silent_peer)
    r0 = next(r for r in res if r != "silent")
    assert r0[0] == 1 and 1.4 < r0[1] < 4


# ----------------------------------------------------------------------------- data path
def test_broken_parquet_shard_raises(tmp_path):
    import pyarrow as pa
    import pyarrow.parquet as pq
    from maester_b200.datasets.parquet_dataset import ParquetDataset

    class Tok:
        def encode(self, text, **kw):
            return [ord(c) % 50 + 3 for c in text]

    good = tmp_path / "a.parquet"
    pq.write_table(pa.table({"text": ["hello world"] * 20}), good)
    bad = tmp_path / "b.parquet"
    bad.write_bytes(good.read_bytes()[:100])  # truncated file
    with pytest.raises(Exception):
        ds = ParquetDataset(str(tmp_path), 0, 1, Tok(), delimiter_token=0)
        it = iter(ds)
        for _ in range(200):
            next(it)


# ----------------------------------------------------------------------------- device-side bounded wait
@pytest.mark.gpu
def test_bounded_wait_expires_sets_status_and_leaves_the_context_usable():
    from maester_b200.ops import cuda as C
    C.check_status()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    seen = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    t0 = time.time()
    C.wait_flag(flag, 1, timeout_ms=200.0, observed=seen)  # nothing ever sets the flag
    with pytest.raises(RuntimeError, match="status 5"):
        C.check_status()
    assert time.time() - t0 < 5 and seen.item() == 0
    C.check_status()  # the status word was cleared by the failed check
    flag.fill_(3)
    C.wait_flag(flag, 2, timeout_ms=200.0, observed=seen)
    C.check_status()
    assert seen.item() == 1
    a = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(64, 128, device="cuda", dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    assert (C.gemm(a, b).float() - ref).abs().max().item() < 0.5  # kernels still run after the expiry
    C.check_status()


@pytest.mark.gpu
def test_cross_rank_barrier_gives_up_when_a_peer_never_arrives():
    """The library's own barrier kernel on a local table of signal pads: with the peer's arrival already posted it
    passes; with a peer that never posts it returns at the deadline with the status word set, and later kernels run."""
    import ctypes

    from maester_b200.ops import cuda as C
    C.check_status()
    pads = torch.zeros(2, 64, dtype=torch.int32, device="cuda")  # pads[r]: signal pad of rank r
    table = (ctypes.c_void_p * 2)(pads[0].data_ptr(), pads[1].data_ptr())
    pads[0, 1] = 1                                   # "rank 1" has already posted epoch 1 into rank 0's pad
    C.symm_barrier(table, 2, 0, 0, 1, timeout_ms=300.0)
    C.check_status()
    assert pads[:, 0].tolist() == [1, 1]             # rank 0's arrival reached both pads
    t0 = time.time()
    C.symm_barrier(table, 2, 0, 0, 2, timeout_ms=300.0)   # nobody posts epoch 2 for rank 1
    with pytest.raises(RuntimeError, match="status 5"):
        C.check_status()
    assert time.time() - t0 < 5
    x = torch.randn(128, 64, device="cuda", dtype=torch.bfloat16)
    assert torch.isfinite(C.gemm(x, x).float()).all()
    C.check_status()


def test_a_failed_kernel_status_blocks_the_checkpoint(tmp_path, monkeypatch):
    """If a kernel gave up on a bounded wait, its output is garbage: ``save`` must raise before writing anything."""
    import maester_b200.checkpoint as ckpt
    from test_checkpoint_cpu import _mk, _trainer_with_ckpt
    tr, state, ck = _trainer_with_ckpt(_mk(tmp_path))

    def bad():
        raise RuntimeError("maester_b200 kernel reported status 5: timed out waiting on a peer GPU's flag")

    monkeypatch.setattr(ckpt, "_check_device_status", bad)
    with pytest.raises(RuntimeError, match="status 5"):
        ck.save(2)
    assert not (tmp_path / "job" / "checkpoints" / "step-2").exists()
    monkeypatch.undo()
    ck.save(2)
    assert (tmp_path / "job" / "checkpoints" / "step-2" / ".metadata").exists()


@pytest.mark.gpu
def test_an_expired_wait_blocks_the_checkpoint_on_the_gpu(tmp_path):
    from maester_b200.ops import cuda as C
    from test_checkpoint_cpu import _mk, _trainer_with_ckpt
    C.check_status()
    tr, state, ck = _trainer_with_ckpt(_mk(tmp_path))
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    C.wait_flag(flag, 1, timeout_ms=100.0)  # nothing sets the flag: the wait runs out
    with pytest.raises(RuntimeError, match="status 5"):
        ck.save(2)
    assert not (tmp_path / "job" / "checkpoints" / "step-2").exists()
    ck.save(2)  # the failed check cleared the status word
    assert (tmp_path / "job" / "checkpoints" / "step-2" / ".metadata").exists()


def _preflight_rank(rank, world):
    import torch.distributed as dist
    from maester_b200.parallel.symm import preflight, symmetric_memory_available
    res = preflight(dist.group.WORLD)
    return res["ok"], res["reason"], symmetric_memory_available(dist.group.WORLD)


def test_peer_memory_preflight_declines_without_a_gpu_plane():
    """On a gloo group the start-up check of the peer-memory plane answers "no" with a reason on every rank (and the
    framework then uses the process group's collectives); it neither raises nor waits."""
    from test_parallel_cpu import run_ranks
    for ok, reason, avail in run_ranks(2, _preflight_rank):
        assert ok is False and avail is False
        assert reason
