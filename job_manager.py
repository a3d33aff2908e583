"""Keeps one training job alive on SLURM by maintaining a queue of resubmissions.

    python job_manager.py jobs/<job_name> [--submit-interval 3600] [--once]

Recovery model (as in the reference, job_manager.py:36-419): a job dies or times out, a queued copy
starts, ``train.py`` resumes from the newest checkpoint and the data loader from its saved state.
The manager (1) keeps enough copies of ``slurm.sh`` pending to cover ``horizon`` seconds at one
submission per ``submit_interval``, (2) treats a running job as healthy while its log file
``logs/<job_id>.out`` was written within the last ``stale_after`` seconds, (3) cancels every running
copy except the longest-running healthy one, and pending copies that are about to start while a
healthy one runs, (4) records every job in ``job_manager.db`` (sqlite) with its final ``sacct``
state.  All scheduler access goes through ``SlurmCLI`` so tests can substitute a fake.
"""
from __future__ import annotations

import argparse
import logging
import sqlite3
import subprocess
import sys
import time
from dataclasses import dataclass
from datetime import datetime, timedelta
from pathlib import Path

logger = logging.getLogger("job_manager")


@dataclass
class QueueEntry:
    job_id: str
    name: str
    state: str        # "R", "PD", ...
    start_time: str   # ISO time or "N/A"
    time_used: str    # [days-]hh:mm:ss or mm:ss


class SlurmCLI:
    """The four scheduler calls the manager needs."""

    def queue(self) -> dict[str, QueueEntry]:
        try:
            r = subprocess.run(["squeue", "-o", "%i %j %t %S %M", "--noheader"], capture_output=True, text=True,
                               check=True)
        except (subprocess.CalledProcessError, FileNotFoundError):
            logger.error("squeue failed")
            return {}
        out = {}
        for line in r.stdout.splitlines():
            f = line.split()
            if len(f) >= 5:
                out[f[0]] = QueueEntry(f[0], f[1], f[2], f[3], f[4])
        return out

    def submit(self, script: Path, job_name: str) -> str | None:
        try:
            r = subprocess.run(["sbatch", f"--job-name={job_name}", str(script)], capture_output=True, text=True,
                               check=True)
        except (subprocess.CalledProcessError, FileNotFoundError) as e:
            logger.error(f"sbatch failed: {getattr(e, 'stderr', e)}")
            return None
        return r.stdout.strip().split()[-1]

    def cancel(self, job_id: str) -> bool:
        try:
            subprocess.run(["scancel", job_id], check=True)
            return True
        except (subprocess.CalledProcessError, FileNotFoundError):
            return False

    def final_state(self, job_id: str) -> tuple[str, str] | None:
        try:
            r = subprocess.run(["sacct", "-j", job_id, "-o", "State,ExitCode", "--noheader"], capture_output=True,
                               text=True)
        except FileNotFoundError:
            return None
        f = r.stdout.split()
        return (f[0], f[1]) if r.returncode == 0 and len(f) >= 2 else None


def parse_slurm_time(s: str) -> timedelta:
    days = 0
    if "-" in s:
        d, s = s.split("-", 1)
        days = int(d)
    parts = [int(p) for p in s.split(":")]
    if len(parts) == 3:
        return timedelta(days=days, hours=parts[0], minutes=parts[1], seconds=parts[2])
    if len(parts) == 2:
        return timedelta(days=days, minutes=parts[0], seconds=parts[1])
    raise ValueError(f"Invalid time string: {s}")


class JobManager:
    def __init__(self, job_dir: str | Path, scheduler: SlurmCLI | None = None, submit_interval: int = 3600,
                 horizon: int = 172800, stale_after: int = 600, cancel_threshold: int = 600, clock=time.time):
        self.job_dir = Path(job_dir)
        self.sched = scheduler or SlurmCLI()
        self.submit_interval, self.horizon = submit_interval, horizon
        self.stale_after, self.cancel_threshold = stale_after, cancel_threshold
        self.clock = clock
        self.db_path = self.job_dir / "job_manager.db"
        self._init_db()
        self.sync_existing_state()

    # ------------------------------------------------------------------ persistence
    def _db(self):
        return sqlite3.connect(self.db_path)

    def _init_db(self) -> None:
        with self._db() as c:
            c.execute("""CREATE TABLE IF NOT EXISTS jobs (job_id TEXT PRIMARY KEY, submit_time TEXT, start_time TEXT,
                         end_time TEXT, status TEXT, exit_code TEXT, processed BOOLEAN DEFAULT FALSE)""")

    def _upsert(self, job_id: str, **fields) -> None:
        with self._db() as c:
            if c.execute("SELECT 1 FROM jobs WHERE job_id=?", (job_id,)).fetchone() is None:
                c.execute("INSERT INTO jobs (job_id, submit_time, status) VALUES (?, datetime('now'), 'QUEUED')",
                          (job_id,))
            for k, v in fields.items():
                c.execute(f"UPDATE jobs SET {k}=? WHERE job_id=?", (v, job_id))

    def open_jobs(self) -> list[str]:
        with self._db() as c:
            return [r[0] for r in c.execute("SELECT job_id FROM jobs WHERE end_time IS NULL")]

    # ------------------------------------------------------------------ health and policy
    def is_job_healthy(self, job_id: str) -> bool:
        log = self.job_dir / "logs" / f"{job_id}.out"
        return log.exists() and (self.clock() - log.stat().st_mtime) <= self.stale_after

    def healthy_runners(self, queue: dict[str, QueueEntry]) -> list[tuple[str, timedelta]]:
        out = []
        for jid in self.open_jobs():
            q = queue.get(jid)
            if q is not None and q.state == "R" and self.is_job_healthy(jid):
                out.append((jid, parse_slurm_time(q.time_used)))
        return out

    def should_cancel(self, job_id: str, queue: dict[str, QueueEntry]) -> bool:
        q = queue.get(job_id)
        if q is None:
            return False
        runners = self.healthy_runners(queue)
        if not runners:
            return False
        if q.state == "R":
            oldest = max(runners, key=lambda x: x[1])[0]
            return len(runners) > 1 and job_id in dict(runners) and job_id != oldest
        if q.state == "PD" and q.start_time != "N/A":
            try:
                start = datetime.strptime(q.start_time, "%Y-%m-%dT%H:%M:%S")
            except ValueError:
                return False
            return (start - datetime.fromtimestamp(self.clock())).total_seconds() < self.cancel_threshold
        return False

    # ------------------------------------------------------------------ actions
    def sync_existing_state(self) -> None:
        """Adopt jobs that already exist: queued jobs with our name and jobs that left log files."""
        queue = self.sched.queue()
        name = self.job_dir.name
        for jid, q in queue.items():
            if q.name == name:
                self._upsert(jid, status="RUNNING" if q.state == "R" else "QUEUED")
        for log in (self.job_dir / "logs").glob("*.out") if (self.job_dir / "logs").exists() else []:
            jid = log.stem
            if not jid.isdigit() or jid in queue:
                continue
            fin = self.sched.final_state(jid)
            if fin is not None:
                self._upsert(jid, status=fin[0], exit_code=fin[1], end_time=datetime.now().isoformat(), processed=True)

    def submit_job(self) -> str | None:
        jid = self.sched.submit(self.job_dir / "slurm.sh", self.job_dir.name)
        if jid:
            self._upsert(jid)
            logger.info(f"Submitted job {jid}")
        return jid

    def cancel_job(self, job_id: str) -> None:
        if self.sched.cancel(job_id):
            self._upsert(job_id, status="CANCELLED", end_time=datetime.now().isoformat())
            logger.info(f"Cancelled job {job_id}")

    def update_job_states(self, queue: dict[str, QueueEntry]) -> None:
        for jid in self.open_jobs():
            q = queue.get(jid)
            if q is not None:
                if q.state == "R":
                    self._upsert(jid, status="RUNNING", start_time=datetime.now().isoformat())
                continue
            fin = self.sched.final_state(jid)
            if fin is not None:
                self._upsert(jid, status=fin[0], exit_code=fin[1], end_time=datetime.now().isoformat())

    def target_pending(self) -> int:
        return max(1, self.horizon // max(1, self.submit_interval))

    def tick(self) -> dict[str, int]:
        """One management round; returns counters (for logs and tests)."""
        queue = self.sched.queue()
        self.update_job_states(queue)
        cancelled = 0
        for jid in list(self.open_jobs()):
            if self.should_cancel(jid, queue):
                self.cancel_job(jid)
                cancelled += 1
        queue = self.sched.queue()
        ours = [jid for jid in self.open_jobs() if jid in queue]
        pending = [j for j in ours if queue[j].state == "PD"]
        submitted = 0
        while len(pending) + submitted < self.target_pending():
            if self.submit_job() is None:
                break
            submitted += 1
        return {"running": sum(queue[j].state == "R" for j in ours), "pending": len(pending) + submitted,
                "cancelled": cancelled, "submitted": submitted}

    def run(self, poll: int = 30) -> None:
        while True:
            stats = self.tick()
            logger.info(f"running={stats['running']} pending={stats['pending']} cancelled={stats['cancelled']} "
                        f"submitted={stats['submitted']}")
            time.sleep(poll)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("job_dir")
    ap.add_argument("--submit-interval", type=int, default=3600)
    ap.add_argument("--once", action="store_true", help="run a single management round and exit")
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO, format="[%(asctime)s %(levelname)s] %(message)s")
    if not (Path(a.job_dir) / "slurm.sh").exists():
        print(f"{a.job_dir}/slurm.sh not found: create the job with submit.py first")
        return 1
    mgr = JobManager(a.job_dir, submit_interval=a.submit_interval)
    if a.once:
        print(mgr.tick())
        return 0
    mgr.run()
    return 0


if __name__ == "__main__":
    sys.exit(main())
