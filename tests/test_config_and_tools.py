"""Config round trip, LR schedules, job-directory tooling, sweeps and the job manager (CPU only)."""
import json
import math
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from maester_b200.config import Config, DatasetConfig, SFTConfig  # noqa: E402
from maester_b200.lr_scheduling import get_lr_scheduler, linear_warmup_constant_sqrt_decay, linear_warmup_cosine  # noqa: E402


def test_config_defaults_and_json_round_trip():
    cfg = Config()
    assert cfg.model_name == "gemma3" and cfg.flavor == "1B" and cfg.seq_len == 8192
    assert cfg.mixed_precision_param == "bfloat16" and cfg.mixed_precision_reduce == "float32"
    assert cfg.optimizer_groups[0]["exclude_names"] == ["tok_embeddings", "output"]
    again = Config(**json.loads(cfg.model_dump_json()))
    assert again.model_dump(mode="json") == cfg.model_dump(mode="json")  # tuples become lists in JSON
    with pytest.raises(Exception):
        cfg.seq_len = 4  # frozen


def test_config_nested_and_sft():
    cfg = Config(dataset=DatasetConfig(eos_token=1, bos_token=2), sft=SFTConfig(use_packed=False))
    d = json.loads(cfg.model_dump_json())
    assert d["dataset"]["eos_token"] == 1 and d["sft"]["use_packed"] is False
    assert Config(**d).sft.template == "chatml"


def test_reference_config_json_loads_unchanged():
    # a job directory written by the reference has none of this framework's extra fields
    ref_fields = {"model_name": "llama3", "flavor": "8B", "tensor_parallel_degree": 2,
                  "data_parallel_shard_degree": 4, "ac_mode": "selective", "selective_ac_option": "op"}
    cfg = Config(**ref_fields)
    assert cfg.context_parallel_degree == 1 and not cfg.synthetic_data


def test_lr_schedules():
    f = linear_warmup_cosine(10, 100)
    assert f(0) == pytest.approx(0.1) and f(9) == pytest.approx(1.0)
    # phase is step/total (warm-up not subtracted) and the floor is 0.1
    assert f(50) == pytest.approx(0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * 0.5)))
    assert f(100) == pytest.approx(0.1)
    g = linear_warmup_constant_sqrt_decay(10, 100, 20)
    assert g(50) == 1.0 and g(80) == 1.0 and g(85) == pytest.approx(1 - math.sqrt(0.25)) and g(99) < 0.03
    opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0)
    sched = get_lr_scheduler(opt, Config(scheduler="linear_warmup_constant_sqrt_decay", warmup_steps=2,
                                         train_num_steps=10, cooldown_steps=4))
    lrs = []
    for _ in range(10):
        lrs.append(opt.param_groups[0]["lr"])
        opt.step()
        sched.step()
    assert lrs[0] == 0.5 and lrs[2] == 1.0 and lrs[-1] < lrs[5]


def test_submit_dry_run_creates_job_dir(tmp_path):
    r = subprocess.run([sys.executable, str(ROOT / "submit.py"), "--config-file",
                        str(ROOT / "configs/gemma3/4b-synthetic.toml"), "--job-name", "j1", "--dump-dir",
                        str(tmp_path), "--dry-run", "--yes", "--dataset.eos-token", "7"],
                       capture_output=True, text=True, cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    job = tmp_path / "j1"
    assert (job / "config.json").exists() and (job / "slurm.sh").exists()
    assert (job / "logs").is_dir() and (job / "checkpoints").is_dir()
    cfg = Config(**json.loads((job / "config.json").read_text()))
    assert cfg.flavor == "4B" and cfg.dataset.eos_token == 7 and cfg.synthetic_data
    assert "dry_run" not in json.loads((job / "config.json").read_text())
    assert "--job-name=j1" in (job / "slurm.sh").read_text()


def test_every_shipped_config_is_a_valid_job_whose_degrees_fill_its_gpus():
    import tomllib
    from maester_b200.models import models_config
    for path in sorted((ROOT / "configs").rglob("*.toml")):
        cfg = Config(**tomllib.loads(path.read_text()))
        assert cfg.flavor in models_config[cfg.model_name], path
        shard = cfg.data_parallel_shard_degree
        fixed = cfg.data_parallel_replicate_degree * cfg.tensor_parallel_degree * cfg.context_parallel_degree
        gpus = cfg.num_nodes * 8
        assert gpus % fixed == 0 and (shard == -1 or shard * fixed == gpus), (path, shard, fixed, gpus)
        if cfg.tensor_parallel_degree > 1 and cfg.model_name == "gemma3":
            a = models_config["gemma3"][cfg.flavor]
            assert a.n_heads % cfg.tensor_parallel_degree == 0 and a.num_key_value_heads % cfg.tensor_parallel_degree == 0


def test_sweep_generation(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    import sweep
    sc = sweep.SweepConfig(sweep_name="s", base_config=Config(synthetic_data=True),
                           parameter_space={"opt_cfg.lr": sweep.SweepValues.logspace(-3, -2, 2),
                                            "flavor": ["1B", "4B"], "dataset.eos_token": [1]})
    cfgs = sweep.generate_configs(sc)
    assert len(cfgs) == 4
    name, cfg = next(iter(cfgs.items()))
    assert cfg.dump_dir == "jobs/s" and cfg.job_name == name and "lr1.0en03" in name
    assert all(g["opt_cfg"]["lr"] == pytest.approx(1e-3) for g in cfg.optimizer_groups)
    sweep.run_sweep(sc, dry_run=True)
    assert (tmp_path / "jobs/s/sweep_config.json").exists()
    assert len(list((tmp_path / "jobs/s").glob("*/config.json"))) == 4
    assert sweep.SweepValues.linspace(0, 1, 3).values == [0, 0.5, 1.0]


class FakeScheduler:
    def __init__(self):
        self.q, self.final, self.n = {}, {}, 100

    def queue(self):
        return dict(self.q)

    def submit(self, script, job_name):
        from job_manager import QueueEntry
        self.n += 1
        self.q[str(self.n)] = QueueEntry(str(self.n), job_name, "PD", "N/A", "0:00")
        return str(self.n)

    def cancel(self, job_id):
        self.q.pop(job_id, None)
        return True

    def final_state(self, job_id):
        return self.final.get(job_id)


def test_job_manager_policy(tmp_path):
    from job_manager import JobManager, QueueEntry, parse_slurm_time
    assert parse_slurm_time("1-02:03:04").total_seconds() == 93784 and parse_slurm_time("5:06").total_seconds() == 306
    job = tmp_path / "myjob"
    (job / "logs").mkdir(parents=True)
    (job / "slurm.sh").write_text("#!/bin/bash\n")
    now = [1_000_000.0]
    sched = FakeScheduler()
    mgr = JobManager(job, scheduler=sched, submit_interval=3600, horizon=3 * 3600, clock=lambda: now[0])
    s = mgr.tick()
    assert s["submitted"] == 3 and s["pending"] == 3  # horizon / interval copies kept pending
    ids = sorted(sched.q)
    # two copies start; only the longer-running healthy one may survive
    for jid, used in zip(ids[:2], ("2:00:00", "0:10:00")):
        sched.q[jid] = QueueEntry(jid, "myjob", "R", "N/A", used)
        log = job / "logs" / f"{jid}.out"
        log.write_text("step")
        os.utime(log, (now[0], now[0]))
    s = mgr.tick()
    assert s["cancelled"] == 1 and ids[1] not in sched.q and ids[0] in sched.q
    # the survivor goes stale: it is no longer a reason to cancel anything
    now[0] += 3600
    assert not mgr.is_job_healthy(ids[0])
    assert not mgr.should_cancel(ids[2], sched.queue())
    # a job that left the queue gets its final state recorded
    sched.q.pop(ids[0])
    sched.final[ids[0]] = ("TIMEOUT", "0:0")
    mgr.tick()
    assert ids[0] not in mgr.open_jobs()


def test_preflight_two_gloo_ranks(tmp_path):
    env = dict(os.environ, NCCL_PREFLIGHT_MAX_MB="1", NCCL_PREFLIGHT_ITERS="2", NCCL_PREFLIGHT_WARMUP="1",
               NCCL_PREFLIGHT_REPORT_DIR=str(tmp_path), NCCL_PREFLIGHT_DTYPES="fp32,bf16")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
                        "--nproc-per-node", "2", str(ROOT / "nccl_preflight.py")], capture_output=True, text=True,
                       env=env, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    rep = json.loads((tmp_path / "nccl_preflight_report.json").read_text())
    assert rep["world_size"] == 2 and len(rep["ranks"]) == 2
    assert rep["ranks"][1]["results"][0]["all_reduce"]["p50_us"] > 0
