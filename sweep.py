"""Cartesian hyper-parameter sweeps over job configs.

    python sweep.py submit sweep_config.py [--dry-run]
    python sweep.py status|cancel|retry|summarize|plot <sweep_name>

A sweep config is a Python file exposing ``config = SweepConfig(sweep_name=..., base_config=Config(...),
parameter_space={"dotted.key": [values] | SweepValues...})``.  Each combination becomes a job
directory under ``jobs/<sweep_name>/<job_name>`` (job names like ``lr1.0en03-wd1.0en01``); the
sweep itself is recorded in ``sweep_config.json`` and ``submission_summary.txt``.  Reference tool:
sweep.py:35-562.  ``status``/``cancel`` talk to SLURM (squeue/scancel), ``summarize``/``plot`` read
metrics from W&B when it is installed and reachable.
"""
from __future__ import annotations

import argparse
import importlib.util
import itertools
import json
import subprocess
import sys
from pathlib import Path
from typing import Any, Dict, List, Union

from pydantic import BaseModel
from pydantic_settings import BaseSettings, SettingsConfigDict

sys.path.insert(0, str(Path(__file__).resolve().parent))
from maester_b200.config import Config  # noqa: E402
from submit import setup_job_dir, submit_job, validate_config  # noqa: E402


class SweepValues(BaseModel):
    values: List[Any]

    @classmethod
    def from_list(cls, values: List[Any]) -> "SweepValues":
        return cls(values=list(values))

    @classmethod
    def linspace(cls, start: float, end: float, num: int) -> "SweepValues":
        step = (end - start) / (num - 1) if num > 1 else 0.0
        return cls(values=[start + step * i for i in range(num)])

    @classmethod
    def logspace(cls, start: float, end: float, num: int, base: float = 10) -> "SweepValues":
        return cls(values=[base ** e for e in cls.linspace(start, end, num).values])


class SweepConfig(BaseSettings):
    model_config = SettingsConfigDict(frozen=True, env_prefix="SWEEP_", cli_parse_args=False)
    base_config: Config = Config()
    sweep_name: str
    parameter_space: Dict[str, Union[List[Any], SweepValues]]


def format_param_value(value: Any) -> str:
    if isinstance(value, float):
        return f"{value:.1e}".replace("-", "n").replace("+", "p")
    return str(value).replace("-", "n")


def get_job_name(params: Dict[str, Any]) -> str:
    parts = []
    for key in sorted(params):
        short, val = key.split(".")[-1], params[key]
        if short == "lr":
            parts.append(f"lr{format_param_value(val)}")
        elif short == "weight_decay":
            parts.append(f"wd{format_param_value(val)}")
        elif short == "flavor":
            parts.append(str(val))
        else:
            parts.append(f"{short}{format_param_value(val)}")
    return "-".join(parts)


def set_nested_key(d: Dict[str, Any], key: str, value: Any) -> None:
    """``a.b.c`` walks dicts; the special prefix ``opt_cfg.`` sets the field in every optimizer group."""
    if key.startswith("opt_cfg."):
        for g in d.get("optimizer_groups", []):
            g.setdefault("opt_cfg", {})[key.split(".", 1)[1]] = value
        return
    keys = key.split(".")
    for k in keys[:-1]:
        d = d.setdefault(k, {})
    d[keys[-1]] = value


def generate_configs(sweep: SweepConfig) -> Dict[str, Config]:
    space = {k: (v if isinstance(v, SweepValues) else SweepValues.from_list(v)) for k, v in sweep.parameter_space.items()}
    names = list(space)
    out: Dict[str, Config] = {}
    for combo in itertools.product(*(space[n].values for n in names)):
        d = sweep.base_config.model_dump()
        d["dump_dir"] = str(Path("jobs") / sweep.sweep_name)
        chosen = dict(zip(names, combo))
        for k, v in chosen.items():
            set_nested_key(d, k, v)
        d["job_name"] = get_job_name(chosen)
        try:
            cfg = Config(**d)
        except Exception as e:  # noqa: BLE001
            print(f"Invalid config {d['job_name']}: {e}")
            continue
        if not [e for e in validate_config(cfg) if "Warning" not in e]:
            out[d["job_name"]] = cfg
    return out


def run_sweep(sweep: SweepConfig, dry_run: bool = False) -> None:
    configs = generate_configs(sweep)
    print(f"Generated {len(configs)} valid configurations")
    sweep_dir = Path("jobs") / sweep.sweep_name
    sweep_dir.mkdir(parents=True, exist_ok=True)
    (sweep_dir / "sweep_config.json").write_text(sweep.model_dump_json(indent=2))
    submitted, failed = [], []
    for name, cfg in configs.items():
        try:
            job_dir = setup_job_dir(cfg, assume_yes=True)
            if dry_run:
                print(f"Would submit {name}")
            else:
                job_id = submit_job(job_dir)
                submitted.append((name, job_id))
                print(f"Submitted {name} ({job_id})")
        except Exception as e:  # noqa: BLE001
            print(f"Failed to submit {name}: {e}")
            failed.append(name)
    lines = [f"Submitted jobs ({len(submitted)}):"] + [f"{n}: {j}" for n, j in submitted]
    if failed:
        lines += ["", f"Failed jobs ({len(failed)}):"] + failed
    (sweep_dir / "submission_summary.txt").write_text("\n".join(lines) + "\n")


def load_sweep_config(path: str) -> SweepConfig:
    spec = importlib.util.spec_from_file_location("sweep_config_module", path)
    if spec is None or spec.loader is None:
        raise SystemExit(f"Could not load {path}")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    if not hasattr(mod, "config"):
        raise SystemExit(f"No 'config' variable found in {path}")
    return mod.config


# ---------------------------------------------------------------------------- SLURM / W&B helpers
def _submitted(sweep_name: str) -> dict[str, str]:
    f = Path("jobs") / sweep_name / "submission_summary.txt"
    jobs: dict[str, str] = {}
    if f.exists():
        for line in f.read_text().splitlines():
            if ": " in line and not line.startswith(("Submitted", "Failed")):
                n, j = line.split(": ", 1)
                jobs[n] = j.strip()
    return jobs


def _squeue_states(job_ids: list[str]) -> dict[str, str]:
    if not job_ids:
        return {}
    try:
        r = subprocess.run(["squeue", "-h", "-j", ",".join(job_ids), "-o", "%i %T"], capture_output=True, text=True)
    except FileNotFoundError:
        return {}
    return dict(line.split()[:2] for line in r.stdout.splitlines() if line.strip())


def sweep_status(sweep_name: str) -> dict[str, str]:
    jobs = _submitted(sweep_name)
    states = _squeue_states(list(jobs.values()))
    table = {}
    for name, jid in jobs.items():
        job_dir = Path("jobs") / sweep_name / name
        done = any((job_dir / "checkpoints").glob("step-*")) if (job_dir / "checkpoints").exists() else False
        table[name] = states.get(jid, "FINISHED" if done else "NOT_IN_QUEUE")
        print(f"{name:40s} {jid:>10s} {table[name]}")
    return table


def sweep_cancel(sweep_name: str) -> None:
    for name, jid in _submitted(sweep_name).items():
        subprocess.run(["scancel", jid])
        print(f"cancelled {name} ({jid})")


def sweep_retry(sweep_name: str, dry_run: bool = False) -> None:
    """Resubmit the jobs of a sweep that are neither queued/running nor finished."""
    for name, state in sweep_status(sweep_name).items():
        if state == "NOT_IN_QUEUE":
            job_dir = Path("jobs") / sweep_name / name
            jid = submit_job(job_dir, dry_run=dry_run)
            print(f"resubmitted {name}: {jid}")


def sweep_summarize(sweep_name: str):
    """Final losses per job from W&B (project = sweep name); returns a pandas DataFrame."""
    import pandas as pd
    try:
        import wandb
        runs = list(wandb.Api().runs(sweep_name))
    except Exception as e:  # noqa: BLE001
        print(f"W&B query failed ({e}); no summary available")
        return pd.DataFrame()
    rows = [{"name": r.name, "state": r.state, "loss": r.summary.get("loss/global_avg"),
             "steps": r.summary.get("_step")} for r in runs]
    df = pd.DataFrame(rows).sort_values("loss")
    print(df.to_string(index=False))
    return df


def sweep_plot(sweep_name: str, out: str | None = None) -> None:
    df = sweep_summarize(sweep_name)
    if df.empty:
        return
    import matplotlib
    matplotlib.use("Agg")
    import matplotlib.pyplot as plt
    ax = df.plot.bar(x="name", y="loss", legend=False)
    ax.set_ylabel("final loss")
    plt.tight_layout()
    path = out or str(Path("jobs") / sweep_name / "sweep_loss.png")
    plt.savefig(path)
    print(f"wrote {path}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("submit")
    s.add_argument("config_path")
    s.add_argument("--dry-run", action="store_true")
    for name in ("status", "cancel", "summarize"):
        sub.add_parser(name).add_argument("sweep_name")
    r = sub.add_parser("retry")
    r.add_argument("sweep_name")
    r.add_argument("--dry-run", action="store_true")
    p = sub.add_parser("plot")
    p.add_argument("sweep_name")
    p.add_argument("--out")
    a = ap.parse_args(argv)
    if a.cmd == "submit":
        run_sweep(load_sweep_config(a.config_path), dry_run=a.dry_run)
    elif a.cmd == "status":
        sweep_status(a.sweep_name)
    elif a.cmd == "cancel":
        sweep_cancel(a.sweep_name)
    elif a.cmd == "retry":
        sweep_retry(a.sweep_name, a.dry_run)
    elif a.cmd == "summarize":
        sweep_summarize(a.sweep_name)
    elif a.cmd == "plot":
        sweep_plot(a.sweep_name, a.out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
