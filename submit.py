"""Create a job directory from a config and submit it to SLURM.

    python submit.py --config-file configs/gemma3/12b-base.toml [--any-config-field value ...]
                     [--dry-run] [--validate-only] [--yes]

Sources, strongest first: command line (kebab-case flag for every ``Config`` field, nested ones as
``--dataset.eos-token``), the TOML file given by ``--config-file``, ``SUBMIT_*`` environment
variables.  The job directory ``<dump_dir>/<job_name>/`` receives ``config.json`` (what ``train.py``
loads), ``slurm.sh`` rendered from ``templates/slurm.sh``, ``logs/``, ``checkpoints/`` and, with
TensorBoard on, the tb folder.  Behaviour follows the reference tool (submit.py:24-208);
``--yes`` (new) answers the interactive prompts for scripted use.
"""
from __future__ import annotations

import argparse
import subprocess
import sys
from pathlib import Path
from typing import Optional

from pydantic import Field
from pydantic_settings import BaseSettings, PydanticBaseSettingsSource, SettingsConfigDict, TomlConfigSettingsSource

sys.path.insert(0, str(Path(__file__).resolve().parent))
from maester_b200.config import Config  # noqa: E402

TEMPLATE_PATH = Path(__file__).resolve().parent / "templates" / "slurm.sh"


class SubmitConfig(Config):
    model_config = SettingsConfigDict(frozen=True, env_prefix="SUBMIT_", protected_namespaces=(),
                                      arbitrary_types_allowed=True, cli_parse_args=True, cli_kebab_case=True,
                                      cli_implicit_flags=True)
    dry_run: bool = False
    validate_only: bool = False
    yes: bool = False
    config_file: Optional[str] = Field(None, exclude=False)

    @classmethod
    def settings_customise_sources(cls, settings_cls: type[BaseSettings], init_settings, env_settings,
                                   dotenv_settings, file_secret_settings) -> tuple[PydanticBaseSettingsSource, ...]:
        pre = argparse.ArgumentParser(add_help=False)
        pre.add_argument("--config-file", type=str)
        known, _ = pre.parse_known_args()
        sources = [init_settings]
        if known.config_file and Path(known.config_file).exists():
            sources.append(TomlConfigSettingsSource(settings_cls, known.config_file))
        sources += [env_settings, dotenv_settings, file_secret_settings]
        return tuple(sources)


SUBMIT_ONLY = ("dry_run", "validate_only", "yes", "config_file")


def validate_config(cfg: Config) -> list[str]:
    """Problems that would make the job fail at start-up; empty list if none."""
    errors = []
    if not cfg.synthetic_data:
        for d in cfg.dataset.data_dirs:
            if not Path(d).exists():
                errors.append(f"Data directory not found: {d}")
    gpus = cfg.num_nodes * 8
    dp_shard = cfg.data_parallel_shard_degree
    fixed = cfg.data_parallel_replicate_degree * cfg.tensor_parallel_degree * cfg.context_parallel_degree
    if dp_shard != -1 and dp_shard * fixed != gpus:
        errors.append(f"Warning: parallel degrees multiply to {dp_shard * fixed} but the job has {gpus} GPUs")
    return errors


def setup_job_dir(cfg: Config, assume_yes: bool = False) -> Path:
    dump = Path(cfg.dump_dir)
    dump.mkdir(exist_ok=True, parents=True)
    job = dump / cfg.job_name
    if job.exists() and not assume_yes:
        if input(f"Job folder {job} already exists. Continue? (y/N): ").lower() != "y":
            raise ValueError("Job folder already exists")
    for sub in ("", "logs", "checkpoints"):
        (job / sub).mkdir(exist_ok=True)
    if cfg.enable_tensorboard:
        (job / cfg.save_tb_folder).mkdir(exist_ok=True)
    (job / "config.json").write_text(cfg.model_dump_json(indent=2))
    script = TEMPLATE_PATH.read_text().format(
        job_name=cfg.job_name, dump_dir=cfg.dump_dir, num_nodes=cfg.num_nodes, partition=cfg.partition,
        account=cfg.account, time=cfg.time, container=cfg.container)
    (job / "slurm.sh").write_text(script)
    return job


def submit_job(job_dir: Path, dry_run: bool = False) -> str | None:
    if dry_run:
        print(f"Would submit job with command: sbatch {job_dir}/slurm.sh")
        return None
    try:
        res = subprocess.run(["sbatch", str(job_dir / "slurm.sh")], capture_output=True, text=True, check=True)
    except subprocess.CalledProcessError as e:
        print(f"Job submission failed: {e.stderr}")
        raise
    return res.stdout.strip().split()[-1]


def main() -> int:
    cfg = SubmitConfig()
    print(cfg.model_dump_json(indent=2))
    if not cfg.yes and input("\nValidate configuration? (y/N): ").lower() != "y":
        return 1
    errors = validate_config(cfg)
    if errors:
        print("Configuration validation failed:")
        for e in errors:
            print(f"- {e}")
        if not all("Warning" in e for e in errors):
            return 1
    if cfg.validate_only:
        return 0
    print("\nJob Configuration:")
    print(f"Name: {cfg.job_name}")
    print(f"Model: {cfg.model_name} ({cfg.flavor})")
    print(f"Nodes: {cfg.num_nodes} ({cfg.num_nodes * 8} GPUs)")
    print(f"Parallelism: DP={cfg.data_parallel_shard_degree}x{cfg.data_parallel_replicate_degree}, "
          f"TP={cfg.tensor_parallel_degree}, CP={cfg.context_parallel_degree}, EP={cfg.expert_parallel_degree}")
    print(f"Batch size: {cfg.train_batch_size} per GPU")
    if not cfg.dry_run and not cfg.yes and input("\nSubmit job? (y/N): ").lower() != "y":
        return 0
    fields = cfg.model_dump()
    for k in SUBMIT_ONLY:
        fields.pop(k, None)
    job_dir = setup_job_dir(Config(**fields), assume_yes=cfg.yes)
    print(f"\nPrepared job directory: {job_dir}")
    try:
        job_id = submit_job(job_dir, dry_run=cfg.dry_run)
        if job_id:
            print(f"Submitted job {job_id}")
    except Exception as e:  # noqa: BLE001
        print(f"Failed to submit job: {e}")
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
