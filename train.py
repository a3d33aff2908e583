"""Training entry point: ``torchrun --standalone --nproc_per_node=N train.py jobs/<job_name>``.

The job directory holds ``config.json`` (written by ``submit.py``).  Flow, as in the reference
trainer (train.py:71-551): load config → take over garbage collection → process group (+ optional
NCCL preflight when ``RUN_NCCL_PREFLIGHT`` is set) → mesh → model on the meta device, parallelised
and initialised → data loader → optimizers / LR scheduler → checkpoint load → loop {micro-batches,
optimizer step, GC every ``gc_freq``, metrics on step 1 and every ``log_freq``, checkpoint save,
profiler step, tighten process-group timeouts after step 1} → final weights-only export.
"""
from __future__ import annotations

import gc
import json
import os
import sys
from dataclasses import dataclass
from datetime import timedelta
from pathlib import Path
from timeit import default_timer as timer
from typing import Any

import numpy as np
import torch
import torch.distributed as dist
from torch.distributed.checkpoint.stateful import Stateful
from torch.distributed.elastic.multiprocessing.errors import record

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from maester_b200.checkpoint import CheckpointManager, resume_step  # noqa: E402
from maester_b200.config import Config  # noqa: E402
from maester_b200.log_utils import init_logger, logger  # noqa: E402
from maester_b200.memory import cleanup_before_training  # noqa: E402
from maester_b200.metrics import WeightScaleMonitor, build_gpu_memory_monitor, build_metric_logger  # noqa: E402
from maester_b200.profiling import maybe_enable_memory_snapshot, maybe_enable_profiling  # noqa: E402
from maester_b200.trainer import Trainer  # noqa: E402
from maester_b200.utils import dist_max, dist_mean, init_distributed, set_pg_timeouts  # noqa: E402


@dataclass
class TrainState(Stateful):
    step: int = 0

    def state_dict(self) -> dict[str, Any]:
        return {"step": torch.tensor(self.step, dtype=torch.int32)}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        self.step = int(state_dict["step"].item())


def load_config(argv: list[str]) -> Config:
    if len(argv) > 1:
        path = Path(argv[1]) / "config.json"
        if not path.exists():
            raise ValueError(f"Config not found: {path}")
        logger.info(f"Loading config from {path}")
        with open(path) as f:
            return Config(**json.load(f))
    logger.info("Using the default configuration")
    return Config()


def build_data_loader(cfg: Config, trainer: Trainer):
    if cfg.synthetic_data:
        from maester_b200.datasets.synthetic import build_synthetic_data_loader
        return build_synthetic_data_loader(cfg, trainer.dp_rank, trainer.dp_degree, trainer.model_args.vocab_size)
    # the loader state that belongs to the model checkpoint this job resumes from (the newest loader state can be ahead)
    step = resume_step(cfg) if cfg.enable_checkpoint else None
    if cfg.sft is not None:
        from maester_b200.sft import build_sft_data_loader
        return build_sft_data_loader(cfg, rank=trainer.dp_rank, world_size=trainer.dp_degree, resume_step=step)
    from maester_b200.datasets.experimental_otf import build_experimental_data_loader
    return build_experimental_data_loader(cfg, rank=trainer.dp_rank, world_size=trainer.dp_degree, resume_step=step)


def tokenizer_vocab_size(cfg: Config) -> int | None:
    if cfg.synthetic_vocab_size > 0:
        return cfg.synthetic_vocab_size
    if cfg.synthetic_data:
        return None
    from transformers import AutoTokenizer, PreTrainedTokenizerFast
    if os.path.isfile(cfg.tokenizer_name):
        return len(PreTrainedTokenizerFast(tokenizer_file=cfg.tokenizer_name))
    return len(AutoTokenizer.from_pretrained(cfg.tokenizer_name))


@record
def main() -> None:
    init_logger()
    logger.info("Starting training.")
    cfg = load_config(sys.argv)
    if cfg.sft is not None:
        logger.info("SFT mode enabled")

    # garbage collection is run on our schedule so that no rank stalls at a random point
    gc.disable()
    gc.collect(1)

    if torch.cuda.is_available():
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    distributed = "WORLD_SIZE" in os.environ
    if distributed:
        init_distributed(cfg)
    if os.environ.get("RUN_NCCL_PREFLIGHT", "0").lower() in {"1", "true", "yes"} and distributed:
        from nccl_preflight import run_nccl_preflight
        logger.info("Running NCCL preflight checks (unset RUN_NCCL_PREFLIGHT or set to 0 to skip)")
        run_nccl_preflight()

    train_state = TrainState()
    with maybe_enable_memory_snapshot(cfg, global_step=train_state.step) as memory_profiler:
        gpu_memory_monitor = build_gpu_memory_monitor()
        trainer = Trainer(cfg, vocab_size=tokenizer_vocab_size(cfg))
        pd = trainer.parallel_dims
        logger.info(f"world mesh: {trainer.world_mesh}")
        mem = gpu_memory_monitor.get_peak_stats()
        logger.info(f"GPU memory usage for model: {mem.max_reserved_gib:.2f}GiB({mem.max_reserved_pct:.2f}%)")

        data_loader = build_data_loader(cfg, trainer)
        metric_logger = build_metric_logger(cfg)
        cleanup_before_training()
        weight_scale_monitor = WeightScaleMonitor(trainer.model, log_freq=cfg.log_freq)

        checkpoint = CheckpointManager(model=trainer.model, optimizer=trainer.optimizers,
                                       lr_scheduler=trainer.scheduler, dataloader=data_loader,
                                       states={"train_state": train_state}, cfg=cfg)
        checkpoint.load()
        trainer.step = train_state.step
        trainer.global_micro_step = train_state.step * trainer.grad_accum
        data_iterator = iter(data_loader)

        logger.info(f"Training starts at step {train_state.step}")
        with maybe_enable_profiling(cfg, global_step=train_state.step) as torch_profiler:
            checkpoint.reset()
            losses_since_last_log: list[torch.Tensor] = []
            padding_lengths: list[torch.Tensor] = []
            ntokens_since_last_log = 0
            total_tokens = 0
            data_loading_times: list[float] = []
            time_last_log = timer()
            gpu_memory_monitor.reset_peak_stats()

            while train_state.step < cfg.train_num_steps:
                micro = []
                for _ in range(trainer.grad_accum):
                    t0 = timer()
                    batch = next(data_iterator)
                    if "stats" in batch and "actual_lengths" in batch["stats"]:
                        padding_lengths.append(batch["stats"]["actual_lengths"])
                    ntokens_since_last_log += batch["labels"].numel()
                    data_loading_times.append(timer() - t0)
                    micro.append(batch)
                loss = trainer.train_step(micro)
                losses_since_last_log.append(loss)
                train_state.step += 1

                if train_state.step % cfg.gc_freq == 0:
                    gc.collect(1)
                weight_scale_stats = weight_scale_monitor.step_monitor()

                if train_state.step == 1 or train_state.step % cfg.log_freq == 0:
                    losses = torch.stack(losses_since_last_log).tolist()  # one device->host transfer
                    trainer.check_device_status()  # the host has just synchronised: a kernel that gave up shows here
                    avg_loss, max_loss = float(np.mean(losses)), float(np.max(losses))
                    if pd.dp_enabled:
                        global_avg_loss = dist_mean(avg_loss, trainer.dp_group).item()
                        global_max_loss = dist_max(max_loss, trainer.dp_group).item()
                    else:
                        global_avg_loss, global_max_loss = avg_loss, max_loss
                    time_delta = timer() - time_last_log
                    total_tokens += ntokens_since_last_log
                    # tokens per second per device, as the reference defines it
                    tps = ntokens_since_last_log / (time_delta * pd.model_parallel_size)
                    mfu = trainer.mfu(tps)
                    time_e2e = time_delta / cfg.log_freq
                    # per rank: mean time per batch and share of the logging interval; reported as the mean and the
                    # maximum over all ranks (tensor-parallel ranks load the same data redundantly)
                    t_data = float(np.mean(data_loading_times))
                    t_data_pct = 100 * float(np.sum(data_loading_times)) / max(time_delta, 1e-9)
                    if distributed:
                        t_data_avg, t_data_max = dist_mean(t_data).item(), dist_max(t_data).item()
                        t_data_pct_avg, t_data_pct_max = dist_mean(t_data_pct).item(), dist_max(t_data_pct).item()
                    else:
                        t_data_avg = t_data_max = t_data
                        t_data_pct_avg = t_data_pct_max = t_data_pct
                    mem = gpu_memory_monitor.get_peak_stats()
                    metrics = {
                        "loss/global_avg": global_avg_loss,
                        "loss/global_max": global_max_loss,
                        "tps": tps,
                        "mfu(%)": mfu,
                        "data/total_tokens": total_tokens * trainer.dp_degree,
                        "time/end_to_end(s)": time_e2e,
                        "time/data_loading_avg(s)": t_data_avg,
                        "time/data_loading_max(s)": t_data_max,
                        "time/data_loading_avg(%)": t_data_pct_avg,
                        "time/data_loading_max(%)": t_data_pct_max,
                        "memory/max_active(GiB)": mem.max_active_gib,
                        "memory/max_active(%)": mem.max_active_pct,
                        "memory/max_reserved(GiB)": mem.max_reserved_gib,
                        "memory/max_reserved(%)": mem.max_reserved_pct,
                        "memory/num_alloc_retries": mem.num_alloc_retries,
                        "memory/num_ooms": mem.num_ooms,
                        "lr": trainer.scheduler.get_last_lr()[0],
                    }
                    if padding_lengths:
                        lengths = torch.cat([p.flatten().float() for p in padding_lengths])
                        metrics["padding/efficiency"] = (lengths.mean() / cfg.seq_len).item()
                        metrics["padding/avg_length"] = lengths.mean().item()
                        metrics["padding/std_length"] = lengths.std().item() if lengths.numel() > 1 else 0.0
                    if weight_scale_stats:
                        metrics.update(weight_scale_stats)
                    metrics.update(trainer.pop_activation_stats())
                    dropped = trainer.pop_dropped_rows()
                    if dropped is not None:
                        metrics["moe/dropped_rows"] = dropped
                    hook_stats = getattr(trainer.optimizers, "_hook_stats", None)
                    if hook_stats:
                        metrics.update(hook_stats)
                    metric_logger.log(metrics, step=train_state.step)
                    logger.info(
                        f"Step {train_state.step:2}: lr={metrics['lr']:.2E}, loss={global_avg_loss:7.4f} "
                        f"(max={global_max_loss:7.4f}), tps={round(tps):,}, mfu={mfu:.2f}%, "
                        f"mem={mem.max_reserved_gib:.2f}GiB({mem.max_reserved_pct:.2f}%), "
                        f"time/data_loading={t_data_avg:.2f}s (max={t_data_max:.2f}s, {t_data_pct_max:.2f}%)"
                    )
                    losses_since_last_log.clear()
                    padding_lengths.clear()
                    ntokens_since_last_log = 0
                    data_loading_times.clear()
                    time_last_log = timer()
                    gpu_memory_monitor.reset_peak_stats()

                last = train_state.step == cfg.train_num_steps
                if checkpoint.will_save(train_state.step, force=last):
                    trainer.check_device_status(sync=True)  # never persist weights a failed kernel may have corrupted
                checkpoint.save(train_state.step, force=last)
                if torch_profiler is not None:
                    torch_profiler.step()
                if memory_profiler is not None:
                    memory_profiler.step()
                # start-up may be slow (first collectives, caches); afterwards a stuck rank should
                # be detected quickly
                if train_state.step == 1 and distributed:
                    set_pg_timeouts(timedelta(seconds=cfg.train_timeout_seconds), trainer.world_mesh)

        if torch.cuda.is_available():
            from maester_b200.ops import cuda as C
            C.check_status()
    metric_logger.close()
    logger.info("Training successfully completed!")
    if distributed:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
