"""``build_experimental_data_loader``: assemble the pre-training pipeline for one data-parallel rank
(reference: maester/datasets/experimental_otf.py:1519-1620)."""
from __future__ import annotations

import os

import torch

from maester_b200.datasets.experimental_otf import (
    Buffer_Dataset,
    Checkpoint_Dataset,
    Preload_Buffer_Dataset,
    Preprocess_Dataset,
    causal_lm,
)
from maester_b200.datasets.parquet_dataset import ParquetDataset, Sampling_Dataset


def parse_data_args(datas, weights):
    """Comma-separated strings (or lists) → (list of sources, list of float weights or None)."""
    def split(x, cast):
        if isinstance(x, (list, tuple)):
            return [cast(v) for v in x]
        return [cast(v) for v in str(x).split(",") if str(v).strip()]

    d = split(datas, str)
    w = split(weights, float) if weights not in (None, "") else None
    return d, w


def build_experimental_data_loader(cfg, rank: int, world_size: int, tokenizer=None, resume_step: int | None = None):
    """Sampling → Buffer(seq_len+1, hard) → Preload(10000) → Preprocess(causal_lm) → Checkpoint → DataLoader.

    The DataLoader uses exactly one worker process: the pipeline keeps its position in Python objects
    that live inside that worker, and ``Checkpoint_Dataset`` saves them from there.
    """
    if tokenizer is None:
        from transformers import AutoTokenizer, PreTrainedTokenizerFast
        if os.path.isfile(cfg.tokenizer_name):
            tokenizer = PreTrainedTokenizerFast(tokenizer_file=cfg.tokenizer_name)
        else:
            tokenizer = AutoTokenizer.from_pretrained(cfg.tokenizer_name)
    dirs, weights = parse_data_args(cfg.dataset.data_dirs, cfg.dataset.dataset_weights)
    drop = {int(x) for x in str(cfg.dataset.drop_tokens).split(",") if str(x).strip()}
    sources = [
        # the reference's arguments (maester/datasets/experimental_otf.py:1565-1578): documents shorter than 3 tokens
        # are skipped, chunks of at most 1024 tokens, no BOS when the config says -1; with them the token stream and
        # the saved loader state are the reference's
        ParquetDataset(d, rank, world_size, tokenizer, delimiter_token=cfg.dataset.eos_token,
                       bos_token=None if cfg.dataset.bos_token == -1 else cfg.dataset.bos_token, strip_tokens=drop,
                       min_length=3, seed=42, max_chunksize=1024, cache_row_groups=cfg.dataset.cache_row_groups)
        for d in dirs
    ]
    ds = Sampling_Dataset(sources, weights, delimiter_token=cfg.dataset.eos_token, rank=rank, worldsize=world_size)
    ds = Buffer_Dataset(ds, cfg.seq_len + 1, pack_hard=True)
    ds = Preload_Buffer_Dataset(ds, 10000)
    ds = Preprocess_Dataset(ds, causal_lm)
    ckpt_dir = os.path.join(cfg.dump_dir, cfg.job_name, cfg.checkpoint_folder, "dataloader")
    ds = Checkpoint_Dataset(ds, ckpt_dir, cfg.checkpoint_interval,
                            steps_per_batch=cfg.train_batch_size * max(1, cfg.gradient_accumulation_steps),
                            save_path=ckpt_dir, load_step=resume_step)
    workers = 1  # more than one worker would duplicate the stateful pipeline
    return torch.utils.data.DataLoader(ds, batch_size=cfg.train_batch_size, num_workers=workers,
                                       prefetch_factor=8, pin_memory=torch.cuda.is_available(),
                                       persistent_workers=True)
