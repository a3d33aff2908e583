"""Supervised fine-tuning data: conversations → ChatML tokens with role-based label masking.

``ConversationParquetDataset`` reads raw conversations through ``ParquetDataset`` in raw mode
(resumable, rank-sharded), renders each message as ``"{im_start}{role}\\n{content}{im_end}\\n"``,
adds BOS/EOS, truncates to ``max_seq_len + 1``, shifts into (input, label) pairs, masks labels with
``-100`` outside assistant turns (``assistant_only``) or nowhere (``all``) and pads.
``build_sft_data_loader`` selects between this and the pre-packed dataset.
Reference: maester/sft/dataset.py:22-309.
"""
from __future__ import annotations

import json
import os
from typing import Any

import torch

from maester_b200.datasets.experimental_otf import Checkpoint_Dataset, _Wrapper_Dataset
from maester_b200.datasets.parquet_dataset import ParquetDataset
from maester_b200.log_utils import logger

IGNORE = -100


def format_message(template: str, role: str, content: str, im_start: str, im_end: str) -> str:
    if template == "chatml":
        return f"{im_start}{role}\n{content}{im_end}\n"
    raise ValueError(f"Unknown template: {template}")


def tokenize_conversation(conversation, tokenizer, template: str, im_start: str, im_end: str):
    """→ (tokens incl. BOS/EOS, spans [(start, end, role)] of the messages inside ``tokens``)."""
    if isinstance(conversation, str):
        conversation = json.loads(conversation)
    tokens: list[int] = []
    spans = []
    if getattr(tokenizer, "bos_token_id", None) is not None:
        tokens.append(tokenizer.bos_token_id)
    for msg in conversation:
        ids = tokenizer.encode(format_message(template, msg["role"], msg["content"], im_start, im_end),
                               add_special_tokens=False)
        spans.append((len(tokens), len(tokens) + len(ids), msg["role"]))
        tokens.extend(ids)
    tokens.append(tokenizer.eos_token_id)
    return tokens, spans


def mask_labels(tokens: list[int], spans, strategy: str) -> list[int]:
    """Labels for ``tokens[1:]``: a label is kept when the *target* token lies in a trainable span."""
    role_at = [None] * len(tokens)
    for s, e, role in spans:
        for i in range(s, min(e, len(tokens))):
            role_at[i] = role
    out = []
    for i in range(1, len(tokens)):
        r = role_at[i]
        keep = r is not None and (strategy == "all" or (strategy == "assistant_only" and r == "assistant"))
        out.append(tokens[i] if keep else IGNORE)
    return out


class ConversationParquetDataset(_Wrapper_Dataset):
    def __init__(self, data_dir: str, rank: int, worldsize: int, tokenizer, max_seq_len: int,
                 template: str = "chatml", mask_strategy: str = "assistant_only",
                 conversation_column: str = "conversations", im_start: str = "<|im_start|>",
                 im_end: str = "<|im_end|>", seed: int = 42, shuffle: bool = True, verbose: bool = False):
        parent = ParquetDataset(data_dir, rank, worldsize, tokenizer, delimiter_token=tokenizer.eos_token_id,
                                bos_token=None, seed=seed, verbose=verbose, shuffle=shuffle,
                                data_column=conversation_column, process_fn=None, raw_data_mode=True)
        super().__init__(parent)
        self._tokenizer, self.max_seq_len = tokenizer, max_seq_len
        self.template, self.mask_strategy = template, mask_strategy
        self.im_start, self.im_end = im_start, im_end
        pad = getattr(tokenizer, "pad_token_id", None)
        self.pad_token_id = pad if pad is not None else tokenizer.eos_token_id

    def _process_conversation(self, conversation) -> dict[str, list[int]]:
        L = self.max_seq_len
        tokens, spans = tokenize_conversation(conversation, self._tokenizer, self.template, self.im_start, self.im_end)
        if len(tokens) < 2:
            return {"input_ids": [self.pad_token_id] * L, "labels": [IGNORE] * L, "attention_mask": [0] * L}
        tokens = tokens[: L + 1]
        inputs, labels = tokens[:-1], mask_labels(tokens, spans, self.mask_strategy)
        n = len(inputs)
        pad = L - n
        return {"input_ids": inputs + [self.pad_token_id] * pad, "labels": labels + [IGNORE] * pad,
                "attention_mask": [1] * n + [0] * pad}

    def __iter__(self):
        for conv in iter(self.dataset):
            item = self._process_conversation(conv)
            yield {k: torch.tensor(v, dtype=torch.long) for k, v in item.items()}


def packed_collate_fn(batch: list[dict[str, Any]]) -> dict[str, Any]:
    """Stack packed samples and report the number of non-padding tokens per sample."""
    out = {k: torch.stack([b[k] for b in batch]) for k in batch[0] if torch.is_tensor(batch[0][k])}
    if "attention_mask" in out:
        out["stats"] = {"actual_lengths": out["attention_mask"].long().sum(dim=1)}
    return out


def build_sft_data_loader(cfg, rank: int, world_size: int, tokenizer=None, resume_step: int | None = None):
    assert cfg.sft is not None, "cfg.sft must be set for SFT data"
    if cfg.sft.use_packed:
        from maester_b200.sft.packed_dataset import PackedSFTDataset
        ds = PackedSFTDataset(cfg.sft.packed_path, rank=rank, world_size=world_size, seed=cfg.sft.seed,
                              seq_len=cfg.seq_len)
        return torch.utils.data.DataLoader(ds, batch_size=cfg.train_batch_size, num_workers=0,
                                           collate_fn=packed_collate_fn, pin_memory=torch.cuda.is_available())
    if tokenizer is None:
        from transformers import AutoTokenizer, PreTrainedTokenizerFast
        tokenizer = (PreTrainedTokenizerFast(tokenizer_file=cfg.tokenizer_name) if os.path.isfile(cfg.tokenizer_name)
                     else AutoTokenizer.from_pretrained(cfg.tokenizer_name))
    if getattr(tokenizer, "eos_token_id", None) is None:
        raise ValueError(f"the tokenizer {cfg.tokenizer_name!r} defines no EOS token: every conversation ends with one "
                         "(a bare tokenizer.json carries no special-token roles; point tokenizer_name at a folder "
                         "saved with save_pretrained)")
    vocab = tokenizer.get_vocab() if hasattr(tokenizer, "get_vocab") else {}
    for tok in (cfg.sft.im_start_token, cfg.sft.im_end_token):
        if vocab and tok not in vocab:
            logger.warning(f"SFT marker token {tok!r} is not a single vocabulary entry; it will be split")
    assert len(cfg.dataset.data_dirs) == 1, "unpacked SFT reads one data directory"
    ds = ConversationParquetDataset(cfg.dataset.data_dirs[0], rank, world_size, tokenizer, cfg.seq_len,
                                    template=cfg.sft.template, mask_strategy=cfg.sft.mask_strategy,
                                    conversation_column=cfg.sft.conversation_column,
                                    im_start=cfg.sft.im_start_token, im_end=cfg.sft.im_end_token, seed=cfg.sft.seed)
    ckpt_dir = os.path.join(cfg.dump_dir, cfg.job_name, cfg.checkpoint_folder, "dataloader")
    ds = Checkpoint_Dataset(ds, ckpt_dir, cfg.checkpoint_interval,
                            steps_per_batch=cfg.train_batch_size * max(1, cfg.gradient_accumulation_steps),
                            save_path=ckpt_dir, load_step=resume_step)
    # the collate function adds the count of real tokens per sample, which the trainer turns into padding metrics
    return torch.utils.data.DataLoader(ds, batch_size=cfg.train_batch_size, num_workers=1, prefetch_factor=4,
                                       collate_fn=packed_collate_fn, pin_memory=torch.cuda.is_available(),
                                       persistent_workers=True)
