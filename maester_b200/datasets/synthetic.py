"""Synthetic packed-document batches (no tokenizer, no files).

Token ids are uniform over the vocabulary; documents have geometric, uniform or full-sequence
lengths and are separated by ``eos_id``; ``document_ids`` number the documents of each row and
``position_ids`` (optional) restart at every document, which is the layout the packed-SFT loader
produces (reference: maester/sft/packed_dataset.py:20-185).  The stream is a pure function of
(seed, rank, batch index), so a resumed run sees the same data.
"""
from __future__ import annotations

import numpy as np
import torch


def parse_doc_len(spec: str):
    kind, *rest = spec.split(":")
    if kind == "geometric":
        mean = float(rest[0])
        return lambda rng: int(rng.geometric(1.0 / mean))
    if kind == "uniform":
        lo, hi = int(rest[0]), int(rest[1])
        return lambda rng: int(rng.integers(lo, hi + 1))
    if kind == "full":
        return None
    raise ValueError(f"unknown synthetic_doc_len {spec!r}")


def make_batch(batch_size: int, seq_len: int, vocab_size: int, rng: np.random.Generator, doc_len=None,
               eos_id: int = 1, with_position_ids: bool = False, pin: bool = False) -> dict[str, torch.Tensor]:
    n = seq_len + 1
    toks = rng.integers(2, vocab_size, size=(batch_size, n), dtype=np.int64)
    docs = np.zeros((batch_size, n), dtype=np.int32)
    pos = np.tile(np.arange(n, dtype=np.int32), (batch_size, 1))
    if doc_len is not None:
        for b in range(batch_size):
            i, d = 0, 0
            while i < n:
                L = max(1, doc_len(rng))
                j = min(n, i + L)
                docs[b, i:j] = d
                pos[b, i:j] = np.arange(j - i)
                if j < n or j - i == L:
                    toks[b, j - 1] = eos_id
                i, d = j, d + 1
    out = {
        "input_ids": torch.from_numpy(toks[:, :-1].copy()),
        "labels": torch.from_numpy(toks[:, 1:].copy()),
        "document_ids": torch.from_numpy(docs[:, :-1].copy()),
    }
    if with_position_ids:
        out["position_ids"] = torch.from_numpy(pos[:, :-1].copy())
    if pin and torch.cuda.is_available():
        out = {k: v.pin_memory() for k, v in out.items()}
    return out


class SyntheticLoader:
    """Infinite iterator of packed batches; ``state_dict`` / ``load_state_dict`` make it resumable."""

    def __init__(self, batch_size: int, seq_len: int, vocab_size: int, doc_len_spec: str = "geometric:1500",
                 seed: int = 0, rank: int = 0, eos_id: int = 1, with_position_ids: bool = False, pin: bool = True):
        self.batch_size, self.seq_len, self.vocab_size = batch_size, seq_len, vocab_size
        self.doc_len = parse_doc_len(doc_len_spec)
        self.seed, self.rank, self.eos_id = seed, rank, eos_id
        self.with_position_ids, self.pin = with_position_ids, pin
        self.index = 0

    def __iter__(self):
        return self

    def __next__(self) -> dict[str, torch.Tensor]:
        rng = np.random.default_rng([self.seed, self.rank, self.index])
        self.index += 1
        return make_batch(self.batch_size, self.seq_len, self.vocab_size, rng, self.doc_len, self.eos_id,
                          self.with_position_ids, self.pin)

    def state_dict(self) -> dict:
        return {"index": self.index, "seed": self.seed, "rank": self.rank}

    def load_state_dict(self, sd: dict) -> None:
        self.index = int(sd["index"])


def build_synthetic_data_loader(cfg, rank: int, world_size: int, vocab_size: int) -> SyntheticLoader:
    return SyntheticLoader(cfg.train_batch_size, cfg.seq_len, vocab_size, cfg.synthetic_doc_len, seed=0, rank=rank,
                           eos_id=cfg.dataset.eos_token if cfg.dataset.eos_token < vocab_size else 1,
                           with_position_ids=cfg.sft is not None)
