"""Pre-packed SFT data: several conversations per fixed-length sequence.

Input: the parquet file written by ``scripts/pack_sft_data.py`` with columns ``pack_id, input_ids,
labels, attention_mask, conversation_ids, boundaries`` where ``boundaries`` lists
``(conversation id, start, length)`` per packed conversation.  Each sample gets ``position_ids``
that restart at 0 for every conversation and ``document_ids`` 0, 1, 2, … per conversation (−1 on
padding), which the attention kernel turns into a block-diagonal causal mask.
Rank r takes samples ``r, r + world, …``; every epoch is reshuffled with ``RandomState(seed + epoch)``;
iteration is endless.  ``state_dict`` / ``load_state_dict`` (an addition over the reference, which
cannot resume) restore the epoch and the position inside it.
Reference: maester/sft/packed_dataset.py:20-258.
"""
from __future__ import annotations

import numpy as np
import torch
from torch.utils.data import Dataset


def position_ids_from_boundaries(boundaries, seq_len: int) -> torch.Tensor:
    pos = torch.zeros(seq_len, dtype=torch.long)
    for _, start, length in boundaries:
        end = min(int(start) + int(length), seq_len)
        pos[int(start):end] = torch.arange(end - int(start))
    return pos


def document_ids_from_boundaries(boundaries, seq_len: int) -> torch.Tensor:
    doc = torch.full((seq_len,), -1, dtype=torch.long)
    for i, (_, start, length) in enumerate(boundaries):
        doc[int(start):min(int(start) + int(length), seq_len)] = i
    return doc


class PackedSFTDataset(Dataset):
    def __init__(self, packed_path: str, rank: int = 0, world_size: int = 1, seed: int = 42, seq_len: int | None = None,
                 infinite: bool = True):
        import pandas as pd

        self.df = pd.read_parquet(packed_path)
        self.rank, self.world_size, self.seed, self.seq_len, self.infinite = rank, world_size, seed, seq_len, infinite
        self.rank_indices = np.arange(len(self.df))[rank::world_size]
        self.num_samples = len(self.rank_indices)
        assert self.num_samples > 0, "no packed samples for this rank"
        self.epoch, self.current_idx = 0, 0
        self._prepare_epoch()

    def _prepare_epoch(self) -> None:
        rng = np.random.RandomState(self.seed + self.epoch)
        self.epoch_indices = self.rank_indices[rng.permutation(self.num_samples)]
        self.current_idx = 0

    def __len__(self) -> int:
        return 2 ** 40 if self.infinite else self.num_samples

    def _fit(self, t: torch.Tensor, fill) -> torch.Tensor:
        if self.seq_len is None or t.numel() == self.seq_len:
            return t
        if t.numel() > self.seq_len:
            return t[: self.seq_len]
        return torch.cat([t, torch.full((self.seq_len - t.numel(),), fill, dtype=t.dtype)])

    def __getitem__(self, idx: int) -> dict[str, torch.Tensor]:
        if self.infinite:  # position is internal state: the sampler's index is ignored
            if self.current_idx >= self.num_samples:
                self.epoch += 1
                self._prepare_epoch()
            actual = self.epoch_indices[self.current_idx]
            self.current_idx += 1
        else:
            actual = self.rank_indices[idx % self.num_samples]
        pack = self.df.iloc[int(actual)]
        ids = torch.tensor(np.asarray(pack["input_ids"]), dtype=torch.long)
        n = ids.numel()
        bounds = [tuple(int(v) for v in b) for b in pack["boundaries"]]
        return {
            "input_ids": self._fit(ids, 0),
            "labels": self._fit(torch.tensor(np.asarray(pack["labels"]), dtype=torch.long), -100),
            "attention_mask": self._fit(torch.tensor(np.asarray(pack["attention_mask"]), dtype=torch.long), 0).bool(),
            "position_ids": self._fit(position_ids_from_boundaries(bounds, n), 0),
            "document_ids": self._fit(document_ids_from_boundaries(bounds, n), -1),
        }

    def state_dict(self) -> dict:
        return {"epoch": self.epoch, "current_idx": self.current_idx}

    def load_state_dict(self, sd: dict) -> None:
        self.epoch = int(sd["epoch"])
        self._prepare_epoch()
        self.current_idx = int(sd["current_idx"])


def create_packed_dataloader(packed_path: str, batch_size: int, rank: int = 0, world_size: int = 1, seed: int = 42,
                             seq_len: int | None = None, num_workers: int = 0):
    from maester_b200.sft.dataset import packed_collate_fn

    ds = PackedSFTDataset(packed_path, rank, world_size, seed, seq_len)
    return torch.utils.data.DataLoader(ds, batch_size=batch_size, num_workers=num_workers, collate_fn=packed_collate_fn,
                                       pin_memory=torch.cuda.is_available())
