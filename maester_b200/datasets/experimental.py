"""Legacy loader over PRE-TOKENISED Arrow IPC shards (reference: maester/datasets/experimental.py,
``Streaming_Doc_Dataset`` :559-874 of the on-the-fly file; unused by the reference's train.py:28-29).

Layout: ``<data_dir>/<dataset>/*.arrow`` files whose record batches hold one document each in a
``tokens`` column (uint32), and ``<data_dir>/meta/*counts*.csv`` with rows
``dataset/filename,documents,tokens``.  Here the format is one more document source of the current
pipeline: ``ArrowShardDataset`` reuses the Parquet source's ownership split, LCG document order,
chunking and resumable state, so everything downstream (sampling, packing, shuffle buffer,
checkpointing) is shared.  ``scripts/generate_fake_data.py`` writes a tiny dataset in this layout.
"""
from __future__ import annotations

import csv
import glob
import os
from typing import Any, Optional, Set

import torch

from maester_b200.datasets.experimental_otf import (Buffer_Dataset, Checkpoint_Dataset, Preload_Buffer_Dataset,
                                                    Preprocess_Dataset, causal_lm)
from maester_b200.datasets.parquet_dataset import ParquetDataset, Sampling_Dataset


class ArrowShardDataset(ParquetDataset):
    def __init__(self, data_dir: str, rank: int, worldsize: int, delimiter_token: Any, bos_token: Optional[Any] = None,
                 strip_tokens: Optional[Set[Any]] = None, seed: int = 42, min_length: int = 1, max_chunksize: int = 1024,
                 verbose: bool = False, shuffle: bool = True, meta_dir: Optional[str] = None, column: str = "tokens"):
        self._meta_dir = meta_dir or os.path.join(os.path.dirname(os.path.normpath(data_dir)), "meta")
        self._column = column
        self._open_arrow: tuple[str, Any] | None = None
        super().__init__(data_dir, rank, worldsize, tokenizer=None, delimiter_token=delimiter_token, bos_token=bos_token,
                         strip_tokens=strip_tokens, seed=seed, min_length=min_length, max_chunksize=max_chunksize,
                         verbose=verbose, shuffle=shuffle, data_column=column, process_fn=lambda toks: toks,
                         cache_row_groups=False)

    file_suffix = ".arrow"

    def _count_docs(self) -> None:
        counts: dict[str, int] = {}
        for meta in sorted(glob.glob(os.path.join(self._meta_dir, "*counts*.csv"))):
            with open(meta) as f:
                for row in csv.DictReader(f):
                    counts[row["dataset/filename"].lstrip("/")] = int(row["documents"])
        root = os.path.dirname(os.path.normpath(self.data))
        for p in self.parquet_files:
            rel = os.path.relpath(p, root)
            if rel in counts:
                self.docs_per_file[p] = counts[rel]
            else:  # no metadata row: ask the file
                import pyarrow as pa
                with pa.memory_map(p) as src:
                    self.docs_per_file[p] = pa.ipc.open_file(src).num_record_batches

    def _read_row(self, path: str, row: int):
        import pyarrow as pa
        if self._open_arrow is None or self._open_arrow[0] != path:
            self._open_arrow = (path, pa.ipc.open_file(pa.memory_map(path)))
        return self._open_arrow[1].get_batch(row)[self._column].to_pylist()

    def __getstate__(self):  # memory maps do not pickle (DataLoader workers)
        d = dict(self.__dict__)
        d["_open_arrow"] = None
        return d


def build_legacy_data_loader(cfg, rank: int, world_size: int):
    """The reference's legacy stack over Arrow shards: per-source document streams -> weighted
    sampling -> packing to ``seq_len + 1`` -> shuffle window -> (input, label) pairs -> batches."""
    ds_cfg = cfg.dataset
    eos, bos = ds_cfg.eos_token, ds_cfg.bos_token
    sources = [ArrowShardDataset(d, rank, world_size, delimiter_token=eos, bos_token=bos,
                                 strip_tokens=set(ds_cfg.drop_tokens or []), max_chunksize=cfg.seq_len + 1)
               for d in ds_cfg.data_dirs]
    data = Sampling_Dataset(sources, ds_cfg.dataset_weights, delimiter_token=eos) if len(sources) > 1 else sources[0]
    data = Buffer_Dataset(data, cfg.seq_len + 1, pack_hard=True, bos_token=bos, eos_token=eos)
    data = Preload_Buffer_Dataset(data, 10000)
    data = Preprocess_Dataset(data, causal_lm)
    data = Checkpoint_Dataset(data, os.path.join(cfg.dump_dir, cfg.job_name, cfg.checkpoint_folder, "dataloader"),
                              cfg.checkpoint_interval, cfg.train_batch_size)
    return torch.utils.data.DataLoader(data, batch_size=cfg.train_batch_size, num_workers=0)
