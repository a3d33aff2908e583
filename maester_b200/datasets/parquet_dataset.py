"""Document sources of the data pipeline: ``ParquetDataset`` (on-the-fly tokenisation), the
weighted ``Sampling_Dataset`` over several sources and the rescalable ``Scalable_Shard_Dataset``.

Reference: maester/datasets/experimental_otf.py:876-1513.
"""
from __future__ import annotations

import bisect
import hashlib
import json
import math
import os
import random
from collections import OrderedDict
from typing import Any, Callable, List, Optional, Set

import torch

from maester_b200.datasets.experimental_otf import (
    _Stateful_Dataset,
    _dist_barrier,
    _dist_rank,
    _shard_partition,
)
from maester_b200.log_utils import logger


class ParquetDataset(_Stateful_Dataset):
    """Yields token chunks (or raw column values) of the documents this rank owns.

    Ownership: every file is cut into ``worldsize`` fragments and rank r takes the fragments
    ``[r*F, (r+1)*F)`` of the file-major fragment list, i.e. a contiguous ``(file, first doc, last doc)``
    range per file.  Within a range documents are visited in the order of a full-period LCG over the
    next power of two (values outside the range are skipped), so no index list is materialised.
    Rank 0 counts rows per file once and caches the counts next to the data, keyed by a hash of file
    names and sizes; other ranks wait at a barrier.
    """

    file_suffix = ".parquet"  # subclasses reading another container format override this

    def __init__(self, data_dir: str, rank: int, worldsize: int, tokenizer, delimiter_token: Any,
                 bos_token: Optional[Any] = None, strip_tokens: Optional[Set[Any]] = None, seed: int = 42,
                 min_length: int = 1, max_chunksize: int = 1024, verbose: bool = False, shuffle: bool = True,
                 data_column: str = "text", process_fn: Optional[Callable] = None, raw_data_mode: bool = False,
                 cache_row_groups: bool = True, max_cached_row_groups: int = 8):
        super().__init__(rank, worldsize)
        assert max_chunksize > 0
        self.seed, self.data, self.tokenizer = seed, data_dir, tokenizer
        self.min_length, self.chunksize = min_length, max_chunksize
        self.eos, self.bos, self.drop = delimiter_token, bos_token, strip_tokens or set()
        self.verbose, self.data_column, self.raw_data_mode = verbose, data_column, raw_data_mode
        self.process_fn = process_fn or self._default_process
        self.cache_row_groups, self.max_cached = cache_row_groups, max_cached_row_groups
        self._row_group_prefix: dict[str, list[int]] = {}
        self._row_group_cache: dict[str, OrderedDict] = {}
        self.docs_per_file: dict[str, int] = {}
        rng = random.Random(seed + rank)  # deliberately different shuffles on different ranks

        self.parquet_files = sorted(os.path.join(r, f) for r, _, fs in os.walk(data_dir) for f in fs
                                    if f.endswith(self.file_suffix))
        assert self.parquet_files, f"No {self.file_suffix} files found in {data_dir}"
        cache_file = os.path.join(data_dir, f"doc_counts_cache_{self._dataset_hash()}.json")
        if _dist_rank() == 0 and not os.path.exists(cache_file):
            self._count_docs()
            with open(cache_file, "w") as f:
                json.dump({os.path.relpath(k, data_dir): v for k, v in self.docs_per_file.items()}, f)
        _dist_barrier()
        with open(cache_file) as f:
            self.docs_per_file = {os.path.join(data_dir, k): v for k, v in json.load(f).items()}
        _dist_barrier()

        nfiles = len(self.parquet_files)
        ranges: "OrderedDict[str, list[int]]" = OrderedDict()
        for i in range(rank * nfiles, (rank + 1) * nfiles):  # fragments i of the file-major list
            path, frag = self.parquet_files[i // worldsize], i % worldsize
            n = self.docs_per_file[path]
            lo, hi = (n * frag) // worldsize, (n * frag + n) // worldsize - 1
            if hi < lo:
                continue
            cur = ranges.setdefault(path, [lo, hi])
            cur[0], cur[1] = min(cur[0], lo), max(cur[1], hi)
        self.docset = [(p, lo, hi) for p, (lo, hi) in ranges.items()]
        self._len = sum(hi - lo + 1 for _, lo, hi in self.docset)
        if verbose:
            logger.info(f"Worker {rank} responsible for docs: {self.docset} (total {self._len})")
        if shuffle:
            rng.shuffle(self.docset)

        self.docset_index = 0
        self.chunk_index = -1
        self.completed_current_doc = False
        self.epochs_seen, self.tokens_seen, self.docs_seen, self.percent_seen = -1, 0, 0, 0
        self.lcg_state = seed + rank
        self.state_params = ["docset_index", "chunk_index", "completed_current_doc", "epochs_seen", "tokens_seen",
                             "docs_seen", "percent_seen", "lcg_state"]

    # ------------------------------------------------------------------ setup helpers
    def _default_process(self, text):
        return self.tokenizer.encode(text, add_special_tokens=False, padding=False, truncation=False)

    def _dataset_hash(self) -> str:
        h = hashlib.md5()
        for p in self.parquet_files:
            h.update(f"{os.path.relpath(p, self.data)}:{os.path.getsize(p)}".encode())
        return h.hexdigest()[:16]

    def _count_docs(self) -> None:
        import pyarrow.parquet as pq
        for p in self.parquet_files:
            self.docs_per_file[p] = pq.ParquetFile(p).metadata.num_rows

    def _locate(self, index: int):
        """Global owned-document index → (file, size of the owned range, first owned row)."""
        cur = 0
        for path, lo, hi in self.docset:
            n = hi - lo + 1
            if cur + n > index:
                return path, n, lo
            cur += n
        raise IndexError(f"document index {index} out of range ({self._len})")

    def _reader(self, path: str):
        import pyarrow.parquet as pq
        if getattr(self, "_open_path", None) != path:
            self._open_path, self._open_reader = path, pq.ParquetFile(path)
            if path not in self._row_group_prefix:
                md = self._open_reader.metadata
                sizes = [md.row_group(i).num_rows for i in range(md.num_row_groups)]
                self._row_group_prefix[path] = [sum(sizes[: i + 1]) for i in range(len(sizes))]
                self._row_group_cache[path] = OrderedDict()
        return self._open_reader

    def _read_row(self, path: str, row: int):
        reader = self._reader(path)
        prefix = self._row_group_prefix[path]
        g = bisect.bisect_right(prefix, row)
        assert g < len(prefix), f"row {row} beyond the end of {path}"
        off = row - (prefix[g - 1] if g else 0)
        cache = self._row_group_cache[path]
        if self.cache_row_groups and g in cache:
            cache.move_to_end(g)
            table = cache[g]
        else:
            table = reader.read_row_group(g, columns=[self.data_column])
            if self.cache_row_groups:
                cache[g] = table
                while len(cache) > self.max_cached:
                    cache.popitem(last=False)
        return table[self.data_column][off].as_py()

    def _next_doc_slot(self, size: int) -> int:
        """Next value of the LCG restricted to [0, size): a bijection over one period."""
        m = 2 ** math.ceil(math.log2(max(size, 2)))
        a, c = 5, (self.rank + self.seed) * 2 + 1
        state = self.lcg_state
        while True:
            state = (a * state + c) % m
            if state < size:
                return state

    def _chunk(self, j: int, doc: list, n_chunks: int) -> list:
        start, pull = j * self.chunksize, self.chunksize
        if self.bos is not None:
            if j == 0:
                pull -= 1
            else:
                start -= 1
        chunk = doc[start:start + pull]
        self.tokens_seen += len(chunk)
        if self.bos is not None and j == 0:
            chunk = [self.bos] + chunk
        if j == n_chunks - 1:
            chunk = chunk + [self.eos]
        return chunk

    def _tokens_of(self, path: str, row: int):
        doc = self.process_fn(self._read_row(path, row))
        if len(doc) < 2:
            return None, 0
        if doc[0] in self.drop:
            doc = doc[1:]
        if doc and doc[-1] in self.drop:
            doc = doc[:-1]
        doclen = len(doc) + (1 if self.bos is None else 2)
        if doclen < self.min_length:
            return None, 0
        return doc, math.ceil(doclen / self.chunksize)

    # ------------------------------------------------------------------ iteration
    def __iter__(self):
        ndocs = self._len
        start_index = self.docset_index
        start_lcg = self.lcg_state
        skip_chunks = self.chunk_index + 1   # chunks of the first document that were already emitted
        resume_same_doc = (not self.completed_current_doc) and self.chunk_index >= 0
        if self.completed_current_doc:       # saved right after a document ended: continue with the next
            start_index = (start_index + 1) % ndocs
            self.completed_current_doc = False
            skip_chunks = 0
        first_slot = None
        while True:
            for i in range(ndocs):
                index = (start_index + i) % ndocs
                self.completed_current_doc = False
                if index == 0:
                    self.epochs_seen += 1
                self.docset_index = index
                path, size, first_row = self._locate(index)
                if i == 0 and resume_same_doc:
                    slot = self.lcg_state          # the LCG already points at the unfinished document
                else:
                    slot = self._next_doc_slot(size)
                    self.lcg_state = slot
                if i == 0:
                    first_slot = slot
                if self.raw_data_mode:
                    self.docs_seen += 1
                    self.percent_seen = self.docs_seen * 100 / (ndocs + 1e-9)
                    self.completed_current_doc = True
                    yield self._read_row(path, slot + first_row)
                    continue
                doc, n_chunks = self._tokens_of(path, slot + first_row)
                if doc is None:
                    continue
                for j in range(n_chunks):
                    if i == 0 and j < skip_chunks:
                        continue
                    self.chunk_index = j
                    if j == n_chunks - 1:
                        self.docs_seen += 1
                        self.percent_seen = self.docs_seen * 100 / (ndocs + 1e-9)
                        self.chunk_index = -1
                        self.completed_current_doc = True
                    yield self._chunk(j, doc, n_chunks)
            # the chunks skipped at the start belong to this epoch too: replay them last
            if not self.raw_data_mode and skip_chunks and first_slot is not None:
                self.docset_index, self.lcg_state = start_index, start_lcg
                path, size, first_row = self._locate(start_index)
                doc, n_chunks = self._tokens_of(path, first_slot + first_row)
                if doc is not None:
                    for j in range(min(skip_chunks, n_chunks)):
                        self.chunk_index = j
                        yield self._chunk(j, doc, n_chunks)

    def load_state_dict(self, state_dicts, sharded_input: bool = False):
        assert self.load_worldsize == self.worldsize, (
            f"ParquetDataset does not support rescaling: from {self.load_worldsize} to {self.worldsize}")
        return super().load_state_dict(state_dicts, sharded_input)


class Sampling_Dataset(_Stateful_Dataset):
    """Mixes several sources by token share: always draws from the source furthest below its target
    weight and keeps drawing from it until the current document ends (delimiter seen)."""

    def __init__(self, datasets: List[_Stateful_Dataset], weights: Optional[List[float]], delimiter_token: Any,
                 rank: int = 0, worldsize: int = 1, verbose: bool = False):
        super().__init__(rank, worldsize)
        assert datasets, "need at least one dataset"
        self.data = datasets
        w = [1.0] * len(datasets) if not weights else [float(x) for x in weights]
        assert len(w) == len(datasets) and all(x > 0 for x in w)
        self.weights = [x / sum(w) for x in w]
        self.delimiter, self.verbose = delimiter_token, verbose
        self.tokens_seen = [0] * len(datasets)
        self.current_iterator = -1
        self.state_params = ["tokens_seen", "current_iterator"]

    def __iter__(self):
        its = [iter(d) for d in self.data]
        while True:
            if self.current_iterator != -1:
                out = next(its[self.current_iterator])
                self.tokens_seen[self.current_iterator] += len(out)
                if out[-1] == self.delimiter:
                    self.current_iterator = -1
                yield out
            else:
                total = sum(self.tokens_seen) + 1e-9
                deficit = [self.weights[i] - self.tokens_seen[i] / total for i in range(len(self.data))]
                # among equally starved sources the LAST one wins, as in the reference (a max over (deficit, index)
                # pairs, maester/datasets/experimental_otf.py:1352-1358): same stream from the first document on
                self.current_iterator = max((x, i) for i, x in enumerate(deficit))[1]

    def state_dict(self) -> dict:
        """The sources' states as a list under ``sample_iterator_states``, in the order of the sources: the layout of
        the reference's loader checkpoints (maester/datasets/experimental_otf.py:1360-1369)."""
        out = {self.statename("sample_iterator_states"): [d.state_dict() for d in self.data]}
        out.update(super().state_dict())
        return out

    def load_state_dict(self, state_dicts, sharded_input: bool = False):
        sharded = super().load_state_dict(state_dicts, sharded_input)
        key = self.statename("sample_iterator_states")
        for i, d in enumerate(self.data):
            d.load_worldsize = self.load_worldsize
            d.load_state_dict([sd[key][i] for sd in sharded], True)
        return sharded


class Scalable_Shard_Dataset(_Stateful_Dataset):
    """Many logical shards per worker so that a checkpoint can be reloaded on a different world
    size: the logical shards (and their states) are re-partitioned over the new workers.  At every
    step one logical shard is drawn with probability proportional to its remaining documents."""

    def __init__(self, make_shard: Callable[[int, int], _Stateful_Dataset], rank: int, worldsize: int,
                 delimiter_token: Any, n_logical_shards: int = 2048, seed: int = 42):
        super().__init__(rank, worldsize)
        assert n_logical_shards % worldsize == 0, "logical shards must divide evenly over workers"
        self.total_shards, self.delimiter = n_logical_shards, delimiter_token
        mine = _shard_partition(list(range(n_logical_shards)), rank, worldsize)
        self.data = [make_shard(i, n_logical_shards) for i in mine]
        self.n_docs_remaining = [len(d) if hasattr(d, "__len__") else getattr(d, "_len", 1) for d in self.data]
        self.generator = torch.Generator().manual_seed(seed + rank)
        self.g_state = None
        self.current_reader = None
        self.logical_shard_states: List[dict] = []
        self.state_params = ["current_reader", "g_state"]
        self.reshard_params = ["n_docs_remaining", "logical_shard_states"]

    def __iter__(self):
        its = [iter(d) for d in self.data]
        while True:
            if self.current_reader is not None:
                out = next(its[self.current_reader])
                if out[-1] == self.delimiter:
                    self.n_docs_remaining[self.current_reader] -= 1
                    if sum(self.n_docs_remaining) == 0:
                        self.n_docs_remaining = [getattr(d, "_len", 1) for d in self.data]
                        self.generator.manual_seed(self.generator.initial_seed() + 1)
                    self.current_reader = None
                yield out
            else:
                w = torch.tensor(self.n_docs_remaining, dtype=torch.float)
                self.current_reader = torch.multinomial(w, 1, generator=self.generator).item()

    def state_dict(self) -> dict:
        self.g_state = self.generator.get_state()
        self.logical_shard_states = [d.state_dict() for d in self.data]
        return super().state_dict()

    def load_state_dict(self, state_dicts, sharded_input: bool = False):
        sharded = super().load_state_dict(state_dicts, sharded_input)
        if self.g_state is not None and self.load_worldsize == self.worldsize:
            self.generator.set_state(self.g_state)
        for d, st in zip(self.data, self.logical_shard_states):
            d.load_worldsize = 1
            d.load_state_dict([st], True)
        return sharded
