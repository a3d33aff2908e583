"""On-the-fly tokenising, resumable, rank-sharded Parquet data pipeline (CPU, Python by design).

Pipeline built by ``build_experimental_data_loader`` (reference:
maester/datasets/experimental_otf.py:1519-1603):

    ParquetDataset (per source) → Sampling_Dataset → Buffer_Dataset(seq_len + 1, hard packing)
      → Preload_Buffer_Dataset(10 000-line shuffle) → Preprocess_Dataset(causal_lm)
      → Checkpoint_Dataset → torch DataLoader (1 worker, pinned memory)

Every layer is a ``_Stateful_Dataset``: ``state_params`` are scalars that are dropped when the world
size changes, ``reshard_params`` are lists that are re-partitioned; ``state_dict`` /
``load_state_dict`` recurse through wrappers, ``save_to_path`` writes
``loader_state_{rank}.pth``.  ``ParquetDataset`` shuffles documents inside a file range with an LCG
bijection (no materialised index lists), chunks documents to ``max_chunksize`` with BOS on the first
and EOS on the last chunk, and resumes mid-document: chunks skipped on resume are replayed at the
end of the epoch so that an epoch always contains every chunk exactly once.
"""
from __future__ import annotations

import math
import os
import time
from typing import Any, Callable, List

import torch
import torch.distributed as dist
import torch.utils.data as data

from maester_b200.log_utils import logger


# --------------------------------------------------------------------------- helpers
def _get_latest(targdir: str, qualifier=lambda x: True):
    """Newest ``<name>-<N>`` entry of a directory (largest N) that passes ``qualifier``; None if none."""
    if not os.path.isdir(targdir):
        return None
    cands = [os.path.join(targdir, x) for x in os.listdir(targdir)]
    cands = [c for c in cands if qualifier(c)]
    if not cands:
        return None
    return max(cands, key=lambda p: int(os.path.basename(p).split("-")[1]))


def _shard_partition(items: List[Any], rank: int, worldsize: int) -> List[Any]:
    return items[(rank * len(items)) // worldsize:((rank + 1) * len(items)) // worldsize]


def _shard_inclusive(items: List[Any], rank: int, worldsize: int) -> List[Any]:
    """Span of items owned by ``rank`` when ownership may be fractional."""
    start = math.floor(len(items) * rank / worldsize)
    end = math.ceil(len(items) * (rank + 1) / worldsize)
    return items[start:end]


def _dist_rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _dist_barrier() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


# --------------------------------------------------------------------------- stateful base classes
class _Stateful_Dataset(data.IterableDataset):
    def __init__(self, rank: int, worldsize: int):
        assert rank >= 0 and worldsize > rank, f"bad rank/worldsize {rank}/{worldsize}"
        self.state_params: List[str] = []
        self.reshard_params: List[str] = []
        self.rank, self.worldsize = rank, worldsize
        self.load_worldsize = worldsize

    def statename(self, x: str) -> str:
        return f"{self.__class__.__name__}.{x}"

    def state_dict(self) -> dict:
        return {self.statename(f): getattr(self, f) for f in self.state_params + self.reshard_params}

    def _reshard(self, sharded_list):
        """Flatten the inclusive span of equally long shard lists and pick the items this rank owns."""
        shard_offset = math.floor(self.load_worldsize * self.rank / self.worldsize)
        shard_len = len(sharded_list[0])
        assert all(len(s) == shard_len for s in sharded_list), "shards must have equal length"
        item_offset = shard_len * shard_offset
        n_items = self.load_worldsize * shard_len
        mine = range(int(n_items * self.rank / self.worldsize) - item_offset,
                     int(n_items * (self.rank + 1) / self.worldsize) - item_offset)
        return [sharded_list[i // shard_len][i % shard_len] for i in mine]

    def load_state_dict(self, state_dicts, sharded_input: bool = False):
        if not sharded_input:
            self.load_worldsize = len(state_dicts)
            state_dicts = _shard_inclusive(state_dicts, self.rank, self.worldsize)
        if self.load_worldsize == self.worldsize:
            for f in self.state_params + self.reshard_params:
                setattr(self, f, state_dicts[0][self.statename(f)])
        else:
            for f in self.reshard_params:
                setattr(self, f, self._reshard([sd[self.statename(f)] for sd in state_dicts]))
        return state_dicts

    def load_from_path(self, path: str) -> None:
        assert os.path.isdir(path), "checkpoint must be a folder of loader_state_*.pth shards"
        shards = sorted((x for x in os.listdir(path) if "loader" in x), key=lambda x: int(x.split("_")[2][:-4]))
        assert shards, "no loader state files found"
        self.load_worldsize = len(shards)
        mine = _shard_inclusive(shards, self.rank, self.worldsize)
        self.load_state_dict([torch.load(os.path.join(path, x), weights_only=False) for x in mine], True)

    def save_to_path(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        torch.save(self.state_dict(), os.path.join(path, f"loader_state_{self.rank}.pth"))


class _Wrapper_Dataset(_Stateful_Dataset):
    """A stateful layer around another stateful dataset; state calls recurse."""

    def __init__(self, dataset: _Stateful_Dataset):
        self.dataset = dataset
        super().__init__(dataset.rank, dataset.worldsize)

    def load_state_dict(self, state_dicts, sharded_input: bool = False):
        sharded = super().load_state_dict(state_dicts, sharded_input)
        self.dataset.load_worldsize = self.load_worldsize
        self.dataset.load_state_dict(sharded, True)
        return sharded

    def state_dict(self) -> dict:
        out = self.dataset.state_dict()
        out.update(super().state_dict())
        return out


# --------------------------------------------------------------------------- simple layers
class Preprocess_Dataset(_Wrapper_Dataset):
    """Applies a stateless function to every item."""

    def __init__(self, dataset: _Stateful_Dataset, aug_fn: Callable):
        super().__init__(dataset)
        self.aug_fn = aug_fn

    def __iter__(self):
        for item in iter(self.dataset):
            yield self.aug_fn(item)


def causal_lm(line, prompt_len: int = 0):
    """seq_len+1 tokens → ``{"input_ids": x[:-1], "labels": x[1:]}`` (labels of the prompt masked)."""
    t = torch.as_tensor(line, dtype=torch.long)
    labels = t[1:].clone()
    if prompt_len:
        labels[:prompt_len] = -100
    return {"input_ids": t[:-1], "labels": labels}


class Checkpoint_Dataset(_Wrapper_Dataset):
    """Saves the whole pipeline's state every ``interval`` optimizer steps from inside the DataLoader
    worker and auto-loads the newest state on construction.  ``steps_per_batch`` converts yielded
    items to optimizer steps (micro-batch size x accumulation steps).  Because the DataLoader
    prefetches, the saved state runs ahead of consumption by the prefetch depth."""

    def __init__(self, dataset: _Stateful_Dataset, load_path: str, interval: int, steps_per_batch: int = 1,
                 save_path: str = "", load_step: int | None = None):
        """``load_step``: the optimizer step of the model checkpoint that the job resumes from.  ``None`` loads the
        NEWEST loader state, as the reference does (maester/datasets/experimental_otf.py:354-381).  That one can be
        ahead of the newest model checkpoint: the worker process saves on its own count of yielded batches, and the
        DataLoader lets it run ahead of the training loop by the prefetch depth, so a job that stopped after the
        loader wrote ``step-12`` but before the model reached it would skip the batches in between.  With a step
        given, exactly ``step-<load_step>`` is loaded (an error if it is missing), and 0 starts from scratch whatever
        states lie around."""
        super().__init__(dataset)
        self.interval, self.spb = interval, steps_per_batch
        self.save_path = save_path or load_path
        self.path = self.save_path
        self.step = 0
        self.ministep = 0
        if load_step is None:
            self.load_from_path(load_path)
        elif load_step > 0:
            exact = os.path.join(self.path, f"step-{load_step}")
            if not (os.path.isdir(exact) and any("loader" in x for x in os.listdir(exact))):
                raise RuntimeError(f"the model resumes from step {load_step} but {exact} holds no loader state: "
                                   "the job would train on the wrong part of the stream")
            self.dataset.load_from_path(exact)
            self.step = load_step
            self._report(f"Dataset checkpoint loaded from {exact}, the step of the model checkpoint")
        else:
            self._report("Data pipeline starts from scratch (the model does)")

    def setup(self) -> None:
        pass

    def __iter__(self):
        self.setup()
        it = iter(self.dataset)
        while True:
            for _ in range(self.interval * self.spb):
                yield next(it)
                self.ministep += 1
                if self.ministep == self.spb:
                    self.ministep = 0
                    self.step += 1
            newpath = os.path.join(self.path, f"step-{self.step}")
            start = time.time()
            self.dataset.save_to_path(newpath)
            self._report(f"Saved dataloader checkpoint to {newpath} in {time.time() - start:.2f}s")

    def _report(self, msg: str) -> None:
        if self.rank == 0:
            logger.info(msg)

    def _validate_ckp_path(self, path: str, verbose: bool = False) -> str:
        """Resolve a checkpoint folder: either it holds loader shards itself or ``step-N`` subfolders."""
        if not os.path.isdir(path) or not os.listdir(path):
            return ""
        if any("loader" in x for x in os.listdir(path)):
            return path
        latest = _get_latest(path, lambda p: os.path.isdir(p) and os.path.basename(p).startswith("step-"))
        if latest is None or not any("loader" in x for x in os.listdir(latest)):
            return ""
        return latest

    def load_from_path(self, path: str) -> None:
        save_latest = self._validate_ckp_path(self.path)
        if save_latest:
            path = save_latest  # a run that already saved states resumes from its own newest one
        else:
            path = self._validate_ckp_path(path)
        if not path:
            self._report("No valid dataloader checkpoint detected: starting from scratch")
            return
        start = time.time()
        self.dataset.load_from_path(path)
        self.step = int(os.path.basename(path).split("-")[1]) if "step-" in os.path.basename(path) else 0
        self._report(f"Dataset checkpoint loaded from {path} (step {self.step}) in {time.time() - start:.2f}s")


class Preload_Buffer_Dataset(_Wrapper_Dataset):
    """Shuffle buffer with one in/out slot array (reference: maester/datasets/experimental_otf.py:383-452).  Every step
    yields a random slot and refills it; while the buffer is below ``window_size`` a step also appends one item first,
    so the buffer grows by one per yielded item (two reads per step) and output starts with the very first step instead
    of after ``window_size`` reads.  The random draws are the same as the reference's, so is the stream."""

    def __init__(self, dataset: _Stateful_Dataset, window_size: int):
        super().__init__(dataset)
        assert window_size > 1
        self.window_size = window_size
        self.g_state = None
        self.generator = torch.Generator().manual_seed(self.rank)
        self.buffer: List[Any] = []
        self.buffer_size = 0
        self.state_params = ["g_state"]
        self.reshard_params = ["buffer"]

    def __iter__(self):
        it = iter(self.dataset)
        while True:
            self._pad_buffer()
            if self.buffer_size < self.window_size:
                self.buffer[self.buffer_size] = next(it)
                self.buffer_size += 1
            i = torch.randint(self.buffer_size, (1,), generator=self.generator).item()
            out = self.buffer[i]
            self.buffer[i] = next(it)
            yield out

    def _pad_buffer(self) -> None:
        if len(self.buffer) < self.window_size:
            self.buffer += [[]] * (self.window_size - len(self.buffer))

    def state_dict(self) -> dict:
        self.g_state = self.generator.get_state()
        self.buffer = self.buffer[: self.buffer_size]  # drop padding before saving
        out = super().state_dict()
        out[self.statename("buffer")] = list(self.buffer)  # snapshot: the live list keeps changing
        return out

    def load_state_dict(self, state_dicts, sharded_input: bool = False):
        sharded = super().load_state_dict(state_dicts, sharded_input)
        if self.g_state is not None:
            self.generator.set_state(self.g_state)
        self.buffer = [b for b in self.buffer if len(b) > 0]
        self.buffer_size = len(self.buffer)
        return sharded


class Buffer_Dataset(_Wrapper_Dataset):
    """Packs variable-length chunks into fixed ``seq_len`` lines.  ``pack_hard=True`` splits chunks
    across lines; otherwise a chunk that does not fit starts a new line and the old one is padded."""

    def __init__(self, dataset: _Stateful_Dataset, seq_len: int, pack_hard: bool, bos_token=None, eos_token=None,
                 pad_token=None):
        super().__init__(dataset)
        self.len, self.pack_hard = seq_len, pack_hard
        self.bos, self.eos, self.pad = bos_token, eos_token, pad_token
        if not pack_hard:
            assert pad_token is not None, "soft packing needs a pad token"
        self.buffer: List[Any] = []
        self.state_params = ["buffer"]

    def __iter__(self):
        it = iter(self.dataset)
        length = self.len - int(self.bos is not None) - int(self.eos is not None)
        while True:
            line: List[Any] = list(self.buffer)  # tokens carried over from the previous line
            self.buffer = []
            if len(line) > length:
                line, self.buffer = line[:length], line[length:]
            while len(line) < length:
                chunk = next(it)
                room = length - len(line)
                if len(chunk) <= room:
                    line += chunk
                elif self.pack_hard:
                    line += chunk[:room]
                    self.buffer = chunk[room:]
                else:  # soft packing: close this line with padding, the chunk opens the next one
                    self.buffer = chunk[:length]
                    line += [self.pad] * room
            if self.bos is not None:
                line = [self.bos] + line
            if self.eos is not None:
                line = line + [self.eos]
            yield line


def __getattr__(name: str):
    """Document sources and the loader builder live in sibling modules; they are reachable from
    here under the names the reference module exposes."""
    if name in {"ParquetDataset", "Sampling_Dataset", "Scalable_Shard_Dataset"}:
        from maester_b200.datasets import parquet_dataset
        return getattr(parquet_dataset, name)
    if name in {"build_experimental_data_loader", "parse_data_args"}:
        from maester_b200.datasets import builder
        return getattr(builder, name)
    raise AttributeError(name)
