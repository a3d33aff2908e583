"""Stateful data pipeline: partitioning, packing, shuffle buffer, resume determinism (CPU only).

Follows the ideas of the reference tests (tests/test_datasets.py, tests/test_experimental_otf*.py):
per-rank objects stand in for ranks; a toy tokenizer replaces a downloaded one.
"""
import os

import pyarrow as pa
import pyarrow.parquet as pq
import pytest
import torch

from maester_b200.datasets import (Buffer_Dataset, Checkpoint_Dataset, ParquetDataset, Preload_Buffer_Dataset,
                                   Preprocess_Dataset, Sampling_Dataset, causal_lm, parse_data_args)
from maester_b200.datasets.experimental_otf import _shard_inclusive, _shard_partition, _Stateful_Dataset


class ToyTokenizer:
    """Words are 'w<number>'; the token id is the number."""

    def encode(self, text, add_special_tokens=False, padding=False, truncation=False):
        return [int(w[1:]) for w in text.split()]


def make_corpus(path, n_files=2, docs_per_file=40, seed=0):
    g = torch.Generator().manual_seed(seed)
    os.makedirs(path, exist_ok=True)
    doc_id = 0
    for f in range(n_files):
        texts = []
        for _ in range(docs_per_file):
            n = int(torch.randint(3, 120, (1,), generator=g))
            # first token encodes the document id (+1000) so coverage can be checked
            texts.append(" ".join([f"w{1000 + doc_id}"] + [f"w{int(t)}" for t in torch.randint(10, 900, (n,), generator=g)]))
            doc_id += 1
        pq.write_table(pa.table({"text": texts}), os.path.join(path, f"part{f}.parquet"), row_group_size=7)
    return doc_id


def take(it, n):
    return [next(it) for _ in range(n)]


def test_shard_helpers():
    items = list(range(10))
    parts = [_shard_partition(items, r, 3) for r in range(3)]
    assert sum(parts, []) == items
    assert _shard_inclusive(items, 1, 4) == [2, 3, 4]
    assert parse_data_args("a,b", "1,3") == (["a", "b"], [1.0, 3.0])


def test_ranks_cover_every_document_once(tmp_path):
    n_docs = make_corpus(tmp_path / "d")
    seen = []
    for rank in range(3):
        ds = ParquetDataset(str(tmp_path / "d"), rank, 3, ToyTokenizer(), delimiter_token=1, max_chunksize=10_000)
        it = iter(ds)
        for _ in range(ds._len):
            seen.append(next(it)[0] - 1000)
    assert sorted(seen) == list(range(n_docs))


def test_chunking_bos_eos(tmp_path):
    make_corpus(tmp_path / "d", n_files=1, docs_per_file=6)
    ds = ParquetDataset(str(tmp_path / "d"), 0, 1, ToyTokenizer(), delimiter_token=1, bos_token=2, max_chunksize=16)
    it = iter(ds)
    doc_tokens = []
    while True:
        c = next(it)
        assert len(c) <= 17  # the last chunk may carry EOS on top of the chunk size
        first = not doc_tokens
        if first:
            assert c[0] == 2
        doc_tokens += c
        if c[-1] == 1:
            break
    assert doc_tokens.count(2) == 1 and doc_tokens[-1] == 1


@pytest.mark.parametrize("stop_after", [1, 7, 23])
def test_resume_continues_identically(tmp_path, stop_after):
    make_corpus(tmp_path / "d")
    mk = lambda: ParquetDataset(str(tmp_path / "d"), 1, 2, ToyTokenizer(), delimiter_token=1, max_chunksize=20)
    ref = take(iter(mk()), 120)
    a = mk()
    it = iter(a)
    got = take(it, stop_after)
    state = a.state_dict()
    b = mk()
    b.load_state_dict([state], sharded_input=True)
    got += take(iter(b), 120 - stop_after)
    assert got == ref
    assert set(state) >= {"ParquetDataset.docset_index", "ParquetDataset.chunk_index", "ParquetDataset.lcg_state",
                          "ParquetDataset.completed_current_doc"}


def test_epoch_contains_each_chunk_once_after_mid_document_resume(tmp_path):
    make_corpus(tmp_path / "d", n_files=1, docs_per_file=12)
    mk = lambda: ParquetDataset(str(tmp_path / "d"), 0, 1, ToyTokenizer(), delimiter_token=1, max_chunksize=8)
    full = mk()
    it = iter(full)
    epoch = []
    while full.epochs_seen < 1:
        epoch.append(tuple(next(it)))
        if full.epochs_seen >= 1:
            epoch.pop()
    n_chunks = len(epoch)
    a = mk()
    ita = iter(a)
    first = [tuple(c) for c in take(ita, 2)]
    assert a.chunk_index >= 0  # stopped inside a document
    b = mk()
    b.load_state_dict([a.state_dict()], sharded_input=True)
    rest = [tuple(c) for c in take(iter(b), n_chunks)]
    assert sorted(first + rest[: n_chunks - 2]) == sorted(epoch)


def test_buffer_dataset_packs_fixed_lines(tmp_path):
    make_corpus(tmp_path / "d")
    src = ParquetDataset(str(tmp_path / "d"), 0, 1, ToyTokenizer(), delimiter_token=1, max_chunksize=50)
    flat = []
    it = iter(ParquetDataset(str(tmp_path / "d"), 0, 1, ToyTokenizer(), delimiter_token=1, max_chunksize=50))
    while len(flat) < 33 * 20:
        flat += next(it)
    lines = take(iter(Buffer_Dataset(src, 33, pack_hard=True)), 20)
    assert all(len(l) == 33 for l in lines)
    assert sum(lines, []) == flat[: 33 * 20]
    soft = take(iter(Buffer_Dataset(ParquetDataset(str(tmp_path / "d"), 0, 1, ToyTokenizer(), delimiter_token=1,
                                                    max_chunksize=20), 33, pack_hard=False, pad_token=0)), 10)
    assert all(len(l) == 33 for l in soft) and any(0 in l for l in soft)


class Counter(_Stateful_Dataset):
    def __init__(self, rank=0, worldsize=1):
        super().__init__(rank, worldsize)
        self.i = 0
        self.state_params = ["i"]

    def __iter__(self):
        while True:
            self.i += 1
            yield [self.i]


def test_preload_buffer_shuffles_and_resumes():
    ds = Preload_Buffer_Dataset(Counter(), 50)
    it = iter(ds)
    first = [x[0] for x in take(it, 400)]
    assert first != sorted(first) and len(set(first)) == 400
    state = ds.state_dict()
    cont = [x[0] for x in take(it, 100)]
    ds2 = Preload_Buffer_Dataset(Counter(), 50)
    ds2.load_state_dict([state], sharded_input=True)
    assert [x[0] for x in take(iter(ds2), 100)] == cont


def test_sampling_dataset_respects_weights(tmp_path):
    make_corpus(tmp_path / "a", seed=1)
    make_corpus(tmp_path / "b", seed=2)
    mk = lambda p: ParquetDataset(str(tmp_path / p), 0, 1, ToyTokenizer(), delimiter_token=1, max_chunksize=64)
    ds = Sampling_Dataset([mk("a"), mk("b")], [3, 1], delimiter_token=1)
    take(iter(ds), 600)
    share = ds.tokens_seen[0] / sum(ds.tokens_seen)
    assert 0.68 < share < 0.82


def test_checkpoint_dataset_saves_and_autoloads(tmp_path):
    make_corpus(tmp_path / "d")
    ck = str(tmp_path / "ckpt")

    def pipeline():
        src = ParquetDataset(str(tmp_path / "d"), 0, 1, ToyTokenizer(), delimiter_token=1, max_chunksize=40)
        ds = Preprocess_Dataset(Buffer_Dataset(src, 17, pack_hard=True), causal_lm)
        return Checkpoint_Dataset(ds, ck, interval=5, steps_per_batch=2, save_path=ck)

    a = pipeline()
    it = iter(a)
    items = take(it, 25)              # 25 items = 12 optimizer steps -> saves at step 5 and 10
    assert sorted(os.listdir(ck)) == ["step-10", "step-5"]
    assert items[0]["input_ids"].shape == (16,) and torch.equal(items[0]["input_ids"][1:], items[0]["labels"][:-1])
    b = pipeline()                    # auto-loads step-10 = state after 20 items
    assert b.step == 10
    resumed = take(iter(b), 5)
    for x, y in zip(resumed, items[20:]):
        assert torch.equal(x["input_ids"], y["input_ids"])


def test_loader_state_of_a_given_step_is_loaded_not_the_newest(tmp_path):
    """The worker saves ahead of the training loop (prefetch); a job resumes from the state of the MODEL's step."""
    make_corpus(tmp_path / "d")

    def pipeline(load_step):
        src = ParquetDataset(str(tmp_path / "d"), 0, 1, ToyTokenizer(), delimiter_token=1, max_chunksize=32)
        ds = Preload_Buffer_Dataset(Buffer_Dataset(Sampling_Dataset([src], None, delimiter_token=1), 17, pack_hard=True), 20)
        return Checkpoint_Dataset(ds, str(tmp_path / "ck"), 3, steps_per_batch=2, save_path=str(tmp_path / "ck"),
                                  load_step=load_step)

    first = pipeline(0)
    lines = take(iter(first), 2 * 9 + 1)                 # 9 steps of 2 lines each: states step-3, step-6, step-9 exist
    assert sorted(os.listdir(tmp_path / "ck")) == ["step-3", "step-6", "step-9"]
    assert take(iter(pipeline(None)), 1)[0] == lines[18]  # the newest state (the reference's choice): line after step 9
    resumed = pipeline(3)                                 # the model checkpoint is at step 3
    assert resumed.step == 3
    assert take(iter(resumed), 6) == lines[6:12]
    assert take(iter(pipeline(0)), 4) == lines[:4]        # no model checkpoint: from scratch despite stale states
    with pytest.raises(RuntimeError, match="holds no loader state"):
        pipeline(4)
