"""SFT data: ChatML masking, packed-sample position/document ids, the packer (CPU only)."""
import json
import os
import sys

import numpy as np
import pyarrow as pa
import pyarrow.parquet as pq
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "scripts"))

from maester_b200.sft import ConversationParquetDataset, PackedSFTDataset, mask_labels, packed_collate_fn, tokenize_conversation  # noqa: E402
from maester_b200.sft.packed_dataset import document_ids_from_boundaries, position_ids_from_boundaries  # noqa: E402


class CharTokenizer:
    """One token per character; '<' and '>' style markers are plain characters."""
    bos_token_id, eos_token_id, pad_token_id = 1, 2, 0

    def encode(self, text, add_special_tokens=False, **kw):
        return [ord(c) + 3 for c in text]

    def decode(self, ids):
        return "".join(chr(i - 3) for i in ids if i > 2)


CONV = [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo!"}, {"role": "user", "content": "k"}]


def test_assistant_only_masking_trains_exactly_the_assistant_turn():
    tok = CharTokenizer()
    tokens, spans = tokenize_conversation(CONV, tok, "chatml", "<<", ">>")
    assert tokens[0] == 1 and tokens[-1] == 2 and [r for _, _, r in spans] == ["user", "assistant", "user"]
    labels = mask_labels(tokens, spans, "assistant_only")
    kept = [t for t in labels if t != -100]
    assert tok.decode(kept) == "<<assistant\nyo!>>\n"
    assert all(l == -100 or l == t for l, t in zip(labels, tokens[1:]))
    all_labels = mask_labels(tokens, spans, "all")
    assert sum(l != -100 for l in all_labels) == len(tokens) - 2  # everything but EOS (outside any span)


def test_conversation_dataset_pads_and_shards(tmp_path):
    convs = [json.dumps([{"role": "user", "content": f"q{i}"}, {"role": "assistant", "content": "a" * (i % 7 + 1)}])
             for i in range(30)]
    pq.write_table(pa.table({"conversations": convs}), tmp_path / "c.parquet")
    seen = []
    for rank in range(2):
        ds = ConversationParquetDataset(str(tmp_path), rank, 2, CharTokenizer(), 64, im_start="<<", im_end=">>")
        it = iter(ds)
        for _ in range(15):
            item = next(it)
            assert item["input_ids"].shape == (64,) and item["labels"].shape == (64,)
            n = int(item["attention_mask"].sum())
            assert (item["labels"][n:] == -100).all() and (item["input_ids"][n:] == 0).all()
            seen.append(CharTokenizer().decode(item["input_ids"][:n].tolist()))
    assert len(set(seen)) == 30  # the two ranks saw disjoint conversations


def test_boundaries_to_position_and_document_ids():
    b = [(7, 0, 3), (9, 3, 4)]
    assert position_ids_from_boundaries(b, 10).tolist() == [0, 1, 2, 0, 1, 2, 3, 0, 0, 0]
    assert document_ids_from_boundaries(b, 10).tolist() == [0, 0, 0, 1, 1, 1, 1, -1, -1, -1]


def test_packer_and_packed_dataset(tmp_path):
    import pack_sft_data as P
    rng = np.random.default_rng(0)
    lengths = rng.integers(5, 120, size=300)
    convs = [(list(range(10, 10 + n)), [-100] * (n // 2) + list(range(n - n // 2))) for n in lengths]
    packs = P.plan_packs(np.array(lengths), 256, 4, 20)
    used = sorted(i for p in packs for i in p)
    assert used == list(range(300))                       # every conversation packed exactly once
    assert all(sum(lengths[i] for i in p) <= 256 for p in packs)
    eff = lengths.sum() / (len(packs) * 256)
    assert eff > 0.8
    rows = P.materialise(packs, convs, 256, pad_id=0)
    pq.write_table(pa.table(dict(rows)), tmp_path / "packed.parquet")
    ds = PackedSFTDataset(str(tmp_path / "packed.parquet"), rank=0, world_size=2, seed=1)
    other = PackedSFTDataset(str(tmp_path / "packed.parquet"), rank=1, world_size=2, seed=1)
    assert set(ds.rank_indices).isdisjoint(other.rank_indices)
    s = ds[0]
    assert s["input_ids"].shape == (256,) and s["document_ids"].max() >= 0
    n = int(s["attention_mask"].sum())
    assert (s["document_ids"][n:] == -1).all()
    starts = (s["position_ids"][:n] == 0).nonzero().flatten()
    assert len(starts) == int(s["document_ids"].max()) + 1  # positions restart once per conversation
    batch = packed_collate_fn([ds[0], ds[0]])
    assert batch["stats"]["actual_lengths"].shape == (2,) and batch["document_ids"].shape == (2, 256)
    state = ds.state_dict()
    nxt = ds[0]["input_ids"]
    ds2 = PackedSFTDataset(str(tmp_path / "packed.parquet"), rank=0, world_size=2, seed=1)
    ds2.load_state_dict(state)
    assert torch.equal(ds2[0]["input_ids"], nxt)
