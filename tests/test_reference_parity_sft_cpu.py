"""Supervised fine-tuning data against the reference's own classes (installed copy of the reference package,
maester/sft/dataset.py and maester/sft/packed_dataset.py): the same conversations give the same padded samples and
label masks in the same order, and a packed file written by this repository's packer is read by the reference's
``PackedSFTDataset`` into the same tensors (position and document ids included) in the same per-epoch order."""
import json
import os
import sys

import numpy as np
import pyarrow as pa
import pyarrow.parquet as pq
import pytest
import torch

from test_parallel_cpu import run_ranks
from test_sft import CharTokenizer

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "maester")), reason="the reference is not installed")


def _sft(rank, world, tmp):
    sys.path.insert(0, os.path.join(ROOT, "baseline", "shims"))
    sys.path.insert(0, REF)
    sys.path.insert(0, os.path.join(ROOT, "scripts"))
    import maester.models  # noqa: F401  (first, or the reference's packages import each other in a circle)
    from maester.sft.dataset import ConversationParquetDataset as RefConversations
    from maester.sft.packed_dataset import PackedSFTDataset as RefPacked
    from maester_b200.sft import ConversationParquetDataset, PackedSFTDataset, packed_collate_fn
    import pack_sft_data as P

    g = torch.Generator().manual_seed(0)
    rnd = lambda lo, hi: int(torch.randint(lo, hi, (1,), generator=g))
    convs = []
    for i in range(60):
        turns = [{"role": ["system", "user", "assistant"][rnd(0, 3)], "content": "x" * rnd(0, 30) + str(i)}
                 for _ in range(rnd(1, 6))]
        convs.append(json.dumps(turns))
    os.makedirs(os.path.join(tmp, "conv"))
    pq.write_table(pa.table({"messages": convs}), os.path.join(tmp, "conv", "c.parquet"), row_group_size=7)
    tok = CharTokenizer()
    for r, w in [(0, 1), (1, 2)]:
        for strategy in ("assistant_only", "all"):
            ref = RefConversations(os.path.join(tmp, "conv"), r, w, tok, template="chatml", mask_strategy=strategy,
                                   max_seq_len=48, conversation_column="messages")
            ref.im_start, ref.im_end = "<<", ">>"   # the reference's loader builder sets them after construction
            ours = ConversationParquetDataset(os.path.join(tmp, "conv"), r, w, tok, 48, template="chatml",
                                              mask_strategy=strategy, conversation_column="messages",
                                              im_start="<<", im_end=">>")
            ri, oi = iter(ref), iter(ours)
            truncated = 0
            for n in range(150):   # more than two passes over the shard
                a, b = next(ri), next(oi)
                assert sorted(a) == sorted(b)
                for k in a:
                    assert list(a[k]) == b[k].tolist(), (strategy, r, w, n, k)
                truncated += int(sum(a["attention_mask"]) == 48)
            assert truncated > 0   # the truncation path was compared too

    # packed data: written by this repository's packer, read by both
    lengths = np.random.default_rng(0).integers(5, 120, size=200)
    samples = [(list(range(10, 10 + n)), [-100] * (n // 2) + list(range(n - n // 2))) for n in lengths]
    rows = P.materialise(P.plan_packs(np.array(lengths), 256, 4, 20), samples, 256, pad_id=0)
    path = os.path.join(tmp, "packed.parquet")
    pq.write_table(pa.table(dict(rows)), path)
    for r, w in [(0, 1), (1, 3)]:
        ref, ours = RefPacked(path, rank=r, world_size=w, seed=5), PackedSFTDataset(path, rank=r, world_size=w, seed=5)
        assert ref.num_samples == ours.num_samples
        for n in range(2 * ref.num_samples + 3):   # into the third epoch: the per-epoch reshuffles agree
            a, b = ref[0], ours[0]
            assert sorted(a) == sorted(b)
            for k in a:
                assert a[k].dtype == b[k].dtype and torch.equal(a[k], b[k]), (r, w, n, k)
        batch = packed_collate_fn([ours[0], ours[0]])
        assert sorted(batch) == ["attention_mask", "document_ids", "input_ids", "labels", "position_ids", "stats"]
    return True


def test_sft_data_is_the_reference_data(tmp_path):
    assert run_ranks(1, _sft, str(tmp_path)) == [True]
