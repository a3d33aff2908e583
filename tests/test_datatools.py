"""Offline data tools and the legacy Arrow loader."""
import gzip
import json
import subprocess
import sys

import pyarrow as pa
import pyarrow.parquet as pq
import pytest
import torch

from maester_b200.datatools.ingest import conversations_to_parquet, jsonl_to_parquet, normalise_messages, tokenize_to_arrow
from maester_b200.datatools.inspect import inspect_packed_data, inspect_parquet, random_dataset_sample
from maester_b200.datatools.shuffle import shuffle_split
from maester_b200.datatools.stats import count_tokens, estimate_tokens


class WordTokenizer:
    eos_token_id = 1

    def __call__(self, texts, **kw):
        return {"input_ids": [[2 + (hash(w) % 1000) for w in t.split()] for t in texts]}

    def encode(self, text, **kw):
        return self([text])["input_ids"][0]

    def decode(self, ids):
        return " ".join(f"w{i}" for i in ids)


def _corpus(tmp_path, n=300):
    src = tmp_path / "raw"
    src.mkdir()
    with gzip.open(src / "a.jsonl.gz", "wt") as f:
        for i in range(n // 2):
            f.write(json.dumps({"text": " ".join(["tok"] * (1 + i % 17)), "id": i}) + "\n")
    with open(src / "b.jsonl", "w") as f:
        for i in range(n // 2, n):
            f.write(json.dumps({"text": " ".join(["tok"] * (1 + i % 17)), "id": i}) + "\n")
        f.write(json.dumps({"text": ""}) + "\n")
    return src


def test_jsonl_to_parquet_shuffle_and_counts(tmp_path):
    src = _corpus(tmp_path)
    shards = jsonl_to_parquet(str(src), str(tmp_path / "pq"), shard_size_mb=1000, keep_keys=("id",))
    assert len(shards) == 1 and pq.read_table(shards[0]).num_rows == 300
    with pytest.raises(FileExistsError):
        jsonl_to_parquet(str(src), str(tmp_path / "pq"))
    tok = WordTokenizer()
    docs, toks = count_tokens(str(tmp_path / "pq"), tok)
    want = sum(1 + i % 17 for i in range(300))
    assert (docs, toks) == (300, want)
    est = estimate_tokens(str(tmp_path / "pq"), tok, min_samples=100, margin=0.5)
    assert est.documents == 300 and est.low <= want <= est.high
    plan = shuffle_split(str(tmp_path / "pq"), str(tmp_path / "shuf"), max_file_mb=1, chunk_size=16, row_group_size=50)
    out = sorted((tmp_path / "shuf").glob("*.parquet"))
    ids = [i for f in out for i in pq.read_table(f).column("id").to_pylist()]
    assert sorted(ids) == list(range(300)) and ids != sorted(ids) and plan.total_rows == 300
    shuffle_split(str(tmp_path / "pq"), str(tmp_path / "shuf2"), method="full", seed=1)
    ids2 = [i for f in sorted((tmp_path / "shuf2").glob("*.parquet")) for i in pq.read_table(f).column("id").to_pylist()]
    assert sorted(ids2) == list(range(300)) and ids2 != sorted(ids2)
    rep = inspect_parquet(shards[0], row=7, show_length=True, tokenizer=tok)
    assert "300 rows" in rep and "row 7" in rep and "tokens:" in rep
    assert "sample 2" in random_dataset_sample(str(tmp_path / "pq"), 2, seed=0)


def test_conversations_to_parquet(tmp_path):
    rows = [{"messages": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}]},
            {"conversations": [{"from": "human", "value": "a"}, {"from": "gpt", "value": "b"}]},
            {"messages": [{"role": "user", "content": "no answer"}]}, {"messages": "broken"}]
    n, skipped = conversations_to_parquet(rows, str(tmp_path / "c.parquet"), shuffle_seed=0)
    assert (n, skipped) == (2, 2)
    got = pq.read_table(tmp_path / "c.parquet").column("messages").to_pylist()
    assert sorted(m[0]["role"] for m in got) == ["user", "user"] and {m[1]["role"] for m in got} == {"assistant"}
    assert normalise_messages([{"from": "bot", "value": "x"}])[0]["role"] == "assistant"


def test_arrow_ingest_and_legacy_loader(tmp_path):
    from maester_b200.datasets.experimental import ArrowShardDataset
    tok = WordTokenizer()
    docs, toks = tokenize_to_arrow((" ".join(["w"] * (3 + i % 5)) for i in range(40)), tok, str(tmp_path / "data"), "mini")
    assert docs == 40 and toks == sum(3 + i % 5 for i in range(40))
    ds = ArrowShardDataset(str(tmp_path / "data" / "mini"), 0, 1, delimiter_token=0, max_chunksize=4)
    it = iter(ds)
    chunks = [next(it) for _ in range(30)]
    assert all(1 <= len(c) <= 5 for c in chunks) and any(c[-1] == 0 for c in chunks)
    state = ds.state_dict()
    nxt = [next(it) for _ in range(5)]
    ds2 = ArrowShardDataset(str(tmp_path / "data" / "mini"), 0, 1, delimiter_token=0, max_chunksize=4)
    ds2.load_state_dict([state])
    it2 = iter(ds2)
    assert [next(it2) for _ in range(5)] == nxt
    # two ranks see disjoint documents that together cover the shard once per epoch
    seen = []
    for r in range(2):
        d = ArrowShardDataset(str(tmp_path / "data" / "mini"), r, 2, delimiter_token=0, max_chunksize=64)
        i = iter(d)
        seen.append([tuple(next(i)) for _ in range(20)])
    assert len(seen[0]) + len(seen[1]) == 40


def test_fake_data_script_and_packed_inspector(tmp_path):
    subprocess.run([sys.executable, "scripts/generate_fake_data.py", "--root", str(tmp_path / "d"), "--docs", "10"], check=True)
    with pa.memory_map(str(tmp_path / "d" / "fake_dataset" / "fullshard.arrow")) as src:
        assert pa.ipc.open_file(src).num_record_batches == 10
    table = pa.table({"pack_id": [0, 1], "input_ids": [[5, 6, 7, 0], [8, 9, 0, 0]], "labels": [[-100, 6, 7, -100], [-100, 9, -100, -100]],
                      "attention_mask": [[1, 1, 1, 0], [1, 1, 0, 0]], "conversation_ids": [[0], [1]],
                      "boundaries": [[[0, 0, 3]], [[1, 0, 2]]]})
    pq.write_table(table, tmp_path / "packed.parquet")
    rep = inspect_packed_data(str(tmp_path / "packed.parquet"), WordTokenizer())
    assert "2 packs of 4 tokens" in rep and "consistency problems: 0" in rep and "first conversation" in rep


def test_tokenizer_training_with_script_filter(tmp_path):
    import tokenizer_train as tt
    f = tt.ScriptFilter.from_preset("latin", 0.1)
    assert f.should_keep_text("Hello world 123!") and not f.should_keep_text("Привет мир") and not f.should_keep_text("1234 !!")
    assert f.should_keep_text("mostly latin text with one ж letter inside it")
    rows = ["the quick brown fox jumps over the lazy dog"] * 200 + ["съешь ещё этих мягких булок"] * 50
    pq.write_table(pa.table({"text": rows}), tmp_path / "c.parquet", row_group_size=64)
    s = tt.ParquetSampler([tt.ParquetSampler.parse(f"{tmp_path}:0.5")], seed=1, text_filter=f)
    tok = tt.train_tokenizer(s.sample_iterator(32), vocab_size=300)
    assert 60 < s.seen < 190 and 0 < s.kept < s.seen
    ids = tok.encode("the lazy dog").ids
    assert tok.decode(ids).strip() == "the lazy dog" and tok.token_to_id("<bos>") == 0 and tok.token_to_id("<eos>") == 1
    tt.main(["--data-path", f"{tmp_path}:1.0", "--output", str(tmp_path / "out" / "tok.json"), "--vocab-size", "280"])
    assert (tmp_path / "out" / "tok.json").is_file()
