"""Bring raw corpora into the formats the loaders read.

* ``jsonl_to_parquet``  — (compressed) JSONL documents -> size-bounded Parquet shards with a ``text`` column
                          (reference: scripts/jsonl_to_parquet.py).
* ``tokenize_to_arrow`` — documents from JSONL(.gz) files or a Hugging Face dataset -> one pre-tokenised
                          Arrow IPC shard (one record batch per document, ``tokens`` uint32) plus the
                          ``meta/*counts.csv`` row the legacy loader needs (scripts/hf_to_arrow.py,
                          scripts/jsonl_to_arrow.py).
* ``conversations_to_parquet`` — chat data (JSONL or HF dataset rows with a ``messages`` list of
                          ``{role, content}``) -> Parquet with a list<struct> ``messages`` column for the SFT
                          loader (scripts/hf_convo_to_parquet.py, scripts/jsonl_convo_to_parquet.py).
"""
from __future__ import annotations

import csv
import gzip
import json
import os
import random
from pathlib import Path
from typing import Iterable, Iterator

import pyarrow as pa
import pyarrow.parquet as pq


def open_text(path: str | os.PathLike):
    p = str(path)
    if p.endswith(".gz"):
        return gzip.open(p, "rt", encoding="utf-8")
    if p.endswith(".zst"):
        import subprocess
        proc = subprocess.Popen(["zstd", "-dc", p], stdout=subprocess.PIPE, text=True, encoding="utf-8")
        return proc.stdout
    return open(p, "rt", encoding="utf-8")


def iter_jsonl(paths: Iterable[str | os.PathLike]) -> Iterator[dict]:
    for p in paths:
        with open_text(p) as f:
            for line in f:
                line = line.strip()
                if line:
                    yield json.loads(line)


def find_jsonl(root: str | os.PathLike) -> list[Path]:
    root = Path(root)
    if root.is_file():
        return [root]
    return sorted(p for p in root.rglob("*") if p.is_file() and any(
        p.name.endswith(s) for s in (".jsonl", ".jsonl.gz", ".jsonl.zst", ".json.gz")))


# ----------------------------------------------------------------------------------------- jsonl -> parquet
def jsonl_to_parquet(input_dir: str, output_dir: str, shard_size_mb: int = 1000, mode: str = "abort",
                     text_key: str = "text", keep_keys: tuple[str, ...] = (), row_group_size: int = 10_000) -> list[str]:
    out = Path(output_dir)
    if out.exists() and any(out.iterdir()):
        if mode == "abort":
            raise FileExistsError(f"{out} is not empty (use mode='overwrite')")
        for f in out.glob("*.parquet"):
            f.unlink()
    out.mkdir(parents=True, exist_ok=True)
    limit = shard_size_mb * 2**20
    shards: list[str] = []
    rows: dict[str, list] = {k: [] for k in (text_key, *keep_keys)}
    size = 0

    def flush() -> None:
        nonlocal rows, size
        if not rows[text_key]:
            return
        name = out / f"shard_{len(shards):05d}.parquet"
        pq.write_table(pa.table(rows), name, row_group_size=row_group_size, compression="zstd")
        shards.append(str(name))
        rows = {k: [] for k in rows}
        size = 0

    for doc in iter_jsonl(find_jsonl(input_dir)):
        text = doc.get(text_key)
        if not isinstance(text, str) or not text:
            continue
        rows[text_key].append(text)
        for k in keep_keys:
            rows[k].append(doc.get(k))
        size += len(text.encode("utf-8", errors="ignore"))
        if size >= limit:
            flush()
    flush()
    return shards


# ----------------------------------------------------------------------------------------- tokenised arrow
def tokenize_to_arrow(docs: Iterable[str], tokenizer, output_dir: str, dataset_name: str, shard_name: str = "fullshard.arrow",
                      batch_size: int = 128, append_eos: bool = False) -> tuple[int, int]:
    """Returns (documents, tokens).  Layout: ``<output_dir>/<dataset_name>/<shard>`` and
    ``<output_dir>/meta/<dataset_name>_counts.csv``."""
    root = Path(output_dir)
    (root / dataset_name).mkdir(parents=True, exist_ok=True)
    (root / "meta").mkdir(parents=True, exist_ok=True)
    schema = pa.schema([pa.field("tokens", pa.uint32())])
    ndocs = ntok = 0
    eos = getattr(tokenizer, "eos_token_id", None)
    with pa.ipc.new_file(str(root / dataset_name / shard_name), schema) as writer:
        batch: list[str] = []

        def emit(texts: list[str]) -> None:
            nonlocal ndocs, ntok
            enc = tokenizer(texts, padding=False, truncation=False, add_special_tokens=False)["input_ids"]
            for ids in enc:
                if append_eos and eos is not None:
                    ids = ids + [eos]
                if not ids:
                    continue
                writer.write(pa.record_batch([pa.array(ids, type=pa.uint32())], schema=schema))
                ndocs += 1
                ntok += len(ids)

        for text in docs:
            batch.append(text)
            if len(batch) == batch_size:
                emit(batch)
                batch = []
        if batch:
            emit(batch)
    with open(root / "meta" / f"{dataset_name}_counts.csv", "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["dataset/filename", "documents", "tokens"])
        w.writerow([f"/{dataset_name}/{shard_name}", ndocs, ntok])
    return ndocs, ntok


def hf_dataset_texts(name: str, split: str = "train", subset: str | None = None, text_key: str = "text",
                     streaming: bool = True) -> Iterator[str]:
    from datasets import load_dataset  # optional dependency
    for row in load_dataset(name, subset, split=split, streaming=streaming):
        t = row.get(text_key)
        if isinstance(t, str) and t:
            yield t


# ----------------------------------------------------------------------------------------- conversations
MESSAGE_TYPE = pa.list_(pa.struct([("role", pa.string()), ("content", pa.string())]))


def normalise_messages(msgs, role_map: dict[str, str] | None = None) -> list[dict] | None:
    """Accepts ``[{role, content}]`` or ShareGPT-style ``[{from, value}]``; returns None if unusable."""
    role_map = {"human": "user", "gpt": "assistant", "bot": "assistant", **(role_map or {})}
    out = []
    if not isinstance(msgs, (list, tuple)):
        return None
    for m in msgs:
        if not isinstance(m, dict):
            return None
        role = m.get("role", m.get("from"))
        content = m.get("content", m.get("value"))
        if role is None or not isinstance(content, str):
            return None
        out.append({"role": role_map.get(str(role), str(role)), "content": content})
    return out if any(m["role"] == "assistant" for m in out) else None


def conversations_to_parquet(rows: Iterable[dict], output: str, messages_key: str = "messages", row_group_size: int = 50_000,
                             shuffle_seed: int | None = None, extra_keys: tuple[str, ...] = ()) -> tuple[int, int]:
    """Returns (written, skipped)."""
    convs, skipped = [], 0
    for r in rows:
        msgs = normalise_messages(r.get(messages_key, r.get("conversations")))
        if msgs is None:
            skipped += 1
            continue
        convs.append({"messages": msgs, **{k: r.get(k) for k in extra_keys}})
    if shuffle_seed is not None:
        random.Random(shuffle_seed).shuffle(convs)
    cols = {"messages": pa.array([c["messages"] for c in convs], type=MESSAGE_TYPE)}
    for k in extra_keys:
        cols[k] = pa.array([c[k] for c in convs])
    Path(output).parent.mkdir(parents=True, exist_ok=True)
    pq.write_table(pa.table(cols), output, row_group_size=row_group_size, compression="zstd")
    return len(convs), skipped
