"""Shuffle a Parquet corpus and split it into files of bounded size
(reference: scripts/shuffle_split_parquet.py).

Two methods.  ``round_robin`` streams the input once: every chunk of ``chunk_size`` rows goes to a
randomly chosen output file's buffer, buffers are shuffled when written, so memory stays at
``n_outputs x chunk`` rows; adjacent rows end up in different files and in random positions, which is
what the training loader needs on top of its own document shuffle.  ``full`` loads everything and
applies one global permutation.  ``plan`` reports the output layout without touching data.
"""
from __future__ import annotations

import math
import random
from dataclasses import dataclass
from pathlib import Path

import pyarrow as pa
import pyarrow.parquet as pq


@dataclass
class Plan:
    files: list[str]
    total_rows: int
    total_bytes: int
    n_outputs: int
    rows_per_output: int


def plan(input_dir: str, max_file_mb: int = 100) -> Plan:
    files = sorted(str(p) for p in Path(input_dir).rglob("*.parquet"))
    if not files:
        raise FileNotFoundError(f"no parquet files under {input_dir}")
    rows = size = 0
    for f in files:
        md = pq.ParquetFile(f).metadata
        rows += md.num_rows
        size += sum(md.row_group(i).total_byte_size for i in range(md.num_row_groups))
    n_out = max(1, math.ceil(size / (max_file_mb * 2**20)))
    return Plan(files, rows, size, n_out, math.ceil(rows / n_out))


def shuffle_split(input_dir: str, output_dir: str, max_file_mb: int = 100, row_group_size: int = 10_000,
                  compression: str = "snappy", method: str = "round_robin", seed: int = 42, chunk_size: int = 1000,
                  dry_run: bool = False) -> Plan:
    p = plan(input_dir, max_file_mb)
    if dry_run:
        return p
    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    rng = random.Random(seed)
    names = [out / f"shuffled_{i:05d}.parquet" for i in range(p.n_outputs)]
    if method == "full":
        table = pa.concat_tables([pq.read_table(f) for f in p.files], promote_options="default")
        perm = list(range(table.num_rows))
        rng.shuffle(perm)
        table = table.take(pa.array(perm))
        for i, name in enumerate(names):
            lo, hi = i * p.rows_per_output, min(table.num_rows, (i + 1) * p.rows_per_output)
            if hi > lo:
                pq.write_table(table.slice(lo, hi - lo), name, row_group_size=row_group_size, compression=compression)
        return p
    if method != "round_robin":
        raise ValueError(f"unknown method {method}")
    buffers: list[list[pa.Table]] = [[] for _ in names]
    buffered = [0] * len(names)
    writers: list[pq.ParquetWriter | None] = [None] * len(names)
    flush_rows = max(row_group_size, chunk_size)

    def flush(i: int) -> None:
        if not buffers[i]:
            return
        t = pa.concat_tables(buffers[i], promote_options="default")
        perm = list(range(t.num_rows))
        rng.shuffle(perm)
        t = t.take(pa.array(perm))
        if writers[i] is None:
            writers[i] = pq.ParquetWriter(names[i], t.schema, compression=compression)
        writers[i].write_table(t, row_group_size=row_group_size)
        buffers[i], buffered[i] = [], 0

    order = list(p.files)
    rng.shuffle(order)
    for f in order:
        pf = pq.ParquetFile(f)
        for batch in pf.iter_batches(batch_size=chunk_size):
            i = rng.randrange(len(names))
            buffers[i].append(pa.Table.from_batches([batch]))
            buffered[i] += batch.num_rows
            if buffered[i] >= flush_rows:
                flush(i)
    for i in range(len(names)):
        flush(i)
        if writers[i] is not None:
            writers[i].close()
    return p
