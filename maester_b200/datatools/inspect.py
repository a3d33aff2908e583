"""Look inside datasets: one Parquet row, random samples of a corpus, packed SFT files
(reference: scripts/inspect_parquet.py, scripts/random_dataset_sample.py, scripts/inspect_packed_data.py).
Every function returns the report as text (the scripts print it)."""
from __future__ import annotations

import random
import statistics
from pathlib import Path

import pyarrow.parquet as pq

IGNORE = -100


def _clip(s: str, n: int = 400) -> str:
    s = s.replace("\n", "\\n")
    return s if len(s) <= n else s[:n] + f"... [{len(s)} chars]"


def inspect_parquet(path: str, row: int = 0, show_length: bool = False, tokenizer=None, text_column: str = "text") -> str:
    pf = pq.ParquetFile(path)
    md = pf.metadata
    lines = [f"{path}: {md.num_rows} rows, {md.num_row_groups} row groups, {md.serialized_size} B metadata",
             "schema: " + ", ".join(f"{f.name}:{f.type}" for f in pf.schema_arrow)]
    sizes = [md.row_group(i).num_rows for i in range(md.num_row_groups)]
    lines.append(f"row group sizes: min {min(sizes)}, max {max(sizes)}")
    if not 0 <= row < md.num_rows:
        raise IndexError(f"row {row} outside [0, {md.num_rows})")
    g, off = 0, row
    while off >= sizes[g]:
        off -= sizes[g]
        g += 1
    rec = pf.read_row_group(g).slice(off, 1).to_pylist()[0]
    lines.append(f"row {row} (row group {g}, offset {off}):")
    for k, v in rec.items():
        if isinstance(v, str):
            extra = f" [{len(v)} chars]" if show_length else ""
            lines.append(f"  {k}{extra}: {_clip(v)}")
            if tokenizer is not None and k == text_column:
                ids = tokenizer.encode(v, add_special_tokens=False)
                lines.append(f"  {k} tokens: {len(ids)} (first 32: {ids[:32]})")
        elif isinstance(v, list):
            lines.append(f"  {k}: list[{len(v)}] {_clip(str(v[:8]))}")
        else:
            lines.append(f"  {k}: {v!r}")
    return "\n".join(lines)


def random_dataset_sample(data_dir: str, num_samples: int = 5, seed: int | None = None, show_content: bool = False,
                          text_column: str = "text") -> str:
    files = sorted(str(p) for p in Path(data_dir).rglob("*.parquet"))
    if not files:
        raise FileNotFoundError(f"no parquet files under {data_dir}")
    rng = random.Random(seed)
    counts = [pq.ParquetFile(f).metadata.num_rows for f in files]
    total = sum(counts)
    lines = [f"{data_dir}: {len(files)} files, {total} rows"]
    for s in range(num_samples):
        idx = rng.randrange(total)
        fi = 0
        while idx >= counts[fi]:
            idx -= counts[fi]
            fi += 1
        pf = pq.ParquetFile(files[fi])
        g, off = 0, idx
        while off >= pf.metadata.row_group(g).num_rows:
            off -= pf.metadata.row_group(g).num_rows
            g += 1
        rec = pf.read_row_group(g).slice(off, 1).to_pylist()[0]
        text = rec.get(text_column)
        lines.append(f"--- sample {s + 1}: {Path(files[fi]).name} row {idx}")
        for k, v in rec.items():
            if k == text_column and isinstance(v, str):
                lines.append(f"  {k} [{len(v)} chars]: {v if show_content else _clip(v, 200)}")
            else:
                lines.append(f"  {k}: {_clip(str(v), 120)}")
        if text is None:
            lines.append(f"  (no '{text_column}' column)")
    return "\n".join(lines)


def inspect_packed_data(path: str, tokenizer=None, num_samples: int = 5, decode_samples: int = 3) -> str:
    """Statistics of a packed SFT file: fill rate, conversations per pack, supervised-token share,
    boundary consistency; decodes the first conversations of a few packs when a tokenizer is given."""
    t = pq.read_table(path)
    cols = set(t.column_names)
    need = {"input_ids", "labels", "attention_mask", "boundaries"}
    if not need <= cols:
        raise ValueError(f"{path} is not a packed SFT file: missing {sorted(need - cols)}")
    n = t.num_rows
    masks = t.column("attention_mask").to_pylist()
    labels = t.column("labels").to_pylist()
    bounds = t.column("boundaries").to_pylist()
    ids = t.column("input_ids").to_pylist()
    seq_len = len(ids[0]) if n else 0
    fill = [sum(m) / max(1, len(m)) for m in masks]
    per_pack = [len(b) for b in bounds]
    sup = [sum(1 for x in l if x != IGNORE) for l in labels]
    real = [sum(m) for m in masks]
    problems = []
    for r in range(n):
        pos = 0
        for cid, start, length in bounds[r]:
            if start != pos:
                problems.append(f"pack {r}: conversation {cid} starts at {start}, expected {pos}")
            pos = start + length
        if pos != real[r]:
            problems.append(f"pack {r}: boundaries cover {pos} tokens, attention mask {real[r]}")
        if any(x != IGNORE for x in labels[r][real[r]:]):
            problems.append(f"pack {r}: labels set on padding")
    lines = [f"{path}: {n} packs of {seq_len} tokens",
             f"fill rate: mean {statistics.fmean(fill):.4f}, min {min(fill):.4f}" if n else "empty file",
             f"conversations per pack: mean {statistics.fmean(per_pack):.2f}, max {max(per_pack)}" if n else "",
             f"supervised tokens: {sum(sup)} of {sum(real)} real tokens ({100 * sum(sup) / max(1, sum(real)):.1f}%)",
             f"consistency problems: {len(problems)}"]
    lines += [f"  {p}" for p in problems[:10]]
    for r in range(min(num_samples, n)):
        lines.append(f"pack {r}: {per_pack[r]} conversations, {real[r]} tokens, boundaries {bounds[r][:6]}")
        if tokenizer is not None and r < decode_samples and bounds[r]:
            cid, start, length = bounds[r][0]
            lines.append(f"  first conversation ({cid}): {_clip(tokenizer.decode(ids[r][start:start + length]), 300)}")
            tgt = [x for x in labels[r][start:start + length] if x != IGNORE]
            lines.append(f"  its supervised targets: {_clip(tokenizer.decode(tgt), 200)}")
    return "\n".join(l for l in lines if l)
