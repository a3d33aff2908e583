"""Token counts of a Parquet corpus: exact, or estimated from a random sample with a confidence interval
(reference: scripts/count_tokens.py, scripts/estimate_tokens.py)."""
from __future__ import annotations

import math
import random
from dataclasses import dataclass
from pathlib import Path

import pyarrow.parquet as pq

Z = {0.90: 1.6449, 0.95: 1.96, 0.99: 2.5758}


def _files(parquet_dir: str) -> list[str]:
    files = sorted(str(p) for p in Path(parquet_dir).rglob("*.parquet"))
    if not files:
        raise FileNotFoundError(f"no parquet files under {parquet_dir}")
    return files


def _count(tokenizer, texts: list[str]) -> list[int]:
    enc = tokenizer(texts, padding=False, truncation=False, add_special_tokens=False)["input_ids"]
    return [len(x) for x in enc]


def count_tokens(parquet_dir: str, tokenizer, text_column: str = "text", batch_size: int = 1000,
                 progress=lambda docs, toks: None) -> tuple[int, int]:
    """Exact (documents, tokens)."""
    docs = toks = 0
    for f in _files(parquet_dir):
        for batch in pq.ParquetFile(f).iter_batches(batch_size=batch_size, columns=[text_column]):
            texts = [t for t in batch.column(0).to_pylist() if isinstance(t, str)]
            toks += sum(_count(tokenizer, texts))
            docs += len(texts)
            progress(docs, toks)
    return docs, toks


@dataclass
class Estimate:
    documents: int
    sampled: int
    mean_tokens: float
    std_tokens: float
    total_tokens: float
    low: float
    high: float
    confidence: float
    relative_margin: float


def estimate_tokens(parquet_dir: str, tokenizer, text_column: str = "text", confidence: float = 0.95, margin: float = 0.02,
                    min_samples: int = 10_000, max_samples: int = 1_000_000, batch_size: int = 1000, seed: int = 42) -> Estimate:
    """Sample documents uniformly (row groups in random order, all rows of a drawn group) until the
    half-width of the confidence interval of the mean is below ``margin`` x mean, bounded by
    ``min_samples`` / ``max_samples``; total = mean x documents, with a finite-population correction."""
    files = _files(parquet_dir)
    groups, total_docs = [], 0
    for f in files:
        md = pq.ParquetFile(f).metadata
        total_docs += md.num_rows
        groups.extend((f, g) for g in range(md.num_row_groups))
    rng = random.Random(seed)
    rng.shuffle(groups)
    z = Z[confidence]
    n, s1, s2 = 0, 0.0, 0.0
    for f, g in groups:
        col = pq.ParquetFile(f).read_row_group(g, columns=[text_column]).column(0).to_pylist()
        texts = [t for t in col if isinstance(t, str)]
        for i in range(0, len(texts), batch_size):
            for c in _count(tokenizer, texts[i:i + batch_size]):
                n += 1
                s1 += c
                s2 += c * c
        if n >= min_samples or n >= total_docs:
            mean = s1 / n
            var = max(0.0, s2 / n - mean * mean) * n / max(1, n - 1)
            fpc = math.sqrt(max(0.0, (total_docs - n) / max(1, total_docs - 1)))
            half = z * math.sqrt(var / n) * fpc
            if half <= margin * mean or n >= max_samples or n >= total_docs:
                break
    mean = s1 / max(1, n)
    var = max(0.0, s2 / max(1, n) - mean * mean) * n / max(1, n - 1)
    fpc = math.sqrt(max(0.0, (total_docs - n) / max(1, total_docs - 1)))
    half = z * math.sqrt(var / max(1, n)) * fpc
    return Estimate(total_docs, n, mean, math.sqrt(var), mean * total_docs, (mean - half) * total_docs,
                    (mean + half) * total_docs, confidence, half / mean if mean else 0.0)
