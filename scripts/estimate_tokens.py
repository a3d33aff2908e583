"""Estimate the token count of a Parquet corpus from a random sample, with a confidence interval."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from maester_b200.datatools.stats import estimate_tokens  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("parquet_dir")
    ap.add_argument("--tokenizer", default="gpt2")
    ap.add_argument("--text_column", default="text")
    ap.add_argument("--confidence", type=float, default=0.95, choices=[0.90, 0.95, 0.99])
    ap.add_argument("--margin", type=float, default=0.02)
    ap.add_argument("--min_samples", type=int, default=10000)
    ap.add_argument("--max_samples", type=int, default=1000000)
    ap.add_argument("--batch_size", type=int, default=1000)
    ap.add_argument("--seed", type=int, default=42)
    a = ap.parse_args()
    from transformers import AutoTokenizer
    e = estimate_tokens(a.parquet_dir, AutoTokenizer.from_pretrained(a.tokenizer), a.text_column, a.confidence, a.margin,
                        a.min_samples, a.max_samples, a.batch_size, a.seed)
    print(f"{e.documents} documents, {e.sampled} sampled: {e.mean_tokens:.1f} +- {e.std_tokens:.1f} tokens per document")
    print(f"estimated total: {e.total_tokens:,.0f} tokens, {int(100 * e.confidence)}% interval "
          f"[{e.low:,.0f}, {e.high:,.0f}] (+-{100 * e.relative_margin:.2f}%)")
