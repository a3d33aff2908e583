"""Exact number of documents and tokens of a Parquet corpus under a tokenizer."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from maester_b200.datatools.stats import count_tokens  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("parquet_dir")
    ap.add_argument("--tokenizer", default="gpt2")
    ap.add_argument("--text_column", default="text")
    ap.add_argument("--batch_size", type=int, default=1000)
    a = ap.parse_args()
    from transformers import AutoTokenizer
    docs, toks = count_tokens(a.parquet_dir, AutoTokenizer.from_pretrained(a.tokenizer), a.text_column, a.batch_size,
                              lambda d, t: print(f"\r{d} documents, {t} tokens", end="", flush=True))
    print(f"\ntotal: {docs} documents, {toks} tokens ({toks / max(1, docs):.1f} per document)")
