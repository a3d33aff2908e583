"""JSONL(.gz) documents -> one pre-tokenised Arrow IPC shard + ``meta/<name>_counts.csv`` (legacy loader format)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from maester_b200.datatools.ingest import find_jsonl, iter_jsonl, tokenize_to_arrow  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("input_dir")
    ap.add_argument("output_dir")
    ap.add_argument("output_name", help="dataset name (sub-directory of output_dir)")
    ap.add_argument("tokenizer_name")
    ap.add_argument("--text_key", default="text")
    a = ap.parse_args()
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(a.tokenizer_name)
    texts = (d[a.text_key] for d in iter_jsonl(find_jsonl(a.input_dir)) if isinstance(d.get(a.text_key), str))
    docs, toks = tokenize_to_arrow(texts, tok, a.output_dir, a.output_name)
    print(f"{docs} documents, {toks} tokens")
