"""A Hugging Face dataset (streamed) -> one pre-tokenised Arrow IPC shard + counts CSV (legacy loader format)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from maester_b200.datatools.ingest import hf_dataset_texts, tokenize_to_arrow  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("dataset", help="dataset name or path for datasets.load_dataset")
    ap.add_argument("output_dir")
    ap.add_argument("tokenizer_name")
    ap.add_argument("--name", default=None, help="output dataset name (default: last path component)")
    ap.add_argument("--split", default="train")
    ap.add_argument("--subset", default=None)
    ap.add_argument("--text_key", default="text")
    ap.add_argument("--no-streaming", action="store_true")
    a = ap.parse_args()
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(a.tokenizer_name)
    name = a.name or a.dataset.rstrip("/").split("/")[-1]
    docs, toks = tokenize_to_arrow(hf_dataset_texts(a.dataset, a.split, a.subset, a.text_key, not a.no_streaming),
                                   tok, a.output_dir, name)
    print(f"{docs} documents, {toks} tokens")
