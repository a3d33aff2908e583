"""A Hugging Face chat dataset -> shuffled Parquet with a ``messages`` column for the SFT loader."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from maester_b200.datatools.ingest import conversations_to_parquet  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("dataset")
    ap.add_argument("output")
    ap.add_argument("--row-group-size", type=int, default=100)
    ap.add_argument("--split", default="train")
    ap.add_argument("--subset", default=None)
    ap.add_argument("--messages-key", default="messages")
    ap.add_argument("--shuffle-seed", type=int, default=42)
    ap.add_argument("--streaming", action="store_true")
    ap.add_argument("--no-shuffle", action="store_true")
    a = ap.parse_args()
    from datasets import load_dataset
    rows = load_dataset(a.dataset, a.subset, split=a.split, streaming=a.streaming)
    n, skipped = conversations_to_parquet(rows, a.output, a.messages_key, a.row_group_size,
                                          None if a.no_shuffle else a.shuffle_seed)
    print(f"wrote {n} conversations ({skipped} skipped) to {a.output}")
