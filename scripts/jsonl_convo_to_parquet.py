"""Chat JSONL (``messages`` lists of {role, content}, or ShareGPT ``conversations``) -> Parquet for the SFT loader."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from maester_b200.datatools.ingest import conversations_to_parquet, iter_jsonl  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("input", help="input JSONL file (optionally .gz / .zst)")
    ap.add_argument("output", help="output Parquet file")
    ap.add_argument("--row-group-size", type=int, default=50000)
    ap.add_argument("--messages-key", default="messages")
    ap.add_argument("--shuffle-seed", type=int, default=None)
    a = ap.parse_args()
    n, skipped = conversations_to_parquet(iter_jsonl([a.input]), a.output, a.messages_key, a.row_group_size, a.shuffle_seed)
    print(f"wrote {n} conversations ({skipped} skipped) to {a.output}")
