"""(Compressed) JSONL documents -> size-bounded Parquet shards with a ``text`` column."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from maester_b200.datatools.ingest import jsonl_to_parquet  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("input_dir", help="directory (or file) with .jsonl / .jsonl.gz / .jsonl.zst documents")
    ap.add_argument("output_dir")
    ap.add_argument("--shard_size", type=int, default=1000, help="target shard size in MB of text")
    ap.add_argument("--mode", choices=["abort", "overwrite"], default="abort")
    ap.add_argument("--text_key", default="text")
    ap.add_argument("--keep", default="", help="comma-separated extra keys to keep as columns")
    a = ap.parse_args()
    shards = jsonl_to_parquet(a.input_dir, a.output_dir, a.shard_size, a.mode, a.text_key,
                              tuple(k for k in a.keep.split(",") if k))
    print(f"wrote {len(shards)} shard(s) to {a.output_dir}")
