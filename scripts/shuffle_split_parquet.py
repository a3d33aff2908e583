"""Shuffle a Parquet corpus and split it into files of bounded size."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from maester_b200.datatools.shuffle import shuffle_split  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("input_dir")
    ap.add_argument("output_dir")
    ap.add_argument("--max-size-mb", type=int, default=100)
    ap.add_argument("--row-group-size", type=int, default=10000)
    ap.add_argument("--compression", default="snappy", choices=["snappy", "zstd", "gzip", "none"])
    ap.add_argument("--method", default="round_robin", choices=["round_robin", "full"])
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--chunk-size", type=int, default=1000)
    a = ap.parse_args()
    p = shuffle_split(a.input_dir, a.output_dir, a.max_size_mb, a.row_group_size, a.compression, a.method, a.seed,
                      a.chunk_size, a.dry_run)
    print(f"{len(p.files)} input files, {p.total_rows} rows, {p.total_bytes / 2**20:.1f} MiB -> {p.n_outputs} output "
          f"file(s) of ~{p.rows_per_output} rows{' (dry run)' if a.dry_run else ''}")
