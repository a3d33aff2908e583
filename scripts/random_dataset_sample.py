"""Show random rows of a Parquet dataset directory."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from maester_b200.datatools.inspect import random_dataset_sample  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("data_dir")
    ap.add_argument("--num-samples", "-n", type=int, default=5)
    ap.add_argument("--seed", "-s", type=int, default=None)
    ap.add_argument("--show-content", "-c", action="store_true")
    a = ap.parse_args()
    print(random_dataset_sample(a.data_dir, a.num_samples, a.seed, a.show_content))
