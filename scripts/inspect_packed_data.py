"""Statistics and consistency checks of a packed SFT Parquet file (output of pack_sft_data.py)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from maester_b200.datatools.inspect import inspect_packed_data  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("data_path")
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--num_samples", type=int, default=5)
    ap.add_argument("--decode_samples", type=int, default=3)
    a = ap.parse_args()
    tok = None
    if a.tokenizer:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(a.tokenizer)
    print(inspect_packed_data(a.data_path, tok, a.num_samples, a.decode_samples))
