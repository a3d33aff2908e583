"""Show the schema, row-group layout and one row of a Parquet file."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from maester_b200.datatools.inspect import inspect_parquet  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("file_path")
    ap.add_argument("--row", "-r", type=int, default=0)
    ap.add_argument("--show-length", "-l", action="store_true")
    ap.add_argument("--show-tokens", "-t", default=None, metavar="TOKENIZER", help="tokenize the text column with this tokenizer")
    a = ap.parse_args()
    tok = None
    if a.show_tokens:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(a.show_tokens)
    print(inspect_parquet(a.file_path, a.row, a.show_length, tok))
