"""Write a tiny pre-tokenised Arrow dataset (1000 documents of 100 consecutive integers) with its counts CSV."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import csv  # noqa: E402

import pyarrow as pa  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--root", default="data")
    ap.add_argument("--docs", type=int, default=1000)
    ap.add_argument("--doc-len", type=int, default=100)
    a = ap.parse_args()
    os.makedirs(os.path.join(a.root, "fake_dataset"), exist_ok=True)
    os.makedirs(os.path.join(a.root, "meta"), exist_ok=True)
    schema = pa.schema([pa.field("tokens", pa.uint32())])
    with pa.ipc.new_file(os.path.join(a.root, "fake_dataset", "fullshard.arrow"), schema) as w:
        for i in range(a.docs):
            w.write(pa.record_batch([pa.array(range(i * a.doc_len, (i + 1) * a.doc_len), type=pa.uint32())], schema=schema))
    with open(os.path.join(a.root, "meta", "combined_counts.csv"), "w", newline="") as f:
        cw = csv.writer(f)
        cw.writerow(["dataset/filename", "documents", "tokens"])
        cw.writerow(["/fake_dataset/fullshard.arrow", a.docs, a.docs * a.doc_len])
    print(f"wrote {a.docs} documents under {a.root}/fake_dataset")
