"""Pack tokenised conversations into fixed-length training sequences (offline tool).

    python scripts/pack_sft_data.py --input convs.parquet --output packed.parquet --tokenizer <name|file>
        --max-seq-len 8192 [--max-per-pack 4] [--mask-strategy assistant_only] [--buckets 50]

Method (histogram packing solved as a non-negative least-squares problem, as the reference tool does,
scripts/pack_sft_data.py:147-663): conversation lengths are grouped into quantile buckets, every
multiset of up to ``max-per-pack`` buckets whose (conservative, bucket-maximum) lengths fit into
``max-seq-len`` is a packing strategy, and NNLS finds how often to use each strategy so that the
number of conversations drawn from each bucket matches the histogram; residual errors on short
conversations are down-weighted (0.09 below 128 tokens).  The solution is floored, a second NNLS
pass packs what was left over, the rest become singletons.  Output columns: ``pack_id, input_ids,
labels, attention_mask, conversation_ids, boundaries`` with ``boundaries = [(conv id, start, length)]``.
"""
from __future__ import annotations

import argparse
import itertools
import json
import os
import sys
import time
from collections import defaultdict

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

IGNORE = -100


def bucketize(lengths: np.ndarray, n_buckets: int, max_len: int):
    """Quantile buckets → (bucket id per item, {bucket: max length in bucket}, {bucket: count})."""
    edges = np.unique(np.quantile(lengths, np.linspace(0, 1, n_buckets + 1)[1:]).astype(np.int64))
    ids = np.searchsorted(edges, lengths, side="left")
    ids = np.minimum(ids, len(edges) - 1)
    bmax, bcount = {}, {}
    for b in np.unique(ids):
        sel = lengths[ids == b]
        bmax[int(b)], bcount[int(b)] = int(sel.max()), int(sel.size)
    return ids, bmax, bcount


def enumerate_strategies(bmax: dict[int, int], max_len: int, max_per_pack: int):
    out = set()
    keys = sorted(bmax, key=bmax.get)
    for depth in range(1, max_per_pack + 1):
        for combo in itertools.combinations_with_replacement(keys, depth):
            if sum(bmax[b] for b in combo) <= max_len:
                out.add(tuple(sorted(combo)))
    return sorted(out)


def solve_counts(strategies, bcount: dict[int, int], bmax: dict[int, int], short_cutoff: int = 128):
    """NNLS over strategies; returns integer repeat counts (floored) and the per-bucket residual."""
    from scipy import optimize

    buckets = sorted(bcount)
    col = {b: i for i, b in enumerate(buckets)}
    A = np.zeros((len(buckets), len(strategies)))
    for j, s in enumerate(strategies):
        for b in s:
            A[col[b], j] += 1
    target = np.array([bcount[b] for b in buckets], dtype=np.float64)
    w = np.array([0.09 if bmax[b] < short_cutoff else 1.0 for b in buckets])
    x, _ = optimize.nnls(w[:, None] * A, w * target)
    x = np.floor(x).astype(np.int64)
    # never use more items of a bucket than exist
    used = A @ x
    over = used - target
    for i in np.argsort(-over):
        if over[i] <= 0:
            break
        for j in np.argsort(-A[i]):
            while x[j] > 0 and A[i, j] > 0 and (A @ x)[i] > target[i]:
                x[j] -= 1
    residual = target - A @ x
    return x, {b: int(round(residual[col[b]])) for b in buckets}


def plan_packs(lengths: np.ndarray, max_len: int, max_per_pack: int, n_buckets: int):
    """→ list of packs, each a list of conversation indices."""
    ids, bmax, bcount = bucketize(lengths, n_buckets, max_len)
    pools = defaultdict(list)
    for i in np.argsort(-lengths):  # longest first inside a bucket
        pools[int(ids[i])].append(int(i))
    packs: list[list[int]] = []

    def apply(strategies, counts):
        for s, c in zip(strategies, counts):
            for _ in range(int(c)):
                if all(len(pools[b]) >= s.count(b) for b in set(s)):
                    packs.append([pools[b].pop() for b in s])

    strategies = enumerate_strategies(bmax, max_len, max_per_pack)
    counts, residual = solve_counts(strategies, bcount, bmax)
    apply(strategies, counts)
    left = {b: len(p) for b, p in pools.items() if p}
    if sum(left.values()) > 5:
        sub = [s for s in strategies if all(b in left for b in s)]
        if sub:
            counts2, _ = solve_counts(sub, left, bmax)
            apply(sub, counts2)
    # greedy first-fit with exact lengths for whatever remains
    rest = sorted((i for p in pools.values() for i in p), key=lambda i: -lengths[i])
    open_packs: list[tuple[int, list[int]]] = []
    for i in rest:
        for k, (room, members) in enumerate(open_packs):
            if lengths[i] <= room and len(members) < max_per_pack:
                members.append(i)
                open_packs[k] = (room - int(lengths[i]), members)
                break
        else:
            open_packs.append((max_len - int(lengths[i]), [i]))
    packs += [m for _, m in open_packs]
    return packs


def materialise(packs, convs, max_len: int, pad_id: int):
    """convs[i] = (input_ids, labels) already shifted; returns column dict for the output table."""
    rows = defaultdict(list)
    for pid, members in enumerate(packs):
        ids, labs, bounds, cids = [], [], [], []
        for ci in members:
            x, y = convs[ci]
            if len(ids) + len(x) > max_len:
                x, y = x[: max_len - len(ids)], y[: max_len - len(ids)]
            if not x:
                continue
            bounds.append((int(ci), len(ids), len(x)))
            cids.append(int(ci))
            ids += x
            labs += y
        n = len(ids)
        rows["pack_id"].append(pid)
        rows["input_ids"].append(ids + [pad_id] * (max_len - n))
        rows["labels"].append(labs + [IGNORE] * (max_len - n))
        rows["attention_mask"].append([1] * n + [0] * (max_len - n))
        rows["conversation_ids"].append(cids)
        rows["boundaries"].append([list(b) for b in bounds])
    return rows


def tokenize_all(conversations, tokenizer, template, im_start, im_end, mask_strategy, max_len):
    from maester_b200.sft.dataset import mask_labels, tokenize_conversation

    out = []
    for conv in conversations:
        tokens, spans = tokenize_conversation(conv, tokenizer, template, im_start, im_end)
        tokens = tokens[: max_len + 1]
        if len(tokens) < 2:
            continue
        out.append((tokens[:-1], mask_labels(tokens, spans, mask_strategy)))
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--max-seq-len", type=int, default=8192)
    ap.add_argument("--max-per-pack", type=int, default=4)
    ap.add_argument("--buckets", type=int, default=50)
    ap.add_argument("--conversation-column", default="conversations")
    ap.add_argument("--template", default="chatml")
    ap.add_argument("--mask-strategy", default="assistant_only")
    ap.add_argument("--im-start", default="<start_of_turn>")
    ap.add_argument("--im-end", default="<end_of_turn>")
    a = ap.parse_args(argv)
    import pandas as pd
    import pyarrow as pa
    import pyarrow.parquet as pq
    from transformers import AutoTokenizer, PreTrainedTokenizerFast

    tok = PreTrainedTokenizerFast(tokenizer_file=a.tokenizer) if os.path.isfile(a.tokenizer) else \
        AutoTokenizer.from_pretrained(a.tokenizer)
    t0 = time.time()
    df = pd.read_parquet(a.input)
    convs = tokenize_all(df[a.conversation_column].tolist(), tok, a.template, a.im_start, a.im_end, a.mask_strategy,
                         a.max_seq_len)
    lengths = np.array([len(x) for x, _ in convs])
    packs = plan_packs(lengths, a.max_seq_len, a.max_per_pack, a.buckets)
    pad = tok.pad_token_id if tok.pad_token_id is not None else tok.eos_token_id
    rows = materialise(packs, convs, a.max_seq_len, pad)
    pq.write_table(pa.table(rows), a.output)
    eff = lengths.sum() / (len(packs) * a.max_seq_len)
    print(json.dumps({"conversations": len(convs), "packs": len(packs), "efficiency": round(float(eff), 4),
                      "seconds": round(time.time() - t0, 2)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
