"""The data pipeline is the reference's, sample for sample: the reference's own classes (installed copy of the
reference package, maester/datasets/experimental_otf.py) and this repository's read the same Parquet corpus and must
yield the same token lines, keep the same state under the same keys, write the same loader checkpoint files, and each
must resume from the other's files.  Runs as one gloo rank (the reference's dataset constructor asks for the rank)."""
import copy
import glob
import os
import sys

import pytest
import torch

from test_datasets import ToyTokenizer, make_corpus
from test_parallel_cpu import run_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "maester")), reason="the reference is not installed")


def _same(a, b):
    if isinstance(a, torch.Tensor):
        return torch.equal(a, b)
    if isinstance(a, (list, tuple)):
        return len(a) == len(b) and all(_same(x, y) for x, y in zip(a, b))
    if isinstance(a, dict):
        return sorted(a) == sorted(b) and all(_same(a[k], b[k]) for k in a)
    return a == b


def _compare(name, a, b, n):
    ai, bi = iter(a), iter(b)
    for i in range(n):
        x, y = next(ai), next(bi)
        assert _same(x, y), (name, i, list(x)[:10], list(y)[:10])


def _streams(rank, world, tmp):
    sys.path.insert(0, os.path.join(ROOT, "baseline", "shims"))
    sys.path.insert(0, REF)
    import maester.datasets.experimental_otf as R
    import maester_b200.datasets as O
    dirs = [os.path.join(tmp, "a"), os.path.join(tmp, "b")]
    make_corpus(dirs[0], n_files=3, docs_per_file=50, seed=1)
    make_corpus(dirs[1], n_files=2, docs_per_file=30, seed=2)
    tok = ToyTokenizer()
    kw = dict(bos_token=2, min_length=3, seed=42, max_chunksize=64)

    for r, w, weights in [(0, 1, [2.0, 1.0]), (1, 3, [2.0, 1.0]), (0, 2, [1.0, 1.0])]:   # the last one starts on a tie
        def ref_sampling():
            return R.Sampling_Dataset(dirs, r, w, tok, 1, weights=weights, **kw)

        def our_sampling():
            return O.Sampling_Dataset([O.ParquetDataset(d, r, w, tok, delimiter_token=1, **kw) for d in dirs], weights,
                                      delimiter_token=1, rank=r, worldsize=w)

        def pipe(M, source):
            return M.Preprocess_Dataset(M.Preload_Buffer_Dataset(M.Buffer_Dataset(source, 33, pack_hard=True), 50),
                                        O.causal_lm)

        _compare("documents", R.ParquetDataset(dirs[0], r, w, tok, 1, **kw),
                 O.ParquetDataset(dirs[0], r, w, tok, delimiter_token=1, **kw), 300)
        _compare("mixture", ref_sampling(), our_sampling(), 300)
        _compare("packed lines", R.Buffer_Dataset(ref_sampling(), 33, pack_hard=True),
                 O.Buffer_Dataset(our_sampling(), 33, pack_hard=True), 300)
        ref, ours = pipe(R, ref_sampling()), pipe(O, our_sampling())
        ri, oi = iter(ref), iter(ours)
        for i in range(137):   # the shuffle buffer yields from its first step on, like the reference's
            assert _same(next(ri), next(oi)), i
        # (copied at once: the reference's state holds its live shuffle buffer, which the next steps keep changing)
        rs, os_ = copy.deepcopy(ref.state_dict()), copy.deepcopy(ours.state_dict())
        assert _same(rs, os_), sorted(set(rs) ^ set(os_))
        for i in range(100):   # taking the state disturbs neither
            assert _same(next(ri), next(oi)), i
        if w > 1:   # a resume needs the states of all ranks of the saving job
            continue
        # each resumes from the other's state
        a, b = pipe(R, ref_sampling()), pipe(O, our_sampling())
        a.load_state_dict([copy.deepcopy(os_)])
        b.load_state_dict([copy.deepcopy(rs)])
        _compare("resumed", a, b, 200)

    # loader checkpoints: same folders and files, and ours resumes from the folder the reference wrote
    r, w, weights = 0, 1, [2.0, 1.0]
    ref_dir, our_dir = os.path.join(tmp, "ck_ref"), os.path.join(tmp, "ck_ours")
    cr = R.Checkpoint_Dataset(pipe(R, ref_sampling()), ref_dir, 5, 2)
    co = O.Checkpoint_Dataset(pipe(O, our_sampling()), our_dir, 5, 2, save_path=our_dir)
    _compare("checkpointing pipelines", cr, co, 25)
    files = lambda p: sorted(os.path.relpath(x, p) for x in glob.glob(p + "/**", recursive=True) if os.path.isfile(x))
    assert files(ref_dir) == files(our_dir) and files(ref_dir), (files(ref_dir), files(our_dir))
    last = files(ref_dir)[-1]
    assert _same(torch.load(os.path.join(ref_dir, last), weights_only=False),
                 torch.load(os.path.join(our_dir, last), weights_only=False))
    cr2 = R.Checkpoint_Dataset(pipe(R, ref_sampling()), ref_dir, 5, 2)
    co2 = O.Checkpoint_Dataset(pipe(O, our_sampling()), ref_dir, 5, 2, save_path=os.path.join(tmp, "ck_ours2"))
    _compare("resumed from the reference's folder", cr2, co2, 100)
    return True


def test_data_pipeline_is_the_reference_stream_state_and_files(tmp_path):
    assert run_ranks(1, _streams, str(tmp_path)) == [True]


def _builders(rank, world, tmp):
    """Both ``build_experimental_data_loader`` functions on the same configuration: tokenizer file, Parquet folder,
    1-worker DataLoader; the batches are the same tensors under the same keys."""
    sys.path.insert(0, os.path.join(ROOT, "baseline", "shims"))
    sys.path.insert(0, REF)
    import pathlib
    import maester.models  # noqa: F401
    import test_train_end_to_end_cpu as e2e
    from maester.config import Config as RefConfig
    from maester.datasets.experimental_otf import build_experimental_data_loader as ref_build
    from maester_b200.config import Config
    from maester_b200.datasets.experimental_otf import build_experimental_data_loader
    tmp = pathlib.Path(tmp)
    tok = e2e._tokenizer_file(tmp / "tokenizer.json")
    e2e._corpus(tmp / "data")
    kw = dict(seq_len=64, train_batch_size=2, tokenizer_name=tok, enable_checkpoint=False,
              dataset=dict(data_dirs=[str(tmp / "data")], dataset_weights="1", bos_token=2, eos_token=1))
    ref_it, our_it = iter(ref_build(RefConfig(**kw), 0, 1)), iter(build_experimental_data_loader(Config(**kw), 0, 1))
    for i in range(6):
        a, b = next(ref_it), next(our_it)
        assert sorted(a) == sorted(b) == ["input_ids", "labels"], (sorted(a), sorted(b))
        for k in a:
            assert a[k].dtype == b[k].dtype and torch.equal(a[k], b[k]), (i, k)
    # the SFT builders (conversations tokenised on the fly): same padded samples, label masks and real-token counts
    from maester.sft.dataset import build_sft_data_loader as ref_sft
    from maester_b200.sft import build_sft_data_loader
    chat_tok = e2e._chat_tokenizer_file(tmp / "chat_tokenizer.json")
    e2e._conversations(tmp / "conv", "messages")
    kw = dict(seq_len=64, train_batch_size=2, tokenizer_name=chat_tok, enable_checkpoint=False,
              dataset=dict(data_dirs=[str(tmp / "conv")], dataset_weights="1"),
              sft=dict(use_packed=False, conversation_column="messages", im_start_token="<|im_start|>",
                       im_end_token="<|im_end|>"))
    ref_it, our_it = iter(ref_sft(RefConfig(**kw), 0, 1)), iter(build_sft_data_loader(Config(**kw), 0, 1))
    for i in range(6):
        a, b = next(ref_it), next(our_it)
        assert sorted(a) == sorted(b) == ["attention_mask", "input_ids", "labels", "stats"], (sorted(a), sorted(b))
        for k in ("input_ids", "labels", "attention_mask"):
            assert torch.equal(a[k].long(), b[k].long()), (i, k)
        assert torch.equal(a["stats"]["actual_lengths"], b["stats"]["actual_lengths"])
        assert (b["labels"] != -100).any()   # assistant turns are trained on
    os._exit(0)   # the loaders' worker processes are persistent: leave without waiting for them


def test_loader_builders_give_the_same_batches(tmp_path):
    # a child process of its own, started with the interpreter's default method: the reference's pipeline holds live
    # iterators and only reaches its DataLoader worker by fork
    import subprocess
    r = subprocess.run([sys.executable, os.path.abspath(__file__), str(tmp_path)], capture_output=True, text=True,
                       timeout=600, env={**os.environ, "CUDA_VISIBLE_DEVICES": "", "PYTHONPATH": ROOT})
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]


if __name__ == "__main__":
    import torch.distributed as dist
    from test_parallel_cpu import _free_port
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()))
    dist.init_process_group("gloo", rank=0, world_size=1)   # the reference's dataset constructor asks for the rank
    _builders(0, 1, sys.argv[1])
