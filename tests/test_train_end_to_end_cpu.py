"""``train.py jobs/<job>`` end to end on CPU: a job directory from ``submit.py``, a Parquet corpus tokenised on the fly
with a tokenizer file, metrics, a checkpoint in the middle, a second invocation that resumes from it (model, optimizer,
schedule, step counter and data loader position), and the weights-only export at the last step.  Once as a single
process and once as two gloo ranks under ``torch.distributed.run``."""
import json
import os
import re
import shutil
import subprocess
import sys

import pyarrow as pa
import pyarrow.parquet as pq
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _tokenizer_file(path) -> str:
    from tokenizers import Tokenizer, models, pre_tokenizers
    vocab = {"<unk>": 0, "<eos>": 1, "<bos>": 2, **{f"w{i}": i + 3 for i in range(250)}}
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(str(path))
    return str(path)


def _corpus(path) -> None:
    os.makedirs(path)
    g = torch.Generator().manual_seed(0)
    for f in range(2):
        docs = [" ".join(f"w{int(t)}" for t in torch.randint(0, 250, (int(torch.randint(5, 90, (1,), generator=g)),), generator=g))
                for _ in range(300)]
        pq.write_table(pa.table({"text": docs}), os.path.join(path, f"part{f}.parquet"), row_group_size=50)


def _run(cmd, cwd, env=None):
    r = subprocess.run(cmd, cwd=cwd, capture_output=True, text=True, timeout=900,
                       env={**os.environ, "CUDA_VISIBLE_DEVICES": "", **(env or {})})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-6000:]
    return r.stdout + r.stderr


def _steps(log: str) -> dict[int, float]:
    return {int(m.group(1)): float(m.group(2)) for m in re.finditer(r"Step\s+(\d+): lr=\S+ loss=\s*([0-9.]+)", log)}


@pytest.mark.parametrize("ranks", [1, 2])
def test_train_py_runs_saves_resumes_and_exports(tmp_path, ranks):
    tok = _tokenizer_file(tmp_path / "tokenizer.json")
    _corpus(tmp_path / "data")
    (tmp_path / "job.toml").write_text(f"""
model_name = "llama3"
flavor = "tiny"
seq_len = 64
train_batch_size = 2
tokenizer_name = "{tok}"
data_parallel_shard_degree = {ranks}
log_freq = 2
enable_checkpoint = true
checkpoint_interval = 4
model_weights_only = true
export_dtype = "bfloat16"
scheduler = "linear_warmup_cosine"
warmup_steps = 2
ac_mode = "none"
compile = false

[dataset]
data_dirs = ["{tmp_path / 'data'}"]
dataset_weights = "1"
bos_token = 2
eos_token = 1

[[optimizer_groups]]
opt_class = "torch.optim.AdamW"
min_dim = 0
[optimizer_groups.opt_cfg]
lr = 3e-3
""")
    common = ["--config-file", str(tmp_path / "job.toml"), "--dump-dir", str(tmp_path / "jobs"), "--dry-run", "--yes"]
    launch = [sys.executable] if ranks == 1 else \
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}", "--master-addr",
         "127.0.0.1", "--master-port", str(29650 + ranks)]

    def job(name, steps):
        _run([sys.executable, os.path.join(ROOT, "submit.py"), *common, "--job-name", name, "--train-num-steps", str(steps)],
             cwd=tmp_path)
        return tmp_path / "jobs" / name

    # an uninterrupted run of 8 steps that checkpoints at step 4, and a second job that starts from a copy of that
    # checkpoint (weights are initialised from an unseeded generator, as in the reference, so two fresh runs differ)
    whole = job("whole", 8)
    log_whole = _run([*launch, os.path.join(ROOT, "train.py"), str(whole)], cwd=tmp_path)
    assert (whole / "checkpoints" / "step-4" / ".metadata").exists()
    cut = job("cut", 8)
    shutil.copytree(whole / "checkpoints", cut / "checkpoints", dirs_exist_ok=True,
                    ignore=lambda d, names: [n for n in names if n == "step-8"])
    log_second = _run([*launch, os.path.join(ROOT, "train.py"), str(cut)], cwd=tmp_path)

    a, b = _steps(log_whole), _steps(log_second)
    assert sorted(a) == [1, 2, 4, 6, 8] and sorted(b) == [6, 8], (a, b)
    assert all(0 < v < 8 for v in a.values()), a              # near ln(vocabulary) on random tokens, never diverging
    for s in (6, 8):                                           # resumed: same data, same weights, same schedule
        assert b[s] == pytest.approx(a[s], abs=2e-4), (s, a, b)
    lr = lambda log: re.findall(r"Step\s+8: lr=(\S+),", log)
    assert lr(log_whole) == lr(log_second) and lr(log_whole)

    # the last step of each job wrote a weights-only export in bf16
    from maester_b200.convert.io import read_dcp_model
    for d in (whole, cut):
        flat = read_dcp_model(d / "checkpoints" / "step-8")
        assert flat and all(v.dtype == torch.bfloat16 for v in flat.values())
    w1, w2 = read_dcp_model(whole / "checkpoints" / "step-8"), read_dcp_model(cut / "checkpoints" / "step-8")
    for k in w1:
        assert ((w1[k].float() - w2[k].float()).norm() / (w1[k].float().norm() + 1e-12)).item() < 2e-2, k
