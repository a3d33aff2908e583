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


@pytest.mark.parametrize("layout", ["dp2", "dp1_then_tp2"])
def test_train_py_runs_saves_resumes_and_exports(tmp_path, layout):
    """``dp2``: both jobs run as two data-parallel ranks.  ``dp1_then_tp2``: the first job is a single process, the
    second job resumes the single-process checkpoint as two tensor-parallel ranks (the
    checkpoint is resharded on load; both ranks read the same data) and must still reproduce the losses."""
    ranks = 2 if layout == "dp2" else 1
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
    torchrun = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                "127.0.0.1", "--master-port", str(29650 + len(layout))]
    launch = [sys.executable] if ranks == 1 else torchrun

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
    if layout == "dp1_then_tp2":
        cfg = json.loads((cut / "config.json").read_text())
        (cut / "config.json").write_text(json.dumps({**cfg, "tensor_parallel_degree": 2}))
        launch = torchrun
    log_second = _run([*launch, os.path.join(ROOT, "train.py"), str(cut)], cwd=tmp_path)

    a, b = _steps(log_whole), _steps(log_second)
    assert sorted(a) == [1, 2, 4, 6, 8] and sorted(b) == [6, 8], (a, b)
    assert all(0 < v < 8 for v in a.values()), a              # near ln(vocabulary) on random tokens, never diverging
    for s in (6, 8):                                           # resumed: same data, same weights, same schedule
        assert b[s] == pytest.approx(a[s], abs=2e-4), (s, a, b)
    lr = lambda log: set(re.findall(r"Step\s+8: lr=(\S+),", log))   # every rank writes the line
    assert lr(log_whole) == lr(log_second) and lr(log_whole)

    # the last step of each job wrote a weights-only export in bf16
    from maester_b200.convert.io import read_dcp_model
    for d in (whole, cut):
        flat = read_dcp_model(d / "checkpoints" / "step-8")
        assert flat and all(v.dtype == torch.bfloat16 for v in flat.values())
    w1, w2 = read_dcp_model(whole / "checkpoints" / "step-8"), read_dcp_model(cut / "checkpoints" / "step-8")
    for k in w1:
        assert ((w1[k].float() - w2[k].float()).norm() / (w1[k].float().norm() + 1e-12)).item() < 2e-2, k


def _chat_tokenizer_file(path) -> str:
    from tokenizers import Tokenizer, models, pre_tokenizers
    words = ["<unk>", "<eos>", "<bos>", "<|im_start|>", "<|im_end|>", "system", "user", "assistant"] + [f"w{i}" for i in range(200)]
    tok = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok.add_special_tokens(["<|im_start|>", "<|im_end|>", "<eos>", "<bos>"])
    # a folder as save_pretrained writes it: the special-token roles live in a config beside tokenizer.json
    from transformers import PreTrainedTokenizerFast
    folder = str(path) + ".d"
    PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<bos>", eos_token="<eos>").save_pretrained(folder)
    return folder


def _conversations(path, column) -> None:
    os.makedirs(path)
    g = torch.Generator().manual_seed(0)
    rnd = lambda lo, hi: int(torch.randint(lo, hi, (1,), generator=g))
    rows = []
    for _ in range(200):
        turns = []
        for t in range(rnd(2, 5)):
            turns.append({"role": "user" if t % 2 == 0 else "assistant",
                          "content": " " + " ".join(f"w{rnd(0, 200)}" for _ in range(rnd(2, 12))) + " "})
        rows.append(json.dumps(turns))
    pq.write_table(pa.table({column: rows}), os.path.join(path, "c.parquet"), row_group_size=40)


@pytest.mark.parametrize("mode", ["sft", "sft_packed", "deepseek_default_optimizers", "gemma3_mup_off_selective_ac"])
def test_train_py_other_modes_run_to_the_end(tmp_path, mode):
    """The remaining branches of the entry point, a few steps each on CPU: SFT on conversations tokenised on the fly
    (assistant-only masking, padding statistics), SFT on a file written by the packer, a MoE model under the default
    optimizer groups (Muon + AdamW) with the load-balancing hook, Gemma 3 with selective recomputation."""
    head = ""
    if mode.startswith("sft"):
        tok = _chat_tokenizer_file(tmp_path / "tokenizer.json")
        _conversations(tmp_path / "conv", "conversations")
        packed = tmp_path / "packed.parquet"
        if mode == "sft_packed":
            _run([sys.executable, os.path.join(ROOT, "scripts", "pack_sft_data.py"), "--input", str(tmp_path / "conv"),
                  "--output", str(packed), "--tokenizer", tok, "--max-seq-len", "64", "--im-start", "<|im_start|>",
                  "--im-end", "<|im_end|>"], cwd=tmp_path)
            assert packed.exists()
        head = f'''
model_name = "llama3"
flavor = "tiny"
tokenizer_name = "{tok}"
[dataset]
data_dirs = ["{tmp_path / 'conv'}"]
dataset_weights = "1"
[sft]
use_packed = {"true" if mode == "sft_packed" else "false"}
packed_path = "{packed}"
im_start_token = "<|im_start|>"
im_end_token = "<|im_end|>"
'''
        groups = '[[optimizer_groups]]\nopt_class = "torch.optim.AdamW"\nmin_dim = 0\n[optimizer_groups.opt_cfg]\nlr = 1e-3\n'
    elif mode.startswith("deepseek"):
        head = 'model_name = "deepseek"\nflavor = "debug_flex"\nsynthetic_data = true\nsynthetic_vocab_size = 512\nenable_cut_cross_entropy = false\n'
        groups = ""   # the default: Muon for the matrices, AdamW for the rest
    else:
        head = 'model_name = "gemma3"\nflavor = "debug"\nsynthetic_data = true\nsynthetic_vocab_size = 512\nac_mode = "selective"\nselective_ac_option = "op"\n'
        groups = ""
    top, _, tables = head.partition("[dataset]") if "[dataset]" in head else (head, "", "")
    (tmp_path / "job.toml").write_text(
        top + 'seq_len = 64\ntrain_batch_size = 2\nlog_freq = 1\ntrain_num_steps = 3\nenable_checkpoint = true\n'
        'checkpoint_interval = 2\ncompile = false\nfused_collectives = false\ndata_parallel_shard_degree = 1\n'
        'enable_tensorboard = true\n'
        + (("[dataset]" + tables) if tables else "") + groups)
    _run([sys.executable, os.path.join(ROOT, "submit.py"), "--config-file", str(tmp_path / "job.toml"), "--dump-dir",
          str(tmp_path / "jobs"), "--job-name", "j", "--dry-run", "--yes"], cwd=tmp_path)
    log = _run([sys.executable, os.path.join(ROOT, "train.py"), str(tmp_path / "jobs" / "j")], cwd=tmp_path)
    losses = _steps(log)
    assert sorted(losses) == [1, 2, 3] and all(0 < v < 12 for v in losses.values()), (losses, log[-2000:])
    ck = tmp_path / "jobs" / "j" / "checkpoints"
    assert (ck / "step-2" / ".metadata").exists() and (ck / "step-3" / ".metadata").exists()
    if mode.startswith("sft"):   # both SFT loaders report how much of each sample is real tokens
        from tensorboard.backend.event_processing.event_accumulator import EventAccumulator
        events = [r for r, _, fs in os.walk(tmp_path / "jobs" / "j") for f in fs if "tfevents" in f]
        acc = EventAccumulator(events[0])
        acc.Reload()
        tags = set(acc.Tags()["scalars"])
        assert {"padding/efficiency", "padding/avg_length", "padding/std_length"} <= tags, sorted(tags)
        assert 0 < acc.Scalars("padding/efficiency")[-1].value <= 1
    if mode == "sft_packed":
        # the packed reader runs in the training process; its position is saved beside the model checkpoint, so a job
        # restarted from step 2 sees the same third batch
        assert (ck / "dataloader" / "step-2" / "loader_state_0.pth").exists()
        shutil.rmtree(ck / "step-3")
        again = _steps(_run([sys.executable, os.path.join(ROOT, "train.py"), str(tmp_path / "jobs" / "j")], cwd=tmp_path))
        assert sorted(again) == [3] and again[3] == pytest.approx(losses[3], abs=2e-4), (again, losses)


def test_metrics_written_by_train_py_have_the_reference_names(tmp_path):
    """Gradient accumulation, TensorBoard logging and the profiler hooks switched on: the scalar tags are the
    reference trainer's (train.py:448-465 there), so existing dashboards keep working."""
    (tmp_path / "job.toml").write_text(
        'model_name = "llama3"\nflavor = "tiny"\nsynthetic_data = true\nsynthetic_vocab_size = 512\nseq_len = 64\n'
        'train_batch_size = 2\ngradient_accumulation_steps = 2\nlog_freq = 1\ntrain_num_steps = 3\ncompile = false\n'
        'data_parallel_shard_degree = 1\nenable_tensorboard = true\nenable_profiling = true\nprofile_freq = 2\n'
        'enable_checkpoint = false\n[[optimizer_groups]]\nopt_class = "torch.optim.AdamW"\nmin_dim = 0\n'
        '[optimizer_groups.opt_cfg]\nlr = 1e-3\n')
    _run([sys.executable, os.path.join(ROOT, "submit.py"), "--config-file", str(tmp_path / "job.toml"), "--dump-dir",
          str(tmp_path / "jobs"), "--job-name", "j", "--dry-run", "--yes"], cwd=tmp_path)
    log = _run([sys.executable, os.path.join(ROOT, "train.py"), str(tmp_path / "jobs" / "j")], cwd=tmp_path)
    assert sorted(_steps(log)) == [1, 2, 3]
    from tensorboard.backend.event_processing.event_accumulator import EventAccumulator
    events = [os.path.join(r, f) for r, _, fs in os.walk(tmp_path / "jobs" / "j") for f in fs if "tfevents" in f]
    assert events, "no TensorBoard event file"
    acc = EventAccumulator(os.path.dirname(events[0]))
    acc.Reload()
    tags = set(acc.Tags()["scalars"])
    reference_tags = {
        "loss/global_avg", "loss/global_max", "tps", "mfu(%)", "data/total_tokens", "time/end_to_end(s)",
        "time/data_loading_avg(s)", "time/data_loading_max(s)", "time/data_loading_avg(%)", "time/data_loading_max(%)",
        "memory/max_active(GiB)", "memory/max_active(%)", "memory/max_reserved(GiB)", "memory/max_reserved(%)",
        "memory/num_alloc_retries", "memory/num_ooms"}
    assert reference_tags <= tags, sorted(reference_tags - tags)
    assert [e.step for e in acc.Scalars("loss/global_avg")] == [1, 2, 3]
    # 3 steps x 2 micro-batches x 2 sequences x 64 tokens
    assert acc.Scalars("data/total_tokens")[-1].value == 3 * 2 * 2 * 64
    traces = [f for r, _, fs in os.walk(tmp_path / "jobs" / "j") for f in fs if f.endswith(".json") and "config" not in f]
    assert traces, "the profiler wrote no trace"
