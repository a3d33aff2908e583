"""Command-line front ends shared by ``scripts/convert/<family>/{to,from}_dcp.py``.

    python scripts/convert/llama/to_dcp.py   <hf_dir>  <dcp_dir>
    python scripts/convert/llama/from_dcp.py <dcp_dir> <hf_dir> [--model-name llama3 --flavor 8B]
                                             [--dtype bfloat16] [--max-shard-size-gb 5]
                                             [--tokenizer <dir or hub name>] [--chat-template chatml]

``from_dcp`` recovers ``model_name`` / ``flavor`` (and muP overrides) from the job's ``config.json``
next to the checkpoint when the flags are not given, reads only the ``model.*`` tensors of the
checkpoint, and writes sharded safetensors, an index, an HF ``config.json`` and, on request, the
tokenizer files with a ChatML chat template (what SFT checkpoints need for serving).
"""
from __future__ import annotations

import argparse
import copy
import json
import shutil
from pathlib import Path

import torch

from maester_b200.convert import FAMILIES, arch_from_hf_config, arch_from_model_args, to_hf, to_native
from maester_b200.convert.hf_config import hf_config_from_args
from maester_b200.convert.io import find_job_config, read_dcp_model, read_hf_dir, write_dcp, write_hf_dir

CHATML_TEMPLATE = (
    "{% for message in messages %}{{'<|im_start|>' + message['role'] + '\\n' + message['content'] + '<|im_end|>' + '\\n'}}"
    "{% endfor %}{% if add_generation_prompt %}{{ '<|im_start|>assistant\\n' }}{% endif %}"
)
DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}


def convert_to_dcp(family: str, hf_dir: str, out_dir: str, strict: bool = True) -> dict[str, torch.Tensor]:
    sd, cfg = read_hf_dir(hf_dir)
    arch = arch_from_hf_config(family, cfg)
    native = to_native(FAMILIES[family], sd, arch, strict=strict)
    write_dcp(out_dir, native)
    return native


def resolve_model_args(family: str, checkpoint_dir: str, model_name: str | None, flavor: str | None,
                       job_config: str | None = None):
    """Native ModelArgs for a checkpoint: flags win, else the job's config.json."""
    from maester_b200.models import models_config

    job = json.loads(Path(job_config).read_text()) if job_config else find_job_config(checkpoint_dir)
    model_name = model_name or (job or {}).get("model_name")
    flavor = flavor or (job or {}).get("flavor")
    if not model_name or not flavor:
        raise SystemExit("cannot determine the architecture: pass --model-name and --flavor (no job config.json found)")
    args = copy.deepcopy(models_config[model_name][flavor])
    if job:
        if job.get("enable_mup") and hasattr(args, "enable_mup"):
            args.enable_mup = True
            args.mup_input_alpha = job.get("mup_input_alpha", 1.0)
            args.mup_output_alpha = job.get("mup_output_alpha", 1.0)
            args.mup_width_mul = job.get("model_width", args.dim) / job.get("base_model_width", args.dim)
            args.dim = job.get("model_width", args.dim)
            args.n_heads = args.dim // 128
            if getattr(args, "n_kv_heads", None):
                args.n_kv_heads = min(args.n_kv_heads, args.n_heads)
        if job.get("seq_len"):
            args.max_seq_len = job["seq_len"]
    return args, model_name


def convert_from_dcp(family: str, dcp_dir: str, out_dir: str, *, model_name=None, flavor=None, job_config=None,
                     dtype: torch.dtype = torch.bfloat16, max_shard_bytes: int = 5 * 2**30, tokenizer: str | None = None,
                     chat_template: str | None = None) -> list[str]:
    args, model_name = resolve_model_args(family, dcp_dir, model_name, flavor, job_config)
    native = read_dcp_model(dcp_dir)
    if getattr(args, "vocab_size", 0) <= 0 and "tok_embeddings.weight" in native:
        args.vocab_size = native["tok_embeddings.weight"].shape[0]
    arch = arch_from_model_args(family, args)
    hf = to_hf(FAMILIES[family], native, arch)
    tied = getattr(args, "tied_embeddings", False) or getattr(args, "tie_word_embeddings", False)
    if tied:
        hf.pop("lm_head.weight", None)
    files = write_hf_dir(out_dir, hf, hf_config_from_args(family, args), max_shard_bytes=max_shard_bytes, dtype=dtype)
    if tokenizer:
        export_tokenizer(tokenizer, out_dir, chat_template)
    return files


def export_tokenizer(src: str, out_dir: str, chat_template: str | None) -> None:
    """Copy tokenizer files; optionally install a chat template (``chatml`` or a Jinja string/file)."""
    out = Path(out_dir)
    p = Path(src)
    if p.is_dir():
        for f in p.iterdir():
            if f.name.startswith(("tokenizer", "special_tokens", "vocab", "merges", "added_tokens")):
                shutil.copy(f, out / f.name)
    else:
        from transformers import AutoTokenizer
        AutoTokenizer.from_pretrained(src).save_pretrained(str(out))
    if chat_template:
        template = CHATML_TEMPLATE if chat_template == "chatml" else (
            Path(chat_template).read_text() if Path(chat_template).is_file() else chat_template)
        cfg_file = out / "tokenizer_config.json"
        cfg = json.loads(cfg_file.read_text()) if cfg_file.is_file() else {}
        cfg["chat_template"] = template
        cfg_file.write_text(json.dumps(cfg, indent=2))


def to_dcp_main(family: str, argv=None) -> None:
    ap = argparse.ArgumentParser(description=f"Convert {family} safetensors weights to a DCP checkpoint")
    ap.add_argument("input_dir", help="HF checkpoint directory (safetensors + config.json)")
    ap.add_argument("output_dir", help="DCP checkpoint directory to create")
    ap.add_argument("--combine-qkv", action="store_true", help="accepted for compatibility: q/k/v are always fused where the model fuses them")
    ap.add_argument("--lenient", action="store_true", help="skip tensors that have no rule instead of failing")
    a = ap.parse_args(argv)
    native = convert_to_dcp(family, a.input_dir, a.output_dir, strict=not a.lenient)
    n = sum(t.numel() for t in native.values())
    print(f"wrote {len(native)} tensors ({n / 1e9:.2f} B parameters) to {a.output_dir}")


def from_dcp_main(family: str, argv=None) -> None:
    ap = argparse.ArgumentParser(description=f"Convert a {family} DCP checkpoint to HF safetensors")
    ap.add_argument("checkpoint_dir")
    ap.add_argument("output_dir")
    ap.add_argument("--model-name")
    ap.add_argument("--flavor")
    ap.add_argument("--job-config", help="path of the training job's config.json")
    ap.add_argument("--dtype", choices=sorted(DTYPES), default="bfloat16")
    ap.add_argument("--max-shard-size-gb", type=float, default=5.0)
    ap.add_argument("--tokenizer")
    ap.add_argument("--chat-template", help="'chatml', a Jinja string or a file")
    a = ap.parse_args(argv)
    files = convert_from_dcp(family, a.checkpoint_dir, a.output_dir, model_name=a.model_name, flavor=a.flavor,
                             job_config=a.job_config, dtype=DTYPES[a.dtype],
                             max_shard_bytes=int(a.max_shard_size_gb * 2**30), tokenizer=a.tokenizer,
                             chat_template=a.chat_template)
    print(f"wrote {len(files)} safetensors file(s) to {a.output_dir}")
