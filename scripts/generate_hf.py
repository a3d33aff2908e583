"""Sample text from a Hugging Face causal LM directory (e.g. an export made by ``from_dcp.py``).

    python scripts/generate_hf.py <model_dir> --prompt "..." [--num-samples 3] [--max-new-tokens 200]
           [--temperature 0.8 --top-k 200] [--device cuda] [--dtype bfloat16]

Uses the framework's sampling loop (temperature, top-k, synchronisation-free multinomial; reference:
scripts/generate_hf.py:10-64).  ``mup_llama`` exports load because the model type is registered on
import.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import torch  # noqa: E402

from maester_b200.generate import generate  # noqa: E402


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description="Generate text with an HF causal LM")
    ap.add_argument("model_dir")
    ap.add_argument("--prompt", default="Hello, my name is")
    ap.add_argument("--num-samples", type=int, default=1)
    ap.add_argument("--max-new-tokens", type=int, default=200)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--top-k", type=int, default=200)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    ap.add_argument("--seed", type=int, default=1234)
    a = ap.parse_args(argv)

    from transformers import AutoModelForCausalLM, AutoTokenizer

    import maester_b200.models.hf.modeling_mup_llama  # noqa: F401  (registers the mup_llama model type)

    tok = AutoTokenizer.from_pretrained(a.model_dir)
    model = AutoModelForCausalLM.from_pretrained(a.model_dir, torch_dtype=getattr(torch, a.dtype)).to(a.device).eval()
    torch.manual_seed(a.seed)
    ids = torch.tensor([tok.encode(a.prompt)], device=a.device, dtype=torch.int64)
    eos = [tok.eos_token_id] if tok.eos_token_id is not None else []
    for i in range(a.num_samples):
        t0 = time.perf_counter()
        out = generate(model, ids, a.max_new_tokens, temperature=a.temperature, top_k=a.top_k, eos_ids=eos)
        if a.device.startswith("cuda"):
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        n = out.shape[1] - ids.shape[1]
        print(f"--- sample {i + 1}: {n} tokens in {dt:.2f} s ({n / dt:.1f} tok/s)")
        print(tok.decode(out[0].tolist()))


if __name__ == "__main__":
    main()
