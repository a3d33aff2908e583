"""Token sampling and autoregressive decoding shared by the tools (chat, HF generation, data monitor).

Sampling follows the reference's ``scripts/generate_hf.py:10-64``: temperature, top-k, and a
multinomial draw that needs no device-to-host synchronisation (arg-max of ``p / Exp(1)`` noise, the
exponential-race form of the Gumbel trick).  Decoding recomputes the whole prefix each step (the
reference tools keep no KV cache either); ``window`` bounds the prefix for long chats.
"""
from __future__ import annotations

from typing import Callable, Iterable

import torch


def multinomial_sample_one_no_sync(probs: torch.Tensor, generator: torch.Generator | None = None) -> torch.Tensor:
    """One sample per row of ``probs`` [..., V] without ``torch.multinomial`` (which synchronises)."""
    q = torch.empty_like(probs).exponential_(1.0, generator=generator)
    return torch.argmax(probs / q, dim=-1, keepdim=True).to(torch.int64)


def logits_to_probs(logits: torch.Tensor, temperature: float = 1.0, top_k: int | None = None) -> torch.Tensor:
    logits = logits.float() / max(temperature, 1e-5)
    if top_k is not None and top_k > 0:
        k = min(top_k, logits.size(-1))
        kth = torch.topk(logits, k, dim=-1).values[..., -1:]
        logits = torch.where(logits < kth, torch.full_like(logits, -float("inf")), logits)
    return torch.softmax(logits, dim=-1)


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: int | None = None,
           generator: torch.Generator | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """(next token [B, 1], probabilities [B, V]) from last-position logits [B, V]; temperature 0 = greedy."""
    if temperature <= 0:
        probs = torch.softmax(logits.float(), dim=-1)
        return probs.argmax(dim=-1, keepdim=True), probs
    probs = logits_to_probs(logits, temperature, top_k)
    return multinomial_sample_one_no_sync(probs, generator), probs


def _logits_of(model, tokens: torch.Tensor) -> torch.Tensor:
    out = model(tokens)
    return out.logits if hasattr(out, "logits") else out


@torch.no_grad()
def generate(model, prompt: torch.Tensor, max_new_tokens: int, *, temperature: float = 0.8, top_k: int | None = 200,
             eos_ids: Iterable[int] = (), window: int | None = None, callback: Callable[[torch.Tensor], None] | None = None,
             generator: torch.Generator | None = None) -> torch.Tensor:
    """Append up to ``max_new_tokens`` sampled tokens to ``prompt`` [B, T] (native or HF causal LM).

    Stops early when every row has produced one of ``eos_ids`` (checked on the host once per token
    only if ``eos_ids`` is non-empty).  ``callback`` receives each new token tensor [B, 1]."""
    seq = prompt
    eos = torch.tensor(sorted(set(eos_ids)), device=prompt.device, dtype=torch.int64)
    done = torch.zeros(prompt.shape[0], dtype=torch.bool, device=prompt.device)
    for _ in range(max_new_tokens):
        ctx = seq if window is None else seq[:, -window:]
        logits = _logits_of(model, ctx)[:, -1]
        nxt, _ = sample(logits, temperature, top_k, generator)
        seq = torch.cat([seq, nxt], dim=1)
        if callback is not None:
            callback(nxt)
        if eos.numel():
            done |= (nxt == eos[None, :]).any(dim=-1)
            if bool(done.all()):
                break
    return seq


@torch.no_grad()
def greedy(model, prompt: torch.Tensor, max_new_tokens: int, window: int | None = None) -> torch.Tensor:
    return generate(model, prompt, max_new_tokens, temperature=0.0, top_k=None, window=window)
