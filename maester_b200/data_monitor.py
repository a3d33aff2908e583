"""Human-readable checks of what the model is fed and what it predicts.

Same services as the reference's ``DataMonitor`` (maester/data_monitor.py:8-234: decoded batch
samples, top-k next-token predictions against the labels, greedy generations from fixed prompts and
from batch prefixes, dataset statistics; constructed but disabled in its train.py:243).  Everything
runs on rank 0 every ``log_freq`` steps and returns the text it logged, so it can be tested.
The tokenizer is found on the dataset chain (any wrapper exposing ``.tokenizer``) or passed in.
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist

from maester_b200.generate import greedy
from maester_b200.log_utils import logger


def find_tokenizer(dataset):
    """Walk ``.dataset`` / ``.data[0]`` wrappers until something carries a tokenizer."""
    seen = 0
    while dataset is not None and seen < 16:
        tok = getattr(dataset, "tokenizer", None)
        if tok is not None:
            return tok
        nxt = getattr(dataset, "dataset", None)
        if nxt is None:
            data = getattr(dataset, "data", None)
            nxt = data[0] if isinstance(data, (list, tuple)) and data else None
        dataset, seen = nxt, seen + 1
    return None


class DataMonitor:
    def __init__(self, train_state, log_freq: int = 100, sample_size: int = 3, top_k: int = 5, tokenizer=None,
                 prompts: Sequence[str] = ("The capital of Denmark is", "Once upon a time")):
        self.train_state = train_state
        self.log_freq, self.sample_size, self.top_k = log_freq, sample_size, top_k
        self.tokenizer = tokenizer
        self.prompts = list(prompts)
        self.rank = dist.get_rank() if dist.is_initialized() else 0

    # ------------------------------------------------------------------ helpers
    def _due(self) -> bool:
        return self.rank == 0 and self.train_state.step % self.log_freq == 0

    def _tok(self, dataset=None):
        if self.tokenizer is None and dataset is not None:
            self.tokenizer = find_tokenizer(dataset)
        if self.tokenizer is None:
            raise ValueError("DataMonitor needs a tokenizer (none given, none found on the dataset chain)")
        return self.tokenizer

    def _decode(self, ids, dataset=None) -> str:
        ids = [int(i) for i in ids if int(i) >= 0]
        return self._tok(dataset).decode(ids)

    def _emit(self, lines: list[str]) -> str:
        text = "\n".join(lines)
        logger.info(text)
        return text

    # ------------------------------------------------------------------ services
    def log_batch_samples(self, input_ids: torch.Tensor, labels: torch.Tensor, dataset=None) -> str | None:
        if not self._due():
            return None
        lines = [f"[data monitor] step {self.train_state.step}: {min(self.sample_size, input_ids.shape[0])} batch samples"]
        for b in range(min(self.sample_size, input_ids.shape[0])):
            ids = input_ids[b].tolist()
            lines.append(f"  sample {b}: {len(ids)} tokens, first 16 ids {ids[:16]}")
            lines.append(f"    text : {self._decode(ids[:64], dataset)!r}")
            shifted = bool((labels[b, :-1] == input_ids[b, 1:]).float().mean() > 0.5) if labels.shape == input_ids.shape else False
            masked = int((labels[b] < 0).sum())
            lines.append(f"    labels are inputs shifted by one: {shifted}; masked label positions: {masked}")
        return self._emit(lines)

    def log_predictions(self, pred: torch.Tensor, labels: torch.Tensor, dataset=None, context: torch.Tensor | None = None,
                        positions: int = 5) -> str | None:
        """pred: logits [B, S, V] (position t predicts token t+1 = labels[:, t])."""
        if not self._due():
            return None
        lines = [f"[data monitor] step {self.train_state.step}: top-{self.top_k} predictions"]
        S = pred.shape[1]
        for b in range(min(self.sample_size, pred.shape[0])):
            for t in torch.linspace(0, S - 1, positions).long().tolist():
                probs = torch.softmax(pred[b, t].float(), dim=-1)
                top_p, top_i = probs.topk(self.top_k)
                want = int(labels[b, t])
                cands = ", ".join(f"{self._decode([i], dataset)!r}:{p:.2f}" for i, p in zip(top_i.tolist(), top_p.tolist()))
                ctx = "" if context is None else f" after {self._decode(context[b, max(0, t - 8): t + 1].tolist(), dataset)!r}"
                hit = "hit " if want in top_i.tolist() else "miss"
                target = "<masked>" if want < 0 else repr(self._decode([want], dataset))
                lines.append(f"  [{b},{t}] {hit} target {target}{ctx}: {cands}")
        return self._emit(lines)

    def log_generations(self, model: torch.nn.Module, input_ids: torch.Tensor | None = None, dataset=None,
                        max_tokens: int = 50, prefix_len: int = 16) -> str | None:
        if not self._due():
            return None
        tok = self._tok(dataset)
        device = next(model.parameters()).device
        was_training = model.training
        model.eval()
        lines = [f"[data monitor] step {self.train_state.step}: greedy generations"]
        try:
            for p in self.prompts:
                ids = torch.tensor([tok.encode(p)], device=device, dtype=torch.int64)
                out = greedy(model, ids, max_tokens)
                lines.append(f"  prompt {p!r} -> {self._decode(out[0, ids.shape[1]:].tolist(), dataset)!r}")
            if input_ids is not None:
                for b in range(min(self.sample_size, input_ids.shape[0])):
                    ids = input_ids[b: b + 1, :prefix_len].to(device)
                    out = greedy(model, ids, max_tokens)
                    lines.append(f"  batch prefix {self._decode(ids[0].tolist(), dataset)!r} -> "
                                 f"{self._decode(out[0, ids.shape[1]:].tolist(), dataset)!r}")
        finally:
            model.train(was_training)
        return self._emit(lines)

    def log_dataset_stats(self, dataset) -> str | None:
        if self.rank != 0:
            return None
        lines = ["[data monitor] dataset chain:"]
        depth, d = 0, dataset
        while d is not None and depth < 16:
            info = [type(d).__name__]
            for attr in ("seq_len", "window_size", "weights", "datasets", "n_docs", "tokens_seen", "docs_seen", "percent_seen"):
                v = getattr(d, attr, None)
                if v is not None and not callable(v):
                    info.append(f"{attr}={v}")
            lines.append("  " * (depth + 1) + " ".join(str(i) for i in info))
            nxt = getattr(d, "dataset", None)
            if nxt is None:
                data = getattr(d, "data", None)
                nxt = data[0] if isinstance(data, (list, tuple)) and data else None
            d, depth = nxt, depth + 1
        return self._emit(lines)
