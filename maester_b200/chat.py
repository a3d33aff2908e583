"""Chat engine over a training checkpoint: model loading, prompt formats, streaming generation.

Back end of ``scripts/chat_tui.py`` (reference: scripts/chat_tui.py — prompt formatters :102-133,
checkpoint loading :185-294, layer-streaming runner for models larger than the GPU :296-394,
generation :396-517).  No KV cache: every token recomputes the (windowed) prefix, like the
reference tool; the point is inspecting checkpoints, not serving.
"""
from __future__ import annotations

import copy
import json
import threading
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Iterator

import torch
import torch.nn as nn

from maester_b200.generate import sample


# ----------------------------------------------------------------------------------------- prompt formats
@dataclass
class Message:
    role: str
    content: str


class ChatMLFormatter:
    """``<|im_start|>role\\ncontent<|im_end|>`` turns; the prompt ends with an open assistant turn."""
    name = "chatml"

    def __init__(self, im_start: str = "<|im_start|>", im_end: str = "<|im_end|>", system: str | None = None):
        self.im_start, self.im_end, self.system = im_start, im_end, system

    def render(self, history: list[Message]) -> str:
        parts = []
        if self.system:
            parts.append(f"{self.im_start}system\n{self.system}{self.im_end}\n")
        for m in history:
            parts.append(f"{self.im_start}{m.role}\n{m.content}{self.im_end}\n")
        parts.append(f"{self.im_start}assistant\n")
        return "".join(parts)

    def stop_strings(self) -> list[str]:
        return [self.im_end, self.im_start]


class PlainFormatter:
    """``User: ... / Assistant: ...`` transcript for base models."""
    name = "plain"

    def render(self, history: list[Message]) -> str:
        names = {"user": "User", "assistant": "Assistant", "system": "System"}
        lines = [f"{names.get(m.role, m.role)}: {m.content}" for m in history]
        return "\n".join(lines) + "\nAssistant:"

    def stop_strings(self) -> list[str]:
        return ["\nUser:", "\nSystem:"]


class RawFormatter:
    """Pure continuation: the prompt is the concatenation of everything said so far."""
    name = "raw"

    def render(self, history: list[Message]) -> str:
        return "".join(m.content for m in history)

    def stop_strings(self) -> list[str]:
        return []


FORMATTERS = {"chatml": ChatMLFormatter, "plain": PlainFormatter, "raw": RawFormatter}


# ----------------------------------------------------------------------------------------- model loading
def load_model_from_dcp(checkpoint_dir: str, model_name: str | None = None, flavor: str | None = None,
                        device: str | torch.device = "cpu", dtype: torch.dtype = torch.bfloat16, seq_len: int | None = None):
    """Build the model named by the job config (or the flags) and fill it from the checkpoint's
    ``model.*`` tensors.  Returns (model, model_args)."""
    from maester_b200.convert.io import find_job_config, read_dcp_model
    from maester_b200.models import model_name_to_cls, models_config

    job = find_job_config(checkpoint_dir) or {}
    model_name = model_name or job.get("model_name")
    flavor = flavor or job.get("flavor")
    if not model_name or not flavor:
        raise ValueError("pass model_name and flavor: no job config.json was found next to the checkpoint")
    args = copy.deepcopy(models_config[model_name][flavor])
    sd = read_dcp_model(checkpoint_dir)
    if getattr(args, "vocab_size", 0) <= 0:
        args.vocab_size = sd["tok_embeddings.weight"].shape[0]
    if seq_len or job.get("seq_len"):
        args.max_seq_len = int(seq_len or job["seq_len"])
    if hasattr(args, "norm_type") and job.get("norm_type"):
        args.norm_type = job["norm_type"]
    with torch.device("meta"):
        model = model_name_to_cls[model_name].from_model_args(args)
    model.to_empty(device="cpu")
    if hasattr(model, "init_weights"):
        model.init_weights()  # rebuilds non-persistent buffers (RoPE tables)
    missing, unexpected = model.load_state_dict({k: v for k, v in sd.items()}, strict=False)
    real_missing = [k for k in missing if not any(s in k for s in ("rope", "inv_freq", "tokens_per_expert"))]
    if real_missing or unexpected:
        raise KeyError(f"checkpoint does not match {model_name}/{flavor}: missing {real_missing[:5]}, unexpected {unexpected[:5]}")
    model = model.to(dtype=dtype if torch.device(device).type == "cuda" else torch.float32).to(device).eval()
    return model, args


# ----------------------------------------------------------------------------------------- layer streaming
class LayerStreamingRunner(nn.Module):
    """Run a model whose transformer blocks do not fit on the GPU: blocks stay in pinned host memory
    and are copied to the device ``block`` layers at a time on a side stream while the previous
    group computes.  Embedding, final norm and head stay resident."""

    def __init__(self, model: nn.Module, device: torch.device, block: int = 4):
        super().__init__()
        self.model, self.device, self.block = model, torch.device(device), block
        layers = model.layers if hasattr(model, "layers") else model.model.layers
        self.layer_list = list(layers.values()) if isinstance(layers, nn.ModuleDict) else list(layers)
        self.resident = [m for n, m in model.named_children() if m is not layers and n != "model"]
        for m in self.resident:
            m.to(self.device)
        for n, b in model.named_buffers(recurse=False):
            setattr(model, n, b.to(self.device))
        for lyr in self.layer_list:
            for p in lyr.parameters():
                p.data = p.data.pin_memory() if self.device.type == "cuda" else p.data
        self.copy_stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None

    def _fetch(self, group: list[nn.Module]) -> list[tuple[nn.Parameter, torch.Tensor]]:
        moved = []
        ctx = torch.cuda.stream(self.copy_stream) if self.copy_stream is not None else _Null()
        with ctx:
            for lyr in group:
                for p in lyr.parameters():
                    host = p.data
                    p.data = host.to(self.device, non_blocking=True)
                    moved.append((p, host))
        return moved

    @staticmethod
    def _release(moved) -> None:
        for p, host in moved:
            p.data = host

    def run_layers(self, fn: Callable[[nn.Module], None]) -> None:
        """Call ``fn(layer)`` for every block in order, with the block's weights on the device."""
        groups = [self.layer_list[i:i + self.block] for i in range(0, len(self.layer_list), self.block)]
        nxt = self._fetch(groups[0]) if groups else []
        for gi, group in enumerate(groups):
            cur = nxt
            if self.copy_stream is not None:
                torch.cuda.current_stream(self.device).wait_stream(self.copy_stream)
            nxt = self._fetch(groups[gi + 1]) if gi + 1 < len(groups) else []
            for lyr in group:
                fn(lyr)
            if self.copy_stream is not None:
                self.copy_stream.wait_stream(torch.cuda.current_stream(self.device))
            self._release(cur)

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """Works for models whose forward is ``embed -> blocks(h, pos, inv_freq, rope_cs, doc) -> norm -> head``
        and expose ``forward_embed`` / ``forward_head`` hooks; otherwise falls back to moving the whole model."""
        m = self.model
        if not (hasattr(m, "forward_embed") and hasattr(m, "forward_head")):
            raise NotImplementedError("layer streaming needs forward_embed/forward_head on the model")
        state = m.forward_embed(tokens.to(self.device))
        self.run_layers(lambda lyr: state.__setitem__("h", lyr(state["h"], *state["args"])))
        return m.forward_head(state["h"])


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


# ----------------------------------------------------------------------------------------- generation
@dataclass
class GenerationConfig:
    max_new_tokens: int = 256
    temperature: float = 0.7
    top_k: int | None = 50
    window: int = 4096


@dataclass
class ChatSession:
    model: nn.Module
    tokenizer: object
    formatter: object
    cfg: GenerationConfig = field(default_factory=GenerationConfig)
    history: list[Message] = field(default_factory=list)
    _stop: threading.Event = field(default_factory=threading.Event)

    def reset(self) -> None:
        self.history.clear()

    def stop(self) -> None:
        self._stop.set()

    def _device(self) -> torch.device:
        return getattr(self.model, "device", None) or next(self.model.parameters()).device

    @torch.no_grad()
    def stream(self, user_text: str) -> Iterator[str]:
        """Yield text pieces of the assistant's reply; the finished reply is appended to the history."""
        self._stop.clear()
        self.history.append(Message("user", user_text))
        prompt = self.formatter.render(self.history)
        ids = self.tokenizer.encode(prompt)
        seq = torch.tensor([ids], device=self._device(), dtype=torch.int64)
        eos = {i for i in (getattr(self.tokenizer, "eos_token_id", None),) if i is not None}
        new_ids: list[int] = []
        emitted = ""
        stops = self.formatter.stop_strings()
        for _ in range(self.cfg.max_new_tokens):
            if self._stop.is_set():
                break
            out = self.model(seq[:, -self.cfg.window:])
            logits = out.logits if hasattr(out, "logits") else out
            nxt, _ = sample(logits[:, -1], self.cfg.temperature, self.cfg.top_k)
            tok = int(nxt)
            if tok in eos:
                break
            new_ids.append(tok)
            seq = torch.cat([seq, nxt], dim=1)
            text = self.tokenizer.decode(new_ids)
            cut = min([text.find(s) for s in stops if s and s in text], default=-1)
            if cut >= 0:
                text = text[:cut]
            if len(text) > len(emitted) and not text.endswith("�"):
                yield text[len(emitted):]
                emitted = text
            if cut >= 0:
                break
        self.history.append(Message("assistant", emitted))

    def save_transcript(self, path: str) -> None:
        Path(path).write_text(json.dumps([m.__dict__ for m in self.history], indent=2, ensure_ascii=False))
