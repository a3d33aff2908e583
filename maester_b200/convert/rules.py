"""Table-driven, invertible key/tensor mapping used by every model family."""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Callable

import torch

Arch = dict
Transform = Callable[[torch.Tensor, Arch], torch.Tensor]


def _regex(pattern: str) -> re.Pattern:
    esc = re.escape(pattern).replace(r"\{L\}", r"(?P<L>\d+)").replace(r"\{E\}", r"(?P<E>\d+)")
    return re.compile("^" + esc + "$")


@dataclass
class Rule:
    """One HF tensor <-> one native tensor.  ``native=None`` drops the HF tensor on import."""
    hf: str
    native: str | None
    fwd: Transform | None = None   # HF -> native
    inv: Transform | None = None   # native -> HF


@dataclass
class Fuse:
    """Several HF tensors <-> one native tensor, concatenated along dim 0 in the listed order."""
    hf: list[str]
    native: str
    sizes: Callable[[Arch], list[int]]
    fwd: list[Transform | None] | None = None   # per part, applied before concatenation
    inv: list[Transform | None] | None = None   # per part, applied after splitting


@dataclass
class Stack:
    """Per-expert HF matrices ``[out, in]`` <-> one native tensor ``[E, in, out]``."""
    hf: str        # contains {E}
    native: str


@dataclass
class FamilySpec:
    name: str
    entries: list
    strip_prefixes: tuple[str, ...] = ()          # leading HF prefixes removed before matching
    ignore: tuple[str, ...] = ()                  # regexes of HF keys that have no counterpart
    hf_prefix: str = ""                           # prepended to produced HF keys (after rules)
    _hf_index: list = field(default_factory=list, repr=False)

    def __post_init__(self):
        self._hf_index = []
        for e in self.entries:
            pats = e.hf if isinstance(e, Fuse) else [e.hf]
            for i, p in enumerate(pats):
                self._hf_index.append((_regex(p), e, i))
        self._native_index = [(_regex(e.native), e) for e in self.entries if e.native is not None]
        self._ignore = [re.compile(p) for p in self.ignore]


def _fmt(pattern: str, groups: dict) -> str:
    out = pattern
    for k, v in groups.items():
        if v is not None:
            out = out.replace("{" + k + "}", v)
    return out


def _normalise(key: str, prefixes: tuple[str, ...]) -> str:
    for p in prefixes:
        if key.startswith(p):
            return key[len(p):]
    return key


def to_native(spec: FamilySpec, hf_sd: dict[str, torch.Tensor], arch: Arch, strict: bool = True) -> dict[str, torch.Tensor]:
    out: dict[str, torch.Tensor] = {}
    fuse_parts: dict[str, dict[int, torch.Tensor]] = {}
    fuse_entry: dict[str, Fuse] = {}
    stack_parts: dict[str, dict[int, torch.Tensor]] = {}
    unknown = []
    for raw_key, t in hf_sd.items():
        key = _normalise(raw_key, spec.strip_prefixes)
        if any(r.search(key) for r in spec._ignore):
            continue
        for rx, e, part in spec._hf_index:
            m = rx.match(key)
            if not m:
                continue
            g = m.groupdict()
            if isinstance(e, Rule):
                if e.native is not None:
                    out[_fmt(e.native, g)] = e.fwd(t, arch) if e.fwd else t
            elif isinstance(e, Fuse):
                nk = _fmt(e.native, g)
                f = e.fwd[part] if e.fwd else None
                fuse_parts.setdefault(nk, {})[part] = f(t, arch) if f else t
                fuse_entry[nk] = e
            else:
                nk = _fmt(e.native, {"L": g.get("L")})
                stack_parts.setdefault(nk, {})[int(g["E"])] = t
            break
        else:
            unknown.append(raw_key)
    for nk, parts in fuse_parts.items():
        e = fuse_entry[nk]
        if len(parts) != len(e.hf):
            raise KeyError(f"{nk}: found {len(parts)} of {len(e.hf)} tensors to fuse")
        out[nk] = torch.cat([parts[i] for i in range(len(e.hf))], dim=0)
    for nk, parts in stack_parts.items():
        n = max(parts) + 1
        if len(parts) != n:
            raise KeyError(f"{nk}: experts missing ({len(parts)} of {n})")
        out[nk] = torch.stack([parts[i].t() for i in range(n)]).contiguous()
    if unknown and strict:
        raise KeyError(f"{spec.name}: no rule for HF keys {unknown[:8]}{' ...' if len(unknown) > 8 else ''}")
    return out


def to_hf(spec: FamilySpec, native_sd: dict[str, torch.Tensor], arch: Arch, strict: bool = True) -> dict[str, torch.Tensor]:
    out: dict[str, torch.Tensor] = {}
    unknown = []
    for key, t in native_sd.items():
        for rx, e in spec._native_index:
            m = rx.match(key)
            if not m:
                continue
            g = m.groupdict()
            if isinstance(e, Rule):
                out[spec.hf_prefix + _fmt(e.hf, g)] = e.inv(t, arch) if e.inv else t
            elif isinstance(e, Fuse):
                sizes = e.sizes(arch)
                assert sum(sizes) == t.shape[0], f"{key}: rows {t.shape[0]} != {sizes}"
                for i, piece in enumerate(torch.split(t, sizes, dim=0)):
                    f = e.inv[i] if e.inv else None
                    out[spec.hf_prefix + _fmt(e.hf[i], g)] = (f(piece, arch) if f else piece).contiguous()
            else:
                for ei in range(t.shape[0]):
                    out[spec.hf_prefix + _fmt(e.hf, {**g, "E": str(ei)})] = t[ei].t().contiguous()
            break
        else:
            unknown.append(key)
    if unknown and strict:
        raise KeyError(f"{spec.name}: no rule for native keys {unknown[:8]}{' ...' if len(unknown) > 8 else ''}")
    return out


# ---------------------------------------------------------------------------------------------------
# transforms
def rope_rows_half_to_interleaved(n_heads_key: str) -> Transform:
    """HF stores rotary rows as [first halves | second halves] per head (rotate-half convention); the
    Llama model here rotates adjacent pairs.  Reorder the output rows of a projection accordingly."""
    def f(w: torch.Tensor, arch: Arch) -> torch.Tensor:
        h = arch[n_heads_key]
        rows, cols = w.shape
        return w.contiguous().view(h, 2, rows // h // 2, cols).transpose(1, 2).reshape(rows, cols)
    return f


def rope_rows_interleaved_to_half(n_heads_key: str) -> Transform:
    def f(w: torch.Tensor, arch: Arch) -> torch.Tensor:
        h = arch[n_heads_key]
        rows, cols = w.shape
        return w.contiguous().view(h, rows // h // 2, 2, cols).transpose(1, 2).reshape(rows, cols)
    return f
