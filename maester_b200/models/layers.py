"""Building blocks shared by the model families: bias-free Linear / Embedding modules whose
parameters keep the reference's fully-qualified names, and fused views over adjacent weights.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from maester_b200 import ops


class Linear(nn.Module):
    """``y = x Wᵀ`` (+ optional bias); weight is [out_features, in_features]."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        y = ops.linear(x, self.weight, residual)
        if self.bias is not None:
            y = y + self.bias
        return y

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}"


class Embedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.weight = nn.Parameter(torch.empty(num_embeddings, embedding_dim))

    def forward(self, tokens: torch.Tensor, scale: float | None = None) -> torch.Tensor:
        return ops.embedding(tokens, self.weight, scale)


def _adjacent(a: torch.Tensor, b: torch.Tensor) -> bool:
    return (
        a.is_contiguous() and b.is_contiguous() and a.dtype == b.dtype and a.device == b.device
        and a.untyped_storage().data_ptr() == b.untyped_storage().data_ptr()
        and a.storage_offset() + a.numel() == b.storage_offset()
    )


class FusedWeight:
    """Row-wise concatenation of several [out_i, in] weights, presented as one [sum out_i, in] matrix.

    When the parameters sit back to back in one flat buffer (the layout the sharding runtime
    creates) the fused matrix is a zero-copy view whose ``main_grad`` is the matching view of the
    flat fp32 gradient buffer, so one GEMM serves all projections and its wgrad accumulates in
    place.  Otherwise it is ``torch.cat`` of the parameters (ordinary autograd).
    """

    def __init__(self, owners: list[nn.Module], attr: str = "weight"):
        # modules, not Parameters: the sharding runtime replaces Parameter objects after construction
        self.owners, self.attr = owners, attr
        self._view = None
        self._key = None

    def get(self) -> torch.Tensor:
        ps = [getattr(m, self.attr) for m in self.owners]
        grads = [getattr(p, "main_grad", None) for p in ps]
        # the view's gradient reaches the flat buffer only through the native GEMM's ``main_grad`` epilogue; on the
        # plain-PyTorch path (CPU, fp32 compute) autograd must see the parameters themselves
        native = ps[0].is_cuda and ps[0].dtype == torch.bfloat16
        flat_ok = native and all(g is not None for g in grads) and all(
            _adjacent(ps[i].data, ps[i + 1].data) and _adjacent(grads[i], grads[i + 1]) for i in range(len(ps) - 1)
        )
        if not flat_ok:
            return torch.cat(list(ps), dim=0)
        key = (ps[0].data_ptr(), grads[0].data_ptr())
        if self._view is None or self._key != key:
            rows = sum(p.shape[0] for p in ps)
            cols = ps[0].shape[1]
            with torch.no_grad():
                w = torch.as_strided(ps[0].data, (rows, cols), (cols, 1))
                g = torch.as_strided(grads[0], (rows, cols), (cols, 1))
            w.requires_grad_(True)
            w.main_grad = g
            self._view, self._key = w, key
        return self._view
