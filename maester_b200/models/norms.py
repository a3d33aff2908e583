"""Normalisation layer factory (reference: maester/models/norms.py:15-108).

``rmsnorm``, ``compiled_rmsnorm`` and ``fused_rmsnorm`` all resolve to the same module here: there
is a single native RMSNorm kernel (fp32 statistics, one pass forward, two kernels backward), so the
three reference spellings stay valid in job configs without selecting different code.
"""
import torch
import torch.nn as nn

from maester_b200 import ops


class RMSNorm(nn.Module):
    """``x * rsqrt(mean(x²) + eps) * weight`` with fp32 statistics; weight initialised to one."""

    def __init__(self, dim: int, eps: float = 1e-6, compile: bool = False):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, False, residual)

    def fork(self, x: torch.Tensor):
        """(norm(x), x): the second value is the skip connection of the branch that the first one enters."""
        return ops.rmsnorm_fork(x, self.weight, self.eps, False)

    def reset_parameters(self) -> None:
        nn.init.ones_(self.weight)


FusedRMSNorm = RMSNorm


def create_norm(norm_type: str, dim: int, eps: float = 1e-6) -> nn.Module:
    kind = norm_type.lower()
    if kind == "layernorm":
        return nn.LayerNorm(dim, eps=eps, bias=False)
    if kind == "np_layernorm":
        return nn.LayerNorm(dim, eps=eps, elementwise_affine=False, bias=False)
    if kind in ("rmsnorm", "compiled_rmsnorm", "fused_rmsnorm"):
        return RMSNorm(dim, eps=eps)
    raise NotImplementedError(f"Unknown norm_type: '{norm_type}'")
