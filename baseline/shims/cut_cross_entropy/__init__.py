"""Import stand-in for the ``cut_cross_entropy`` package, which cannot be installed offline.

The reference models import ``linear_cross_entropy`` and ``LinearCrossEntropyImpl`` at module load.
The benchmark's reference arm runs the reference's own logits + ``F.cross_entropy`` path
(``enable_cut_cross_entropy=False``), so these names are never called; calling them is an error.
"""
import enum


class LinearCrossEntropyImpl(enum.Enum):
    CCE = "cce"
    TORCH_COMPILE = "torch_compile"


def linear_cross_entropy(*args, **kwargs):
    raise NotImplementedError("cut_cross_entropy is not installed; run with enable_cut_cross_entropy=False")
