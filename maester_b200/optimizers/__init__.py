from maester_b200.optimizers.adamw import FusedAdamW  # noqa: F401
from maester_b200.optimizers.container import OptimizersContainer, build_optimizers  # noqa: F401

try:
    from maester_b200.optimizers.muon import Muon, MuonDDP  # noqa: F401
except ImportError:  # pragma: no cover
    pass
