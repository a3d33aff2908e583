from maester_b200.optimizers.adamw import FusedAdamW  # noqa: F401
