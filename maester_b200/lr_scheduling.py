"""Learning-rate schedules as LambdaLR multipliers (reference: maester/lr_scheduling.py:12-53).

Behaviour kept on purpose: the cosine schedule has a floor of ``eta_min`` = 0.1 and its phase is
``step / total`` (warm-up steps are not subtracted); warm-up returns ``(step + 1) / warmup``.
"""
import math

from torch.optim.lr_scheduler import LambdaLR


def linear_warmup_cosine(warmup_steps: int, total_steps: int, eta_min: float = 0.1):
    def mult(step: int) -> float:
        if step < warmup_steps:
            return (step + 1) / max(1, warmup_steps)
        cos = 0.5 * (1.0 + math.cos(math.pi * step / total_steps))
        return max(0.0, eta_min + (1.0 - eta_min) * cos)

    return mult


def linear_warmup_constant_sqrt_decay(warmup_steps: int, total_steps: int, cooldown_steps: int):
    """Warm-up, stable plateau, then a ``1 - sqrt`` cooldown over the last ``cooldown_steps``."""
    start_decay = total_steps - cooldown_steps

    def mult(step: int) -> float:
        if step < warmup_steps:
            return (step + 1) / max(1, warmup_steps)
        if step < start_decay:
            return 1.0
        return 1.0 - math.sqrt((step - start_decay) / cooldown_steps)

    return mult


def constant():
    return lambda step: 1.0


def get_lr_scheduler(optimizer, cfg) -> LambdaLR:
    name = cfg.scheduler
    if name == "constant":
        fn = constant()
    elif name == "linear_warmup_cosine":
        fn = linear_warmup_cosine(cfg.warmup_steps, cfg.train_num_steps)
    elif name == "linear_warmup_constant_sqrt_decay":
        fn = linear_warmup_constant_sqrt_decay(cfg.warmup_steps, cfg.train_num_steps, cfg.cooldown_steps)
    else:
        raise ValueError(f"LR scheduler '{name}' is not supported")
    return LambdaLR(optimizer, lr_lambda=fn)
