"""Learning-rate schedules as plain functions of the step. The FSDP engine reads ``AdamWConfig.lr`` at every unit's
update, so a training loop sets ``trainer.engine.opt.lr = schedule(step)`` before the step.

    sched = warmup_cosine(peak=3e-4, warmup=2000, total=100_000, floor=3e-5)
    for step in range(total):
        trainer.engine.opt.lr = sched(step)
        trainer.step(tokens, targets)
"""
from __future__ import annotations

import math
from typing import Callable


def warmup_cosine(peak: float, warmup: int, total: int, floor: float = 0.0) -> Callable[[int], float]:
    """Linear from ``peak / warmup`` to ``peak`` over ``warmup`` steps, then half a cosine down to ``floor`` at ``total``."""
    if warmup < 0 or total <= warmup:
        raise ValueError("need 0 <= warmup < total")

    def at(step: int) -> float:
        if step < warmup:
            return peak * (step + 1) / warmup
        t = min(1.0, (step - warmup) / (total - warmup))
        return floor + 0.5 * (peak - floor) * (1.0 + math.cos(math.pi * t))

    return at


def warmup_linear(peak: float, warmup: int, total: int, floor: float = 0.0) -> Callable[[int], float]:
    if warmup < 0 or total <= warmup:
        raise ValueError("need 0 <= warmup < total")

    def at(step: int) -> float:
        if step < warmup:
            return peak * (step + 1) / warmup
        t = min(1.0, (step - warmup) / (total - warmup))
        return peak + (floor - peak) * t

    return at


def warmup_stable_decay(peak: float, warmup: int, stable_until: int, total: int, floor: float = 0.0) -> Callable[[int], float]:
    """Warm-up, a plateau at ``peak`` until ``stable_until``, then linear decay to ``floor`` at ``total``."""
    if not (0 <= warmup <= stable_until < total):
        raise ValueError("need 0 <= warmup <= stable_until < total")

    def at(step: int) -> float:
        if step < warmup:
            return peak * (step + 1) / warmup
        if step < stable_until:
            return peak
        t = min(1.0, (step - stable_until) / (total - stable_until))
        return peak + (floor - peak) * t

    return at
