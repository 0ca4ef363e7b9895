"""Learning-rate schedules: constant, cosine, warmup-stable-decay, all with linear warm-up ``(count+1)/warmup``.

Evaluated at the optimizer's *old* step count, as in the reference (src/jaxtitan/optim/build.py:1112-1223,
steps/train.py:227).
"""

from __future__ import annotations

import math
from typing import Callable

from research_b200.config.specs import ScheduleSpec
from research_b200.errors import ContractError


def _warmup(count: float, peak: float, warmup: int) -> float:
    if warmup == 0:
        return peak
    return peak * min((count + 1.0) / warmup, 1.0)


def _cosine(count: float, peak: float, floor: float, decay_steps: int) -> float:
    if decay_steps == 1:
        return floor
    progress = min(max(count / (decay_steps - 1), 0.0), 1.0)
    return floor + (peak - floor) * 0.5 * (1.0 + math.cos(math.pi * progress))


def build_lr_schedule(spec: ScheduleSpec) -> Callable[[int], float]:
    peak, warmup = float(spec.peak_lr), int(spec.warmup_steps)
    floor = peak * float(spec.min_lr_ratio)
    if spec.name == "constant":
        return lambda count: _warmup(float(count), peak, warmup) if count < warmup else peak
    if spec.total_steps is None:
        raise ContractError(f"optimizer.schedule.total_steps is required for the {spec.name} schedule at runtime")
    total = int(spec.total_steps)
    if spec.name == "cosine":
        if total <= warmup:
            raise ContractError(
                f"cosine schedule requires total_steps > warmup_steps, got warmup_steps={warmup}, total_steps={total}"
            )
        decay_steps = total - warmup

        def cosine(count: int) -> float:
            c = float(count)
            return _warmup(c, peak, warmup) if c < warmup else _cosine(c - warmup, peak, floor, decay_steps)

        return cosine
    if spec.name == "wsd":
        stable = int(spec.stable_steps) if spec.stable_steps is not None else max(total - warmup - max(total // 10, 1), 0)
        decay_start = warmup + stable
        if total <= decay_start:
            raise ContractError(
                "wsd schedule requires total_steps > warmup_steps + stable_steps, "
                f"got warmup_steps={warmup}, stable_steps={stable}, total_steps={total}"
            )
        decay_steps = total - decay_start

        def wsd(count: int) -> float:
            c = float(count)
            if c < warmup:
                return _warmup(c, peak, warmup)
            if c < decay_start:
                return peak
            return _cosine(c - decay_start, peak, floor, decay_steps)

        return wsd
    raise ContractError(f"unsupported schedule {spec.name!r}")
