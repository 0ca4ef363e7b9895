"""Model output containers (reference: src/jaxtitan/models/output.py:8-56)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any


@dataclass(frozen=True)
class AuxLoss:
    name: str
    value: Any    # scalar tensor
    weight: float


@dataclass(frozen=True)
class RouterStats:
    name: str
    layer_index: int
    expert_counts: Any       # [E] fp32
    importance: Any          # [E] fp32
    total_assignments: Any
    load_min: Any
    load_max: Any
    load_mean: Any
    max_vio: Any
    load_entropy: Any
    dropped: Any = None      # assignments dropped by the capacity limit


@dataclass(frozen=True)
class ModelOutput:
    logits: Any
    aux_losses: tuple[AuxLoss, ...] = ()
    aux_metrics: tuple[Any, ...] = ()
    router_stats: tuple[RouterStats, ...] = ()
