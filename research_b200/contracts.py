"""Batch, state and metric containers that cross layer boundaries.

Counterparts of the reference's ``Batch``/``EvalBatch``/``PrefillBatch``/``DecodeBatch`` (src/jaxtitan/batch.py:10-47),
``RngState``/``TrainState``/``HostState`` (state.py:13-76) and ``StepMetrics``/``EvalMetrics`` (metrics.py:10-61).
Arrays are NumPy on the host side of the data pipeline and torch tensors on the device side.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True, slots=True)
class Batch:
    """One fixed-shape language-model microbatch: ``[batch, seq]`` ids, targets and loss mask."""

    input_ids: Any
    target_ids: Any
    loss_mask: Any
    doc_ids: Any | None = None        # first document id of each row
    token_doc_ids: Any | None = None  # document id of every input token (document-aware pipelines)
    # Number of unmasked target tokens of the WHOLE batch.  Set by pipelines that materialise only the rows of this
    # rank (the other rows are zero-filled); consumers that need the global count must use it when it is present.
    mask_count: float | None = None

    @property
    def shape(self) -> tuple[int, ...]:
        return tuple(self.input_ids.shape)


@dataclass(frozen=True, slots=True)
class EvalBatch:
    input_ids: Any
    target_ids: Any
    loss_mask: Any


@dataclass(frozen=True, slots=True)
class PrefillBatch:
    input_ids: Any        # [batch, prompt_len]
    prompt_lengths: Any   # [batch]


@dataclass(frozen=True, slots=True)
class DecodeBatch:
    input_ids: Any        # [batch, 1]
    positions: Any        # [batch]


@dataclass(slots=True)
class RngState:
    """Four independent streams split from the run seed: train, data, eval, sample."""

    train: int
    data: int
    eval: int
    sample: int

    @classmethod
    def from_seed(cls, seed: int) -> "RngState":
        import numpy as np

        keys = np.random.SeedSequence(int(seed)).generate_state(4, dtype=np.uint64)
        return cls(*(int(k) for k in keys))

    def to_json(self) -> dict[str, int]:
        return {"train": self.train, "data": self.data, "eval": self.eval, "sample": self.sample}


@dataclass(slots=True)
class TrainState:
    """Everything a checkpoint's ``train`` item holds."""

    step: int
    tokens_seen: int
    model: Any            # dict name -> fp32 master tensor (this rank's shard)
    opt_state: Any        # nested dict of tensors
    rng: RngState
    schedule_state: Any | None = None
    moe_balance: Any | None = None


@dataclass(slots=True)
class HostState:
    dataset: Any
    last_checkpoint_step: int
    wallclock_start_ns: int
    run_id: str


@dataclass(slots=True)
class StepMetrics:
    """Numerator/denominator style step metrics; every field optional except the two sums."""

    loss_sum: float
    token_count: float
    lr: float | None = None
    grad_norm: float | None = None
    param_norm: float | None = None
    update_norm: float | None = None
    z_loss_sum: float | None = None
    aux_loss: float | None = None
    moe_aux_loss: float | None = None
    microbatch_loss_sums: list[float] | None = None
    microbatch_token_counts: list[float] | None = None
    router: dict[str, Any] = field(default_factory=dict)
    smebu: dict[str, Any] = field(default_factory=dict)
    optimizer_groups: list[dict[str, Any]] = field(default_factory=list)
    router_layers: list[dict[str, Any]] = field(default_factory=list)

    @property
    def loss(self) -> float:
        return self.loss_sum / max(self.token_count, 1.0)


@dataclass(slots=True)
class EvalMetrics:
    loss_sum: float
    token_count: float

    @property
    def loss(self) -> float:
        return self.loss_sum / max(self.token_count, 1.0)
