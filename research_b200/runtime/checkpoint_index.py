"""``checkpoints/index.json``: one record per checkpoint, latest / best-by-eval-loss, retained flags refreshed
from the directories on disk (reference: src/jaxtitan/runtime/checkpoint_index.py:14-141)."""

from __future__ import annotations

import json
from dataclasses import dataclass, replace
from pathlib import Path
from typing import Any, Mapping

from research_b200.config.canonical import normalize
from research_b200.errors import ContractError

CHECKPOINT_INDEX_SCHEMA_VERSION = 1


@dataclass(frozen=True, slots=True)
class CheckpointRecord:
    step: int
    tokens_seen: int
    checkpoint_path: Path
    reason: str
    train_loss: float
    eval_loss: float | None = None
    retained: bool = True

    def __post_init__(self) -> None:
        object.__setattr__(self, "checkpoint_path", Path(self.checkpoint_path))
        if self.step < 0:
            raise ContractError(f"checkpoint index step must be non-negative, got {self.step}")
        if self.tokens_seen < 0:
            raise ContractError(f"checkpoint index tokens_seen must be non-negative, got {self.tokens_seen}")
        if not self.reason:
            raise ContractError("checkpoint index reason must be non-empty")


@dataclass(frozen=True, slots=True)
class CheckpointIndex:
    records: tuple[CheckpointRecord, ...] = ()
    schema_version: int = CHECKPOINT_INDEX_SCHEMA_VERSION

    def __post_init__(self) -> None:
        if self.schema_version != CHECKPOINT_INDEX_SCHEMA_VERSION:
            raise ContractError(
                f"checkpoint index schema_version must be {CHECKPOINT_INDEX_SCHEMA_VERSION}, got {self.schema_version}"
            )
        object.__setattr__(self, "records", tuple(sorted(self.records, key=lambda r: r.step)))

    @property
    def retained_records(self) -> tuple[CheckpointRecord, ...]:
        return tuple(r for r in self.records if r.retained)

    @property
    def latest_record(self) -> CheckpointRecord | None:
        kept = self.retained_records
        return max(kept, key=lambda r: r.step) if kept else None

    @property
    def best_record(self) -> CheckpointRecord | None:
        scored = [r for r in self.retained_records if r.eval_loss is not None]
        return min(scored, key=lambda r: (r.eval_loss, r.step)) if scored else None

    def protected_steps(self) -> set[int]:
        return {r.step for r in (self.latest_record, self.best_record) if r is not None}

    def record_for(self, step: int) -> CheckpointRecord | None:
        for r in self.records:
            if r.step == step:
                return r
        return None

    def to_dict(self) -> dict[str, Any]:
        latest, best = self.latest_record, self.best_record
        return {
            "schema_version": self.schema_version,
            "latest_step": None if latest is None else latest.step,
            "latest_checkpoint_path": None if latest is None else latest.checkpoint_path.as_posix(),
            "best_eval_step": None if best is None else best.step,
            "best_eval_loss": None if best is None else best.eval_loss,
            "best_checkpoint_path": None if best is None else best.checkpoint_path.as_posix(),
            "records": [normalize(r) for r in self.records],
        }


def _record_from(raw: Any) -> CheckpointRecord:
    if not isinstance(raw, Mapping):
        raise ContractError("checkpoint index record must be an object")
    try:
        return CheckpointRecord(
            step=int(raw["step"]), tokens_seen=int(raw["tokens_seen"]), checkpoint_path=Path(raw["checkpoint_path"]),
            reason=str(raw["reason"]), train_loss=float(raw["train_loss"]),
            eval_loss=None if raw.get("eval_loss") is None else float(raw["eval_loss"]),
            retained=bool(raw.get("retained", True)))
    except (KeyError, TypeError, ValueError) as exc:
        raise ContractError(f"checkpoint index record is malformed: {exc}") from exc


def refresh_checkpoint_index(index: CheckpointIndex, run_dir: str | Path) -> CheckpointIndex:
    run_dir = Path(run_dir)
    return CheckpointIndex(tuple(replace(r, retained=(run_dir / r.checkpoint_path).is_dir()) for r in index.records))


def load_checkpoint_index(run_dir: str | Path) -> CheckpointIndex:
    run_dir = Path(run_dir)
    path = run_dir / "checkpoints" / "index.json"
    if not path.exists():
        return CheckpointIndex()
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as exc:
        raise ContractError(f"failed to parse checkpoint index {path}: {exc}") from exc
    if not isinstance(raw, Mapping):
        raise ContractError("checkpoint index must be an object")
    records = raw.get("records", [])
    if not isinstance(records, list):
        raise ContractError("checkpoint index records must be a list")
    index = CheckpointIndex(tuple(_record_from(r) for r in records),
                            int(raw.get("schema_version", CHECKPOINT_INDEX_SCHEMA_VERSION)))
    return refresh_checkpoint_index(index, run_dir)


def record_checkpoint(index: CheckpointIndex, run_dir: str | Path, *, step: int, tokens_seen: int,
                      checkpoint_path: str | Path, reason: str, train_loss: float,
                      eval_loss: float | None) -> CheckpointIndex:
    run_dir = Path(run_dir)
    path = Path(checkpoint_path)
    if not (path.parts and path.parts[0] == "checkpoints" and not path.is_absolute()):
        try:
            path = path.resolve().relative_to(run_dir.resolve())
        except ValueError as exc:
            raise ContractError(f"checkpoint path {checkpoint_path} is outside run directory {run_dir}") from exc
    rec = CheckpointRecord(step, tokens_seen, path, reason, train_loss, eval_loss, (run_dir / path).is_dir())
    others = tuple(r for r in index.records if r.step != step)
    return refresh_checkpoint_index(CheckpointIndex(others + (rec,)), run_dir)
