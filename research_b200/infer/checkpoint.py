"""Checkpoint -> model ready for evaluation or sampling (reference: src/jaxtitan/infer/checkpoint.py:38-126).

Loads the run's resolved config, picks ``latest`` / ``best`` / a step among retained checkpoints, validates the
resume fingerprint, rebuilds the trainer (model + optimizer template) and restores the state into it.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path

from research_b200.config import load_config, load_resolved_config
from research_b200.config.specs import RunSpec
from research_b200.errors import ContractError
from research_b200.optim.build import optimizer_policy_summary
from research_b200.runtime.checkpoint_index import CheckpointRecord, load_checkpoint_index
from research_b200.runtime.resume import build_resume_compat, validate_resume_compat, validate_resume_metadata
from research_b200.runtime.state_io import load_state_tensors
from research_b200.runtime.trainer import Trainer
from research_b200.services.checkpoints import LocalCheckpointService


@dataclass
class InferenceCheckpoint:
    trainer: Trainer
    spec: RunSpec
    record: CheckpointRecord
    path: Path
    runtime_fingerprint: str | None = None

    def describe(self, selector: str | None = None) -> dict:
        """The ``checkpoint`` section of eval and sample artifacts."""

        out = {"step": self.record.step, "path": self.record.checkpoint_path.as_posix(),
               "tokens_seen": self.record.tokens_seen, "runtime_fingerprint": self.runtime_fingerprint}
        return out if selector is None else {"selector": selector, **out}

    @property
    def model(self):
        return self.trainer.result.model


def load_run_spec(run_dir: Path) -> RunSpec:
    resolved = run_dir / "config" / "resolved.json"
    source = run_dir / "config" / "source.toml"
    if resolved.is_file():
        spec = load_resolved_config(resolved)
    elif source.is_file():
        spec = load_config(source)
    else:
        raise ContractError(f"run directory has no config: {run_dir}")
    if spec.run_id != run_dir.name:
        raise ContractError(f"run id {spec.run_id!r} does not match run directory name {run_dir.name!r}")
    return spec


def select_checkpoint(run_dir: Path, selector: str) -> CheckpointRecord:
    index = load_checkpoint_index(run_dir)
    if selector == "latest":
        record = index.latest_record
    elif selector == "best":
        record = index.best_record
        if record is None:
            raise ContractError("no retained checkpoint has an eval loss; cannot select 'best'")
    else:
        try:
            step = int(selector)
        except ValueError as exc:
            raise ContractError(f"--checkpoint must be 'best', 'latest', or a step, got {selector!r}") from exc
        record = index.record_for(step)
        if record is not None and not record.retained:
            raise ContractError(f"checkpoint step {step} is no longer retained")
    if record is None:
        raise ContractError(f"no checkpoint matches {selector!r} in {run_dir}")
    return record


def restore_inference_checkpoint(run_dir: str | Path, selector: str) -> InferenceCheckpoint:
    run_dir = Path(run_dir)
    if not run_dir.is_dir():
        raise ContractError(f"run directory does not exist: {run_dir}")
    spec = load_run_spec(run_dir)
    record = select_checkpoint(run_dir, selector)
    service = LocalCheckpointService(run_dir, is_writer=False)
    trainer = Trainer(spec)
    spec = trainer.spec
    compat = build_resume_compat(spec, optimizer_policy=optimizer_policy_summary(trainer.optimizer_build, trainer.result.metadata),
                                 data_pipeline=trainer.data.describe())
    validate_resume_metadata(service.restore_metadata(record.step), spec, compat=compat)
    restored = service.restore(record.step)
    load_state_tensors(trainer, restored.tensors)
    validate_resume_compat(restored, spec, state_step=trainer.step, state_tokens=trainer.tokens_seen, compat=compat)
    return InferenceCheckpoint(trainer, spec, record, restored.path, compat.runtime_fingerprint)
