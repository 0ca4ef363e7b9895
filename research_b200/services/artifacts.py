"""Run directory layout and the local artifact writer.

Same layout and file formats as the reference (src/jaxtitan/services/artifacts.py:45-176): ``runs/<id>/{config,
metrics,checkpoints,diagnostics,evals,profiles,samples,summaries}``, ``manifest.json``, ``config/source.toml``,
``config/resolved.json``, ``events.jsonl``; every JSON document is canonical (sorted keys, compact separators);
the run directory is created under a temporary name and renamed into place.
"""

from __future__ import annotations

import shutil
from datetime import datetime, timezone
from pathlib import Path
from typing import Any, Mapping
from uuid import uuid4

from research_b200 import __version__
from research_b200.config import load_config, resolved_config_sha256, run_spec_to_json, source_config_sha256
from research_b200.config.canonical import canonical_json, normalize
from research_b200.config.specs import RunManifest, RunSpec
from research_b200.data.manifest import dataset_manifest_summary, validate_dataset_manifest
from research_b200.errors import ContractError

RUN_DIRECTORIES = ("config", "metrics", "checkpoints", "diagnostics", "evals", "profiles", "samples", "summaries")


def utc_now() -> str:
    return datetime.now(timezone.utc).isoformat().replace("+00:00", "Z")


def _data_summary(spec: RunSpec) -> dict[str, Any] | None:
    if spec.data.mode != "prepared" or spec.data.train_manifest is None:
        return None
    manifest = validate_dataset_manifest(spec.data.train_manifest, tokenizer_id=spec.data.tokenizer_id)
    return dataset_manifest_summary(manifest)


class LocalArtifactWriter:
    def __init__(self, run_dir: str | Path) -> None:
        self.run_dir = Path(run_dir)

    @classmethod
    def initialize(cls, *, source_toml: str, resolved: RunSpec, manifest: RunManifest) -> "LocalArtifactWriter":
        run_dir = manifest.run_dir
        if run_dir.exists():
            raise ContractError(f"run directory already exists: {run_dir}")
        run_dir.parent.mkdir(parents=True, exist_ok=True)
        tmp = cls(run_dir.parent / f".{run_dir.name}.tmp-{uuid4().hex}")
        try:
            for name in RUN_DIRECTORIES:
                (tmp.run_dir / name).mkdir(parents=True, exist_ok=False)
            tmp.write_config(source_toml, resolved)
            tmp.write_manifest(manifest)
            tmp.append_event({
                "schema_version": 1, "type": "run_initialized", "run_id": manifest.run_id,
                "created_at": manifest.created_at, "source_config_sha256": manifest.source_config_sha256,
                "resolved_config_sha256": manifest.resolved_config_sha256,
            })
            tmp.run_dir.replace(run_dir)
        except Exception:
            shutil.rmtree(tmp.run_dir, ignore_errors=True)
            raise
        return cls(run_dir)

    # -- writers -----------------------------------------------------------------------------------
    def write_config(self, source_toml: str, resolved: RunSpec) -> None:
        (self.run_dir / "config" / "source.toml").write_text(source_toml)
        (self.run_dir / "config" / "resolved.json").write_text(run_spec_to_json(resolved) + "\n")

    def write_manifest(self, manifest: RunManifest) -> None:
        row = normalize(manifest)
        row.pop("run_dir", None)
        self._write_json(self.run_dir / "manifest.json", row)

    def append_event(self, event: Mapping[str, Any]) -> None:
        self._append_jsonl(self.run_dir / "events.jsonl", event)

    def append_train_metrics(self, row: Mapping[str, Any]) -> None:
        self._append_jsonl(self.run_dir / "metrics" / "train.jsonl", row)

    def append_eval_metrics(self, row: Mapping[str, Any]) -> None:
        self._append_jsonl(self.run_dir / "metrics" / "eval.jsonl", row)

    def write_runtime_diagnostics(self, diagnostics: Mapping[str, Any]) -> None:
        self._write_json(self.run_dir / "diagnostics" / "runtime.json", diagnostics)

    def write_profiling_diagnostics(self, diagnostics: Mapping[str, Any]) -> None:
        self._write_json(self.run_dir / "diagnostics" / "profiling.json", diagnostics)

    def write_wandb_metadata(self, metadata: Mapping[str, Any]) -> None:
        self._write_json(self.run_dir / "diagnostics" / "wandb.json", metadata)

    def write_checkpoint_index(self, index: Mapping[str, Any]) -> None:
        self._write_json(self.run_dir / "checkpoints" / "index.json", index)

    def write_checkpoint_eval(self, step: int, payload: Mapping[str, Any]) -> Path:
        path = self.run_dir / "evals" / "checkpoints" / f"{step:06d}.json"
        path.parent.mkdir(parents=True, exist_ok=True)
        self._write_json(path, payload)
        return path

    def append_checkpoint_sample(self, step: int, row: Mapping[str, Any]) -> Path:
        path = self.run_dir / "samples" / "checkpoints" / f"{step:06d}.jsonl"
        path.parent.mkdir(parents=True, exist_ok=True)
        self._append_jsonl(path, row)
        return path

    def write_summary(self, summary: Mapping[str, Any]) -> None:
        self._write_json(self.run_dir / "summaries" / "final.json", summary)

    def close(self) -> None:
        return None

    def _write_json(self, path: Path, value: Any) -> None:
        path.write_text(canonical_json(value) + "\n")

    def _append_jsonl(self, path: Path, row: Mapping[str, Any]) -> None:
        with path.open("a") as handle:
            handle.write(canonical_json(dict(row)) + "\n")


class NullArtifactWriter(LocalArtifactWriter):
    """Writer for non-zero ranks: artifacts are host-global and written by rank 0 only."""

    def _write_json(self, path: Path, value: Any) -> None:
        return None

    def _append_jsonl(self, path: Path, row: Mapping[str, Any]) -> None:
        return None


def initialize_run(config_path: str | Path) -> RunManifest:
    """Create the run directory skeleton for a config (reference: services/artifacts.py:45-78)."""

    source_path = Path(config_path)
    spec = load_config(source_path)
    manifest = RunManifest(
        schema_version=1, artifact_layout_version=1, run_id=spec.run_id, created_at=utc_now(),
        source_config_path=source_path, source_config_sha256=source_config_sha256(source_path),
        resolved_config_sha256=resolved_config_sha256(spec), package={"name": "research_b200", "version": __version__},
        directories={name: name for name in RUN_DIRECTORIES}, run_dir=spec.dirs.run_dir, data=_data_summary(spec),
    )
    LocalArtifactWriter.initialize(source_toml=source_path.read_text(), resolved=spec, manifest=manifest)
    return manifest


def build_artifact_writer(spec: RunSpec, run_dir: str | Path, *, is_writer: bool = True,
                          resume: bool = False) -> LocalArtifactWriter:
    """Local writer, mirrored to W&B when ``[artifacts].wandb_enabled`` (reference: services/wandb.py:242-273).
    With ``resume`` the mirror continues the W&B run named in ``diagnostics/wandb.json``."""

    if not is_writer:
        return NullArtifactWriter(run_dir)
    if spec.artifacts.wandb_enabled:
        from research_b200.services.wandb import WandbMirroredWriter

        return WandbMirroredWriter(spec, run_dir, resume=resume)
    return LocalArtifactWriter(run_dir)
