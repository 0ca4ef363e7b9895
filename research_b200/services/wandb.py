"""Optional Weights & Biases mirror of the local artifacts (reference: src/jaxtitan/services/wandb.py:60-349).

Local files are always written first.  The first mirrored call that fails writes a ``wandb_failed`` event, raises a
:class:`ContractError` (which ends the run) and switches the mirror off, so the ``training_failed`` event that follows
is still written locally.  A new run takes the deterministic id ``<run_id>-<first 16 hex of the resolved config
sha256>`` with ``resume="allow"``; a resumed run reads the id back from ``diagnostics/wandb.json`` and must find that
W&B run (``resume="must"``).  Scalars are namespaced ``perf/ data/ router/ optimizer/`` by key and ``train/`` or
``eval/`` otherwise; four kinds of event become ``event/<type>`` markers; the final per-group optimizer and per-layer
router tables are logged as ``wandb.Table`` objects.
"""

from __future__ import annotations

import importlib
import json
import math
import re
from pathlib import Path
from typing import Any, Callable, Mapping

from research_b200.config import resolved_config_sha256
from research_b200.config.specs import RunSpec
from research_b200.errors import ContractError
from research_b200.services.artifacts import LocalArtifactWriter, utc_now

SKIPPED_KEYS = frozenset({"optimizer_groups", "moe_router_layers", "final_optimizer_groups", "final_moe_router_layers"})
PERF_KEYS = frozenset({
    "tokens_per_sec", "train_tokens_per_sec", "examples_per_sec", "flops_per_token", "flops_per_step",
    "flops_per_sec", "mfu", "mfu_exact", "peak_flops_total", "step_sec", "train_step_sec", "train_dispatch_sec",
    "metrics_sync_sec", "device_memory_used_bytes", "device_memory_peak_bytes", "device_memory_limit_bytes",
    "gpu_memory_used_bytes", "gpu_memory_total_bytes", "gpu_utilization_pct", "gpu_memory_utilization_pct",
    "gpu_power_w", "gpu_temperature_c"})
DATA_KEYS = frozenset({
    "epoch", "token_start", "token_end", "token_count", "tokens_seen", "examples", "target_tokens",
    "documents_touched", "global_batch_size", "per_device_batch_size", "data_axis_size", "data_sec", "placement_sec",
    "data_worker_count", "data_worker_buffer_size", "data_prefetch"})
OPTIMIZER_KEYS = frozenset({"grad_norm", "param_norm", "update_norm", "lr", "clip_scale"})
MIRRORED_EVENTS = frozenset({"training_started", "checkpoint_saved", "training_completed", "training_failed"})


def safe_run_name(run_id: str) -> str:
    return re.sub(r"[^A-Za-z0-9_.-]+", "-", run_id).strip("-") or "run"


def wandb_run_id(spec: RunSpec) -> str:
    return f"{safe_run_name(spec.run_id)}-{resolved_config_sha256(spec)[:16]}"


def is_scalar(value: Any) -> bool:
    """Booleans and finite numbers are logged; strings, containers, nulls and non-finite numbers are not."""

    if isinstance(value, bool):
        return True
    return isinstance(value, (int, float)) and math.isfinite(float(value))


def metric_key(namespace: str, key: str) -> str:
    if key in PERF_KEYS:
        return f"perf/{key}"
    if key in DATA_KEYS:
        return f"data/{key}"
    if key.startswith(("router_", "smebu_")):
        return f"router/{key}"
    if key.startswith("optimizer_") or key in OPTIMIZER_KEYS:
        return f"optimizer/{key}"
    return f"{namespace}/{key}"


def namespaced_metrics(row: Mapping[str, Any], namespace: str = "train") -> dict[str, Any]:
    return {metric_key(namespace, k): v for k, v in row.items()
            if k != "step" and k not in SKIPPED_KEYS and is_scalar(v)}


def step_of(row: Mapping[str, Any]) -> int | None:
    step = row.get("step")
    return step if isinstance(step, int) and not isinstance(step, bool) else None


def read_wandb_metadata(run_dir: str | Path) -> Mapping[str, Any]:
    path = Path(run_dir) / "diagnostics" / "wandb.json"
    if not path.is_file():
        raise ContractError("W&B resume requested but diagnostics/wandb.json is missing")
    try:
        raw = json.loads(path.read_text())
    except Exception as exc:
        raise ContractError(f"failed to read W&B metadata {path}: {exc}") from exc
    if not isinstance(raw, Mapping):
        raise ContractError("diagnostics/wandb.json must be a JSON object")
    return raw


def final_tables(summary: Mapping[str, Any], wandb_module: Any) -> dict[str, Any]:
    """``final/optimizer_groups`` and ``final/moe_router_layers`` as tables with the union of the rows' keys."""

    tables = {}
    for key in ("final_optimizer_groups", "final_moe_router_layers"):
        rows = [dict(r) for r in (summary.get(key) or []) if isinstance(r, Mapping)]
        if rows:
            columns = sorted({str(k) for r in rows for k in r})
            tables[f"final/{key[len('final_'):]}"] = wandb_module.Table(
                columns=columns, data=[[r.get(c) for c in columns] for r in rows])
    return tables


class WandbMirroredWriter(LocalArtifactWriter):
    def __init__(self, spec: RunSpec, run_dir: str | Path, *, resume: bool = False):
        super().__init__(run_dir)
        self.spec = spec
        self._failed = False
        self._finished = False
        try:
            self._wandb = importlib.import_module("wandb")
        except ImportError as exc:
            raise ContractError("artifacts.wandb_enabled=true but the wandb package is not importable") from exc
        a = spec.artifacts
        if resume:
            try:
                run_id = read_wandb_metadata(self.run_dir).get("wandb_run_id")
                if not isinstance(run_id, str) or not run_id:
                    raise ContractError("wandb metadata.wandb_run_id must be a non-empty string")
            except ContractError as exc:
                self._record_failure("init", exc)
                raise
        else:
            run_id = wandb_run_id(spec)
        mode = "must" if resume else "allow"
        self._run = self._guard("init", lambda: self._wandb.init(
            project=a.wandb_project, entity=a.wandb_entity, group=a.wandb_group, tags=list(a.wandb_tags),
            mode=a.wandb_mode, id=run_id, name=spec.run_id, resume=mode, dir=str(self.run_dir),
            config={"run_id": spec.run_id, "model": spec.model.name, "model_variant": spec.model.variant,
                    "optimizer": spec.optimizer.name, "parallelism": spec.parallelism.mode,
                    "data_mode": spec.data.mode, "seq_len": spec.training.seq_len,
                    "global_batch_size": spec.training.global_batch_size}))
        run = self._run
        self.metadata = {"schema_version": 1, "enabled": True, "run_id": run_id,
                         "wandb_run_id": str(getattr(run, "id", None) or run_id), "project": a.wandb_project,
                         "entity": a.wandb_entity, "group": a.wandb_group, "tags": list(a.wandb_tags),
                         "mode": a.wandb_mode, "url": getattr(run, "url", None), "name": getattr(run, "name", None),
                         "resume": mode, "created_at": utc_now()}
        self.write_wandb_metadata(self.metadata)

    # ---- plumbing ---------------------------------------------------------------------------------
    def _record_failure(self, what: str, exc: Exception) -> None:
        self._failed = True
        LocalArtifactWriter.append_event(self, {
            "schema_version": 1, "type": "wandb_failed", "run_id": self.spec.run_id, "created_at": utc_now(),
            "operation": what, "phase": what, "error_type": type(exc).__name__, "error_message": str(exc),
            "error": str(exc)})

    def _guard(self, what: str, fn: Callable[[], Any]) -> Any:
        if self._failed:
            return None
        try:
            return fn()
        except Exception as exc:
            self._record_failure(what, exc)
            raise ContractError(f"wandb {what} failed: {exc}") from exc

    def _log(self, payload: Mapping[str, Any], step: int | None) -> None:
        if payload:
            target = self._run if hasattr(self._run, "log") else self._wandb
            target.log(dict(payload), step=step)

    def _summary_update(self, payload: Mapping[str, Any]) -> None:
        summary = getattr(self._run, "summary", None)
        if summary is None:
            summary = getattr(getattr(self._wandb, "run", None), "summary", None)
        if payload and hasattr(summary, "update"):
            summary.update(dict(payload))

    # ---- mirrored artifact calls -------------------------------------------------------------------
    def append_event(self, event: Mapping[str, Any]) -> None:
        super().append_event(event)
        kind = event.get("type")
        if kind in MIRRORED_EVENTS:
            payload = namespaced_metrics(event, f"event/{kind}")
            payload[f"event/{kind}"] = 1
            self._guard("log_event", lambda: self._log(payload, step_of(event)))

    def append_train_metrics(self, row: Mapping[str, Any]) -> None:
        super().append_train_metrics(row)
        self._guard("log_train", lambda: self._log(namespaced_metrics(row, "train"), step_of(row)))

    def append_eval_metrics(self, row: Mapping[str, Any]) -> None:
        super().append_eval_metrics(row)
        self._guard("log_eval", lambda: self._log(namespaced_metrics(row, "eval"), step_of(row)))

    def write_runtime_diagnostics(self, diagnostics: Mapping[str, Any]) -> None:
        super().write_runtime_diagnostics(diagnostics)
        perf = diagnostics.get("performance") or {}
        payload = {f"diagnostics/{k}": perf.get(k) for k in ("device_count", "flops_per_token", "peak_flops_total")}
        self._guard("runtime_diagnostics",
                    lambda: self._summary_update({k: v for k, v in payload.items() if is_scalar(v)}))

    def write_summary(self, summary: Mapping[str, Any]) -> None:
        super().write_summary(summary)

        def push():
            scalars = namespaced_metrics(summary, "final")
            # plain keys as well, so that a summary panel can show ``steps`` or ``final_loss`` without a namespace
            scalars.update({k: v for k, v in summary.items() if k not in SKIPPED_KEYS and is_scalar(v)})
            self._summary_update(scalars)
            tables = final_tables(summary, self._wandb) if hasattr(self._wandb, "Table") else {}
            self._log(tables, step_of(summary))
        self._guard("summary", push)

    def close(self) -> None:
        if self._finished:
            return
        self._finished = True
        target = self._run if hasattr(self._run, "finish") else self._wandb
        if self._failed:
            try:                                    # best effort: the run already failed, do not mask its error
                target.finish()
            except Exception:
                pass
            return
        self._guard("finish", target.finish)
