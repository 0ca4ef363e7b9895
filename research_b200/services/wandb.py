"""Optional Weights & Biases mirror of the local artifacts (reference: src/jaxtitan/services/wandb.py:172-349).

Local files are always written first; every mirrored call that fails writes a ``wandb_failed`` event and aborts the
run.  The W&B run id is deterministic (``<run_id>-<first 16 hex of the resolved config sha256>``) so a resumed run
continues the same W&B run; metrics are namespaced ``train/ perf/ data/ router/ optimizer/ eval/``.
"""

from __future__ import annotations

import importlib
from pathlib import Path
from typing import Any, Mapping

from research_b200.config import resolved_config_sha256, run_spec_to_dict
from research_b200.config.specs import RunSpec
from research_b200.errors import ContractError
from research_b200.services.artifacts import LocalArtifactWriter, utc_now

PERF_KEYS = ("tokens_per_sec", "train_tokens_per_sec", "examples_per_sec", "mfu", "mfu_exact", "flops_per_sec",
             "step_sec", "train_step_sec", "data_sec", "placement_sec", "metrics_sync_sec")
DATA_KEYS = ("epoch", "token_start", "token_end", "examples", "target_tokens", "documents_touched")


def wandb_run_id(spec: RunSpec) -> str:
    return f"{spec.run_id}-{resolved_config_sha256(spec)[:16]}"


def namespaced_metrics(row: Mapping[str, Any]) -> dict[str, Any]:
    out: dict[str, Any] = {}
    for key, value in row.items():
        if not isinstance(value, (int, float)) or isinstance(value, bool):
            continue
        if key in PERF_KEYS or key.startswith("nvml_") or key.startswith("device_memory"):
            out[f"perf/{key}"] = value
        elif key in DATA_KEYS:
            out[f"data/{key}"] = value
        elif key.startswith("router_") or key.startswith("smebu_"):
            out[f"router/{key}"] = value
        elif key.startswith("optimizer_") or key in ("grad_norm", "param_norm", "update_norm", "lr", "clip_scale"):
            out[f"optimizer/{key}"] = value
        else:
            out[f"train/{key}"] = value
    return out


class WandbMirroredWriter(LocalArtifactWriter):
    def __init__(self, spec: RunSpec, run_dir: str | Path):
        super().__init__(run_dir)
        self.spec = spec
        try:
            self._wandb = importlib.import_module("wandb")
        except ImportError as exc:
            raise ContractError("artifacts.wandb_enabled=true but the wandb package is not importable") from exc
        a = spec.artifacts
        self._guard("init", lambda: self._wandb.init(
            project=a.wandb_project, entity=a.wandb_entity, group=a.wandb_group, tags=list(a.wandb_tags),
            mode=a.wandb_mode, id=wandb_run_id(spec), name=spec.run_id, resume="allow",
            config=run_spec_to_dict(spec), dir=str(self.run_dir)))
        self.write_wandb_metadata({"schema_version": 1, "enabled": True, "project": a.wandb_project,
                                   "entity": a.wandb_entity, "group": a.wandb_group, "mode": a.wandb_mode,
                                   "run_id": wandb_run_id(spec), "created_at": utc_now()})

    def _guard(self, what: str, fn) -> Any:
        try:
            return fn()
        except Exception as exc:
            super().append_event({"schema_version": 1, "type": "wandb_failed", "run_id": self.spec.run_id,
                                  "created_at": utc_now(), "operation": what, "error_type": type(exc).__name__,
                                  "error_message": str(exc)})
            raise ContractError(f"wandb {what} failed: {exc}") from exc

    def append_train_metrics(self, row: Mapping[str, Any]) -> None:
        super().append_train_metrics(row)
        self._guard("log_train", lambda: self._wandb.log(namespaced_metrics(row), step=int(row["step"])))

    def append_eval_metrics(self, row: Mapping[str, Any]) -> None:
        super().append_eval_metrics(row)
        payload = {f"eval/{k}": v for k, v in row.items() if isinstance(v, (int, float)) and not isinstance(v, bool)}
        self._guard("log_eval", lambda: self._wandb.log(payload, step=int(row["step"])))

    def write_summary(self, summary: Mapping[str, Any]) -> None:
        super().write_summary(summary)

        def push():
            run = getattr(self._wandb, "run", None)
            if run is not None:
                for k, v in summary.items():
                    if isinstance(v, (int, float, str)) and not isinstance(v, bool):
                        run.summary[k] = v
        self._guard("summary", push)

    def close(self) -> None:
        self._guard("finish", lambda: self._wandb.finish())
