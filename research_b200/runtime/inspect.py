"""``run inspect``: read-only summary of a run directory - manifest, config hash, progress, last metrics,
checkpoints, evals, router and optimizer health (reference: src/jaxtitan/runtime/inspect.py:20-63)."""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any

from research_b200.errors import ContractError
from research_b200.runtime.checkpoint_index import load_checkpoint_index


def _read_json(path: Path) -> Any:
    try:
        return json.loads(path.read_text())
    except (OSError, json.JSONDecodeError) as exc:
        raise ContractError(f"failed to read {path}: {exc}") from exc


def _read_jsonl(path: Path) -> list[dict[str, Any]]:
    if not path.is_file():
        return []
    rows = []
    for n, line in enumerate(path.read_text().splitlines(), 1):
        if not line.strip():
            continue
        try:
            rows.append(json.loads(line))
        except json.JSONDecodeError as exc:
            raise ContractError(f"failed to parse {path} line {n}: {exc}") from exc
    return rows


def _num(value: Any) -> float:
    return float(value) if isinstance(value, (int, float)) and not isinstance(value, bool) else 0.0


def router_health(final: dict[str, Any], recent: list[dict[str, Any]]) -> dict[str, Any] | None:
    """Router roll-up from the newest row that carries per-layer statistics: the summary figures plus the layer with
    the worst load imbalance (reference: src/jaxtitan/runtime/inspect.py:197-222)."""

    last = next((r for r in reversed(recent) if r.get("moe_router_layers")), recent[-1] if recent else {})
    layers = final.get("final_moe_router_layers") or last.get("moe_router_layers")
    if not isinstance(layers, list) or not layers:
        return None
    worst = max(layers, key=lambda item: _num(item.get("load_cv")))
    pick = lambda key: final.get(f"final_{key}", last.get(key))  # noqa: E731
    return {
        "layer_count": len(layers), "dead_experts_count": pick("router_dead_experts_count"),
        "mean_load_cv": pick("router_mean_load_cv"), "mean_importance_cv": pick("router_mean_importance_cv"),
        "mean_importance_entropy": pick("router_mean_importance_entropy"),
        "worst_layer": {k: worst.get(k) for k in ("layer_index", "load_cv", "load_entropy", "experts_active",
                                                  "importance_cv", "importance_entropy")},
    }


def optimizer_health(final: dict[str, Any], recent: list[dict[str, Any]]) -> dict[str, Any] | None:
    """Optimizer roll-up from the newest row with group norms: counts, update/parameter ratios and the group whose
    update is largest relative to its parameters (reference: src/jaxtitan/runtime/inspect.py:225-266)."""

    last = next((r for r in reversed(recent) if r.get("optimizer_groups")), recent[-1] if recent else {})
    groups = final.get("final_optimizer_groups") or last.get("optimizer_groups")
    if not isinstance(groups, list) or not groups:
        return None
    worst = max(groups, key=lambda item: _num(item.get("update_param_ratio")))

    def pick(key: str):
        value = final.get(f"final_optimizer_{key}")
        return last.get(f"optimizer_{key}") if value is None else value

    return {
        "group_count": len(groups), "update_param_ratio_max_group": worst.get("group"),
        "update_param_ratio_max": pick("update_param_ratio_max"),
        "update_param_ratio_mean": pick("update_param_ratio_mean"),
        "groups_with_zero_grad": pick("groups_with_zero_grad"),
        "groups_with_zero_update": pick("groups_with_zero_update"),
        "nonfinite_groups": pick("nonfinite_groups"),
        "route_backend_counts": pick("route_backend_counts"),
        "worst_update_ratio_group": {k: worst.get(k) for k in ("group", "tag", "backend", "update_param_ratio",
                                                               "grad_param_ratio")},
    }


def inspect_run(run_dir: str | Path) -> dict[str, Any]:
    run_dir = Path(run_dir)
    if not run_dir.is_dir():
        raise ContractError(f"run directory does not exist: {run_dir}")
    manifest_path = run_dir / "manifest.json"
    if not manifest_path.is_file():
        raise ContractError(f"run directory has no manifest.json: {run_dir}")
    manifest = _read_json(manifest_path)
    train = _read_jsonl(run_dir / "metrics" / "train.jsonl")
    evals = _read_jsonl(run_dir / "metrics" / "eval.jsonl")
    events = _read_jsonl(run_dir / "events.jsonl")
    index = load_checkpoint_index(run_dir)
    summary_path = run_dir / "summaries" / "final.json"
    summary = _read_json(summary_path) if summary_path.is_file() else None
    runtime_path = run_dir / "diagnostics" / "runtime.json"
    runtime = _read_json(runtime_path) if runtime_path.is_file() else None
    last = train[-1] if train else None
    event_types = [e.get("type") for e in events]
    status = "initialized"
    if "training_completed" in event_types:
        status = "completed"
    elif "training_failed" in event_types and event_types[::-1].index("training_failed") < \
            (event_types[::-1].index("training_started") if "training_started" in event_types else 10 ** 9):
        status = "failed"
    elif "training_started" in event_types:
        status = "running_or_interrupted"
    router = None
    if last is not None and last.get("router_max_vio") is not None:
        router = {k: last.get(k) for k in last if k.startswith("router_") or k.startswith("smebu_")}
    return {
        "schema_version": 1, "run_id": manifest.get("run_id"), "run_dir": run_dir.as_posix(), "status": status,
        "created_at": manifest.get("created_at"), "resolved_config_sha256": manifest.get("resolved_config_sha256"),
        "data": manifest.get("data"),
        "progress": None if last is None else {"step": last.get("step"), "tokens_seen": last.get("tokens_seen"),
                                                "loss": last.get("loss"), "lr": last.get("lr"),
                                                "grad_norm": last.get("grad_norm"), "mfu": last.get("mfu"),
                                                "train_tokens_per_sec": last.get("train_tokens_per_sec")},
        "train_rows": len(train), "eval_rows": len(evals),
        "last_eval": evals[-1] if evals else None,
        "checkpoints": index.to_dict(),
        "events": {"count": len(events), "types": sorted(set(t for t in event_types if t)),
                   "last": events[-1] if events else None,
                   "failures": [e for e in events if str(e.get("type", "")).endswith("_failed")]},
        "router": router,
        "router_health": router_health(summary or {}, train[-8:]),
        "optimizer_health": optimizer_health(summary or {}, train[-8:]),
        "optimizer": None if runtime is None else runtime.get("optimizer", {}) and {
            "name": runtime["optimizer"].get("name"),
            "backend_parameter_counts": runtime["optimizer"].get("backend_parameter_counts")},
        "runtime": None if runtime is None else {"mesh": runtime.get("mesh"), "parallelism": runtime.get("parallelism"),
                                                 "model": runtime.get("model")},
        "summary": summary,
    }
