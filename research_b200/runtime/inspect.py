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


def checkpoint_summary(run_dir: Path, record) -> dict[str, Any]:
    path = Path(record.checkpoint_path)
    return {"step": record.step, "tokens_seen": record.tokens_seen, "checkpoint_path": path.as_posix(),
            "reason": record.reason, "train_loss": record.train_loss, "eval_loss": record.eval_loss,
            "retained": record.retained, "exists": (run_dir / path).is_dir()}


def validate_checkpoint_paths(run_dir: Path) -> None:
    """Every record that ``checkpoints/index.json`` itself calls retained must still be on disk
    (reference: inspect.py:275-287).  The loaded index cannot tell: it refreshes the flags from the directory."""

    path = run_dir / "checkpoints" / "index.json"
    if not path.is_file():
        return
    records = _read_json(path).get("records")
    if not isinstance(records, list):
        raise ContractError("checkpoint index records must be a list")
    for n, item in enumerate(records):
        if not isinstance(item, dict):
            raise ContractError(f"checkpoint index record {n} must be a JSON object")
        if item.get("retained") is True:
            rel = item.get("checkpoint_path")
            if not isinstance(rel, str) or not rel:
                raise ContractError(f"checkpoint index record {n} checkpoint_path must be a non-empty string")
            if not (run_dir / rel).is_dir():
                raise ContractError(f"checkpoint index retained path does not exist: {rel}")


def diagnostics_summary(raw: dict[str, Any] | None) -> dict[str, Any] | None:
    """The parts of ``diagnostics/runtime.json`` a reader wants first (reference: inspect.py:290-321)."""

    if raw is None:
        return None
    perf, runtime = raw.get("performance"), raw.get("runtime")
    if not isinstance(perf, dict) or not isinstance(runtime, dict):
        raise ContractError("runtime diagnostics must include performance and runtime objects")
    for key in ("parallelism", "sharding", "data_pipeline"):
        if raw.get(key) is not None and not isinstance(raw[key], dict):
            raise ContractError(f"runtime diagnostics {key} must be an object")
    par, pipe = raw.get("parallelism"), raw.get("data_pipeline")
    return {
        "path": "diagnostics/runtime.json", "backend": runtime.get("backend"),
        "process_count": runtime.get("process_count"), "process_index": runtime.get("process_index"),
        "device_kind": perf.get("device_kind", runtime.get("device_kind")),
        "device_count": perf.get("device_count", runtime.get("selected_device_count")),
        "flops_per_token": perf.get("flops_per_token"), "peak_flops_per_device": perf.get("peak_flops_per_device"),
        "peak_flops_total": perf.get("peak_flops_total"),
        "parallelism": None if par is None else {k: par.get(k) for k in (
            "execution_mode", "metrics_scope", "artifact_writer", "single_process", "process", "devices", "mesh",
            "batch", "host_artifacts")},
        "sharding": raw.get("sharding"),
        "data_pipeline": None if pipe is None else {k: pipe.get(k) for k in (
            "backend", "backend_version", "state_schema_version", "split", "order", "shuffle_seed", "worker_count",
            "worker_buffer_size", "prefetch", "batch_size", "seq_len", "num_records", "manifest_sha256",
            "tokenizer_id", "document_aware", "document_count", "document_offsets_path", "document_offsets_sha256",
            "document_buffer_size", "document_refill_size")},
        "kernels": kernel_summary(raw), "wandb": wandb_summary(None, raw),
    }


def kernel_summary(diagnostics: dict[str, Any] | None) -> dict[str, Any] | None:
    raw = None if diagnostics is None else diagnostics.get("kernels")
    if not isinstance(raw, dict):
        return None
    ops = raw.get("ops") or []
    return {"enabled": raw.get("enabled"), "strict": raw.get("strict"), "compile": raw.get("compile"),
            "arch": raw.get("arch"), "device_kind": raw.get("device_kind"), "active_count": raw.get("active_count"),
            "fallback_count": raw.get("fallback_count"), "disabled_count": raw.get("disabled_count"),
            "unavailable_count": raw.get("unavailable_count"),
            "active": [op["op"] for op in ops if op.get("selected")],
            "fallback": [op["op"] for op in ops if not op.get("selected") and op.get("built")],
            "unavailable": [op["op"] for op in ops if not op.get("built")]}


def wandb_summary(raw: dict[str, Any] | None, diagnostics: dict[str, Any] | None) -> dict[str, Any] | None:
    if raw is None and diagnostics is not None and isinstance(diagnostics.get("wandb"), dict):
        raw = diagnostics["wandb"]
    if raw is None:
        return None
    return {k: raw.get(k) for k in ("enabled", "wandb_run_id", "project", "entity", "group", "tags", "mode", "url",
                                    "name", "resume")}


def profiling_summary(raw: dict[str, Any] | None, diagnostics: dict[str, Any] | None) -> dict[str, Any] | None:
    """From ``diagnostics/profiling.json`` when a trace was taken, else from the configured window
    (reference: inspect.py:361-393)."""

    source = raw
    if source is None and diagnostics is not None and isinstance(diagnostics.get("profiling"), dict):
        source = diagnostics["profiling"]
    if source is None:
        return None
    files = source.get("trace_files") if isinstance(source.get("trace_files"), list) else []
    span = source.get("traced_step_range")
    if not isinstance(span, dict):
        start, end = source.get("trace_start_step"), source.get("trace_end_step")
        span = None if start is None or end is None else {"start": start, "end": end}
    return {"enabled": source.get("enabled"),
            "status": source.get("status", "configured" if source.get("enabled") else "disabled"),
            "trace_dir": source.get("trace_dir", "profiles"), "trace_step_range": span,
            "trace_start_step": source.get("trace_start_step"), "trace_steps": source.get("trace_steps"),
            "trace_end_step": source.get("trace_end_step"), "trace_files": files,
            "perfetto_trace_available": any(isinstance(f, str) and f.lower().endswith(
                (".trace.json.gz", ".json.gz", ".trace", ".trace.json")) for f in files),
            "started_at": source.get("started_at"), "stopped_at": source.get("stopped_at"),
            "error": source.get("error")}


def inspect_run(run_dir: str | Path) -> dict[str, Any]:
    run_dir = Path(run_dir)
    if not run_dir.is_dir():
        raise ContractError(f"run directory does not exist: {run_dir}")
    manifest_path = run_dir / "manifest.json"
    if not manifest_path.is_file():
        raise ContractError(f"run directory has no manifest.json: {run_dir}")
    manifest = _read_json(manifest_path)
    if not isinstance(manifest.get("run_id"), str) or not manifest["run_id"]:
        raise ContractError("run manifest.run_id must be a non-empty string")
    train = _read_jsonl(run_dir / "metrics" / "train.jsonl")
    evals = _read_jsonl(run_dir / "metrics" / "eval.jsonl")
    events = _read_jsonl(run_dir / "events.jsonl")
    index = load_checkpoint_index(run_dir)
    validate_checkpoint_paths(run_dir)

    def optional(*parts: str):
        path = run_dir.joinpath(*parts)
        return _read_json(path) if path.is_file() else None

    summary = optional("summaries", "final.json")
    runtime = optional("diagnostics", "runtime.json")
    wandb = optional("diagnostics", "wandb.json")
    profiling = optional("diagnostics", "profiling.json")
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
    final = summary or {}
    latest, best = index.latest_record, index.best_record
    return {
        "schema_version": 1, "run_id": manifest.get("run_id"), "run_dir": run_dir.as_posix(), "status": status,
        "created_at": manifest.get("created_at"), "resolved_config_sha256": manifest.get("resolved_config_sha256"),
        "data": manifest.get("data"),
        "final": None if summary is None else {
            "step": final.get("steps"), "tokens_seen": final.get("tokens_seen"),
            "target_tokens": final.get("target_tokens"), "loss": final.get("final_loss"),
            "eval_loss": final.get("final_eval_loss"), "eval_token_count": final.get("final_eval_token_count"),
            "eval_num_batches": final.get("final_eval_num_batches")},
        "progress": None if last is None else {"step": last.get("step"), "tokens_seen": last.get("tokens_seen"),
                                                "loss": last.get("loss"), "lr": last.get("lr"),
                                                "grad_norm": last.get("grad_norm"), "mfu": last.get("mfu"),
                                                "train_tokens_per_sec": last.get("train_tokens_per_sec")},
        "train_rows": len(train), "eval_rows": len(evals),
        "last_eval": evals[-1] if evals else None,
        "latest_checkpoint": None if latest is None else checkpoint_summary(run_dir, latest),
        "best_checkpoint": None if best is None else checkpoint_summary(run_dir, best),
        "checkpoints": [checkpoint_summary(run_dir, r) for r in index.records],
        "checkpoint_index": index.to_dict(),
        "diagnostics": diagnostics_summary(runtime), "wandb": wandb_summary(wandb, runtime),
        "profiling": profiling_summary(profiling, runtime), "kernels": kernel_summary(runtime),
        "events": {"count": len(events), "types": sorted(set(t for t in event_types if t)),
                   "last": events[-1] if events else None,
                   "failures": [e for e in events if str(e.get("type", "")).endswith("_failed")]},
        "router": router,
        "router_health": router_health(final, train[-8:]),
        "optimizer_health": optimizer_health(final, train[-8:]),
        "optimizer": None if runtime is None else runtime.get("optimizer", {}) and {
            "name": runtime["optimizer"].get("name"),
            "backend_parameter_counts": runtime["optimizer"].get("backend_parameter_counts")},
        "runtime": None if runtime is None else {"mesh": runtime.get("mesh"), "parallelism": runtime.get("parallelism"),
                                                 "model": runtime.get("model")},
        "recent_train_metrics": train[-5:], "recent_eval_metrics": evals[-5:],
        "summary": summary,
    }


def run_inspection_to_json(report: dict[str, Any]) -> str:
    return json.dumps(report, sort_keys=True, separators=(",", ":"))


def _checkpoint_ref(record: dict[str, Any] | None) -> str:
    if record is None:
        return "none"
    tail = "" if record["eval_loss"] is None else f" eval_loss={record['eval_loss']}"
    return f"step={record['step']} path={record['checkpoint_path']}{tail}"


def format_run_inspection(report: dict[str, Any]) -> str:
    """The inspection as lines for a terminal (reference: inspect.py:72-171); a run without a final summary shows its
    newest logged step instead."""

    lines = [f"run: {report['run_id']}", f"status: {report['status']}"]
    final, prog = report["final"], report["progress"]
    if final is not None:
        lines.append(f"final: step={final['step']} tokens={final['tokens_seen']}/{final['target_tokens']} "
                     f"loss={final['loss']}")
        if final["eval_loss"] is not None:
            lines.append(f"validation: loss={final['eval_loss']} tokens={final['eval_token_count']} "
                         f"batches={final['eval_num_batches']}")
    elif prog is not None:
        lines.append(f"progress: step={prog['step']} tokens={prog['tokens_seen']} loss={prog['loss']}")
    diag = report["diagnostics"]
    if diag is not None:
        lines.append(f"runtime: backend={diag['backend']} device={diag['device_kind']} devices={diag['device_count']}")
        par = diag["parallelism"]
        if par is not None and par.get("batch") and par.get("mesh"):
            lines.append(f"parallelism: mode={par['execution_mode']} metrics={par['metrics_scope']} "
                         f"artifacts={par['artifact_writer']} data_axis={par['mesh']['data_axis_size']} "
                         f"global_batch={par['batch']['global_batch_size']} "
                         f"per_device_batch={par['batch']['per_device_batch_size']}")
        pipe = diag["data_pipeline"]
        if pipe is not None:
            lines.append(f"data pipeline: backend={pipe['backend']} version={pipe['backend_version']} "
                         f"order={pipe['order']} shuffle_seed={pipe['shuffle_seed']} workers={pipe['worker_count']} "
                         f"prefetch={pipe['prefetch']} documents={pipe['document_aware']} "
                         f"count={pipe['document_count']}")
    wb = report["wandb"]
    if wb is not None:
        tail = "" if wb["url"] is None else f" url={wb['url']}"
        lines.append(f"wandb: project={wb['project']} entity={wb['entity']} mode={wb['mode']} "
                     f"id={wb['wandb_run_id']}{tail}")
    prof = report["profiling"]
    if prof is not None and prof["enabled"]:
        lines.append(f"profiling: status={prof['status']} range={prof['trace_step_range']} dir={prof['trace_dir']} "
                     f"perfetto={'yes' if prof['perfetto_trace_available'] else 'no'}")
    kern = report["kernels"]
    if kern is not None:
        lines.append(f"kernels: enabled={kern['enabled']} strict={kern['strict']} active={kern['active_count']} "
                     f"fallback={kern['fallback_count']} unavailable={kern['unavailable_count']}")
    rh = report["router_health"]
    if rh is not None:
        worst = rh["worst_layer"]
        lines.append(f"router health: layers={rh['layer_count']} worst_layer={worst['layer_index']} "
                     f"load_cv={worst['load_cv']} dead_experts={rh['dead_experts_count']} "
                     f"importance_cv={worst['importance_cv']}")
    oh = report["optimizer_health"]
    if oh is not None:
        lines.append(f"optimizer health: groups={oh['group_count']} max_update_ratio={oh['update_param_ratio_max']} "
                     f"group={oh['update_param_ratio_max_group']} zero_grad={oh['groups_with_zero_grad']} "
                     f"zero_update={oh['groups_with_zero_update']} backends={oh['route_backend_counts']}")
    failures = report["events"]["failures"]
    if failures:
        lines.append(f"failures: {len(failures)} (last: {failures[-1].get('type')})")
    lines.append(f"latest checkpoint: {_checkpoint_ref(report['latest_checkpoint'])}")
    lines.append(f"best checkpoint: {_checkpoint_ref(report['best_checkpoint'])}")
    lines.append("checkpoints:")
    if not report["checkpoints"]:
        lines.append("  none")
    for r in report["checkpoints"]:
        lines.append(f"  step={r['step']} tokens={r['tokens_seen']} reason={r['reason']} train_loss={r['train_loss']} "
                     f"eval_loss={r['eval_loss']} retained={r['retained']} path={r['checkpoint_path']}")
    return "\n".join(lines)
