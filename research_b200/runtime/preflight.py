"""``run preflight``: prove a config can train before a run directory exists.

Loads the config, refuses if the run directory exists, builds data / mesh / model / optimizer exactly as training
does, runs ONE real optimizer step on the first batch and, when evals are configured, one validation pass, then
reports devices, mesh, data pipeline, first-batch provenance, model and optimizer policy, the batch arithmetic of the
run, first-step loss / tokens per second / MFU, the placement each rank observed, and the runtime diagnostics that a
run would write - writing nothing itself (reference: src/jaxtitan/runtime/preflight.py:58-412).
"""

from __future__ import annotations

import json
import math
import time
from pathlib import Path
from typing import Any, Mapping

from research_b200.config import load_config, resolved_config_sha256
from research_b200.config.canonical import normalize
from research_b200.errors import ContractError
from research_b200.optim.build import optimizer_policy_summary
from research_b200.runtime.diagnostics import (PhaseTimer, build_runtime_diagnostics, enrich_train_metrics,
                                               sample_device_telemetry)
from research_b200.runtime.trainer import Trainer


def _document_fields(provenances) -> dict[str, Any]:
    aware = all(p.row_doc_ids is not None for p in provenances)
    ids = [d for p in provenances if p.row_doc_ids is not None for d in p.row_doc_ids]
    return {"document_aware": aware, "documents_touched": len(set(ids)) if aware else None,
            "document_min": min(ids) if aware and ids else None, "document_max": max(ids) if aware and ids else None}


def _tensor_summary(t) -> dict[str, Any]:
    return {"shape": [int(d) for d in t.shape], "dtype": str(t.dtype).replace("torch.", ""),
            "device": str(t.device)}


def run_preflight(config_path: str | Path) -> dict[str, Any]:
    config_path = Path(config_path)
    spec = load_config(config_path)
    if spec.dirs.run_dir.exists():
        raise ContractError(f"run directory already exists: {spec.dirs.run_dir}")
    from research_b200.kernels.registry import require_kernel_plan_supported
    from research_b200.parallel.mesh import init_distributed
    from research_b200.runtime.training import metrics_row

    init_distributed()
    trainer = Trainer(spec)
    spec = trainer.spec
    mesh = trainer.mesh
    t = spec.training
    policy = optimizer_policy_summary(trainer.optimizer_build, trainer.result.metadata)
    pipeline = trainer.data.describe()
    runtime = build_runtime_diagnostics(spec, trainer, optimizer_policy=policy, data_pipeline=pipeline)
    require_kernel_plan_supported(runtime["kernels"], spec)

    timer = PhaseTimer()
    with timer.phase("data"):
        batches = trainer.next_accumulated_batch()
    prov = trainer.last_provenance
    with timer.phase("train_step"):
        metrics = trainer.train_on(batches, diagnostics=True)
    timings = timer.to_dict()
    step_sec = timings["train_step"]
    row = enrich_train_metrics(metrics_row(trainer, metrics, spec), timings=timings, runtime=runtime,
                               telemetry=sample_device_telemetry(trainer.device))
    tokens = sum(p.target_tokens for p in prov)

    eval_report = None
    if spec.evals:
        ev = spec.evals[0]
        t0 = time.perf_counter()
        result = trainer.evaluate(ev.num_batches)
        if result["num_batches"] < ev.num_batches:
            raise ContractError(f"validation split ended before eval.num_batches={ev.num_batches} completed")
        eval_report = {
            "name": ev.name, "every_steps": ev.every_steps, "num_batches": result["num_batches"],
            "manifest": spec.data.validation_manifest or spec.data.train_manifest, "split": "val",
            "loss": result["loss"], "bpb": result.get("bpb"), "token_count": int(result["token_count"]),
            "eval_sec": time.perf_counter() - t0, "compile": "passed",
            **{k: result.get(k) for k in ("token_start", "token_end", "examples", "target_tokens", "document_aware",
                                          "documents_touched", "document_min", "document_max")}}

    data_axis = mesh.size("data") * mesh.size("fsdp")
    micro_tokens = t.global_batch_size * t.seq_len
    batch_tokens = micro_tokens * t.gradient_accumulation_steps
    streaming = spec.data.mode == "hf_streaming"
    split_start = None if streaming else getattr(trainer.data, "split_start", None)
    split_end = None if streaming else getattr(trainer.data, "split_end", None)
    first_batch = {"token_start": min(p.token_start for p in prov), "token_end": max(p.token_end for p in prov),
                   "examples": sum(p.examples for p in prov), "target_tokens": tokens,
                   "row_start_offsets": list(prov[0].row_start_offsets),
                   "row_doc_ids": None if prov[0].row_doc_ids is None else list(prov[0].row_doc_ids),
                   **_document_fields(prov)}
    fallback = spec.optimizer.adamw_fallback_schedule
    host_batch = batches[0]
    store = trainer.store.describe()
    report = {
        "schema_version": 1, "status": "ok", "config_path": config_path.as_posix(), "run_id": spec.run_id,
        "run_dir": spec.dirs.run_dir.as_posix(), "resolved_config_sha256": resolved_config_sha256(spec),
        "devices": {"kind": runtime["runtime"]["device_kind"], "count": mesh.world_size,
                    "backend": trainer.device.type, "selected_device_count": mesh.world_size,
                    "local_device_count": mesh.world_size, "global_device_count": mesh.world_size,
                    "process_count": mesh.world_size, "process_index": mesh.rank,
                    "single_process": mesh.world_size == 1, "platforms": [trainer.device.type],
                    "kinds": [runtime["runtime"]["device_kind"]]},
        "mesh": runtime["mesh"], "parallelism": runtime["parallelism"], "data_pipeline": pipeline,
        "data": {"mode": spec.data.mode, "train_manifest": spec.data.train_manifest,
                 "tokenizer_id": spec.data.tokenizer_id, "train_split_start": split_start,
                 "train_split_end": split_end,
                 "train_split_tokens": None if split_start is None or split_end is None else split_end - split_start,
                 "pipeline": pipeline, "first_batch": first_batch},
        "first_batch": first_batch,
        "model": {**runtime["model"], "parameters": trainer.parameter_count()},
        "optimizer": {"name": spec.optimizer.name, "schedule": spec.optimizer.schedule.name,
                      "peak_lr": spec.optimizer.schedule.peak_lr, "total_steps": spec.optimizer.schedule.total_steps,
                      "adamw_fallback_peak_lr": None if fallback is None else fallback.peak_lr,
                      "description": trainer.optimizer_build.description,
                      "backend_parameter_counts": policy["backend_parameter_counts"], "policy": policy},
        "training": {
            "seq_len": t.seq_len, "global_batch_size": t.global_batch_size,
            "micro_global_batch_size": t.global_batch_size,
            "effective_global_batch_size": t.global_batch_size * t.gradient_accumulation_steps,
            "target_tokens": t.target_tokens, "batch_tokens": batch_tokens, "micro_tokens_per_step": micro_tokens,
            "effective_tokens_per_step": batch_tokens,
            "gradient_accumulation_steps": t.gradient_accumulation_steps, "z_loss_weight": t.loss.z_loss_weight,
            "data_axis_size": data_axis, "per_device_batch_size": t.global_batch_size // data_axis,
            "per_device_target_tokens": batch_tokens // data_axis,
            "estimated_steps": math.ceil(t.target_tokens / batch_tokens), "log_every_steps": t.log_every_steps,
            "checkpoint_every_steps": t.checkpoint_every_steps, "compile": "passed",
            "first_step_loss": row["loss"], "first_step_total_loss": row.get("total_loss"),
            "first_step_z_loss": row.get("z_loss"), "first_step_moe_aux_loss": row.get("moe_aux_loss"),
            "first_step_router_max_vio": row.get("router_max_vio"),
            "first_step_train_tokens_per_sec": row["train_tokens_per_sec"], "first_step_mfu": row["mfu"]},
        "first_step": {"loss": metrics.loss, "token_count": int(metrics.token_count), "grad_norm": metrics.grad_norm,
                       "param_norm": metrics.param_norm, "update_norm": metrics.update_norm, "lr": metrics.lr,
                       "step_sec": step_sec, "data_sec": timings["data"],
                       "train_tokens_per_sec": row["train_tokens_per_sec"], "mfu": row["mfu"],
                       "mfu_exact": row["mfu_exact"]},
        "eval": eval_report, "diagnostics": runtime, "compile": runtime["compile"], "profiling": runtime["profiling"],
        "sharding": runtime["sharding"], "kernels": runtime["kernels"], "performance": runtime["performance"],
        "observed_sharding": {
            # what this rank really held: the host batch of the step and the arenas of the parameter store
            "first_train_batch": {"input_ids": _tensor_summary(host_batch.input_ids),
                                  "target_ids": _tensor_summary(host_batch.target_ids),
                                  "loss_mask": _tensor_summary(host_batch.loss_mask),
                                  **({} if getattr(host_batch, "doc_ids", None) is None
                                     else {"doc_ids": _tensor_summary(host_batch.doc_ids)})},
            "train_state": {"mode": store["mode"], "weights_resident": store["weights_resident"],
                            "arena_elements": store["arena_elements"], "sections": len(store["sections"]),
                            "parameter_leaves": len(trainer.result.metadata)}},
    }
    if hasattr(trainer.data, "close"):
        trainer.data.close()
    return normalize(report)


def preflight_report_to_json(report: Mapping[str, Any]) -> str:
    return json.dumps(normalize(report), sort_keys=True, separators=(",", ":"))


def format_preflight_report(report: Mapping[str, Any]) -> str:
    """The report as the lines a person reads before starting a run (reference: preflight.py:316-412)."""

    d, mesh, par, data = report["devices"], report["mesh"], report["parallelism"], report["data"]
    model, opt, tr, fs = report["model"], report["optimizer"], report["training"], report["first_step"]
    comp, prof, kern, perf = report["compile"], report["profiling"], report["kernels"], report["performance"]
    pipe = data["pipeline"]

    def num(v, fmt="{:.4g}"):
        return "n/a" if v is None else fmt.format(v)

    lines = [
        f"preflight: {report['status']}",
        f"run: {report['run_id']}",
        f"run_dir: {report['run_dir']}",
        f"devices: selected={d['selected_device_count']} global={d['global_device_count']} "
        f"process_count={d['process_count']} platforms={','.join(d['platforms'])} kind={d['kind']}",
        f"mesh: axes={mesh['axis_names']} sizes={mesh['axis_sizes']}",
        f"parallelism: mode={par['execution_mode']} metrics={par['metrics_scope']} artifacts={par['artifact_writer']} "
        f"data_axis={par['mesh']['data_axis_size']} global_batch={par['batch']['global_batch_size']} "
        f"per_device_batch={par['batch']['per_device_batch_size']}",
        f"runtime: backend={d['backend']} device_kind={perf['device_kind']} "
        f"peak_flops={num(perf['peak_flops_per_device'], '{:.3e}')}",
        f"train data: mode={data['mode']} manifest={data['train_manifest']} tokens={data['train_split_tokens']} "
        f"first_batch={data['first_batch']['target_tokens']} pipeline={pipe.get('backend')} order={pipe.get('order')} "
        f"documents={pipe.get('document_aware')} count={pipe.get('document_count')}",
        f"model: {model['name']} variant={model['variant']} parameters={model['parameters']} "
        f"param_dtype={model['param_dtype']} compute_dtype={model['compute_dtype']} remat={model['remat']}",
        f"optimizer: {opt['name']} schedule={opt['schedule']} peak_lr={opt['peak_lr']} total_steps={opt['total_steps']} "
        f"adamw_fallback_peak_lr={opt['adamw_fallback_peak_lr']} routes={opt['backend_parameter_counts']}",
        f"training: estimated_steps={tr['estimated_steps']} batch_tokens={tr['batch_tokens']} "
        f"grad_accum={tr['gradient_accumulation_steps']} effective_batch={tr['effective_global_batch_size']} "
        f"per_device_batch={tr['per_device_batch_size']} log_every={tr['log_every_steps']} "
        f"checkpoint_every={tr['checkpoint_every_steps']} compile={tr['compile']}",
        f"first step: loss={num(fs['loss'], '{:.4f}')} grad_norm={num(fs['grad_norm'])} lr={num(fs['lr'])} "
        f"step_sec={num(fs['step_sec'])} train_tokens_per_sec={num(fs['train_tokens_per_sec'], '{:.0f}')} "
        f"mfu={num(fs['mfu'], '{:.2f}')}",
        f"compile contract: train_shape={comp['train']['expected_batch_shape']} "
        f"donate_train={comp['train']['donate_state']} eval_shape={comp['eval']['expected_batch_shape']} "
        f"donate_eval={comp['eval']['donate_state']}",
        f"profiling: enabled={prof.get('enabled')} start={prof.get('trace_start_step')} "
        f"steps={prof.get('trace_steps')}",
        f"kernels: enabled={kern.get('enabled')} strict={kern.get('strict')} active={kern.get('active_count')} "
        f"fallback={kern.get('fallback_count')} unavailable={kern.get('unavailable_count')}",
    ]
    ev = report["eval"]
    if ev is None:
        lines.append("eval: skipped")
    else:
        lines.append(f"eval: name={ev['name']} every={ev['every_steps']} batches={ev['num_batches']} "
                     f"loss={num(ev['loss'], '{:.4f}')} compile={ev['compile']}")
    return "\n".join(lines)
