"""The host training loop: artifacts, events, logging cadence, evals, checkpoints, resume, failure events.

Flow and artifact contract follow the reference loop (src/jaxtitan/runtime/training.py:157-650): initialise the run
directory (fresh) or reopen it (resume), write ``diagnostics/runtime.json``, then ``while tokens_seen <
target_tokens``: data -> placement + step -> metrics row (+ timing / MFU / telemetry) -> non-finite guard ->
log (``step % log_every == 0`` or at target) -> eval (when due or a checkpoint is due) -> checkpoint (after the
eval, so its loss lands in the index); finally the last row, a final eval and checkpoint, ``summaries/final.json``
and ``training_completed``; any exception writes ``training_failed`` first.

Multi-GPU: every rank runs this loop; rank 0 writes the host-global artifacts, all ranks take part in the gathers
of a checkpoint save and read checkpoints themselves on resume.
"""

from __future__ import annotations

import math
import os
import time
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any, Callable, Mapping

import torch

from research_b200.config import load_config
from research_b200.config.canonical import normalize
from research_b200.config.specs import RunSpec
from research_b200.contracts import StepMetrics
from research_b200.data.pipeline import data_pipeline_state_to_dict
from research_b200.errors import ContractError, JaxtitanError
from research_b200.optim.build import optimizer_policy_summary
from research_b200.runtime.checkpoint_index import load_checkpoint_index, record_checkpoint
from research_b200.runtime.diagnostics import (ARTIFACT_WRITER, METRICS_SCOPE, PhaseTimer,
                                               build_runtime_diagnostics, device_kind, device_telemetry,
                                               enrich_eval_metrics, enrich_train_metrics, runtime_execution_mode,
                                               training_diagnostics_summary)
from research_b200.runtime.profiling import ProfilingManager
from research_b200.runtime.resume import (build_resume_compat, checkpoint_metadata, validate_resume_compat,
                                          validate_resume_metadata)
from research_b200.runtime.state_io import iter_state_tensors, load_state_tensors
from research_b200.runtime.trainer import Trainer
from research_b200.services.artifacts import build_artifact_writer, initialize_run, utc_now
from research_b200.services.checkpoints import LocalCheckpointService

ProgressFn = Callable[[str, dict[str, Any]], None]


@dataclass(frozen=True)
class RunSummary:
    run_id: str
    run_dir: Path
    status: str
    steps: int
    tokens_seen: int
    target_tokens: int
    final_loss: float
    final_eval_loss: float | None = None
    final_eval_token_count: int | None = None
    final_eval_num_batches: int | None = None
    latest_checkpoint_path: str | None = None
    best_eval_step: int | None = None
    best_eval_loss: float | None = None
    best_checkpoint_path: str | None = None
    total_wall_sec: float | None = None
    avg_train_tokens_per_sec: float | None = None
    final_train_tokens_per_sec: float | None = None
    steady_train_tokens_per_sec: float | None = None
    avg_mfu: float | None = None
    final_mfu: float | None = None
    device_kind: str | None = None
    device_count: int | None = None
    runtime_diagnostics_path: str | None = None
    execution_mode: str | None = None
    metrics_scope: str | None = None
    artifact_writer: str | None = None
    model_remat: str | None = None
    data_axis_size: int | None = None
    global_batch_size: int | None = None
    per_device_batch_size: int | None = None
    gradient_accumulation_steps: int | None = None
    effective_global_batch_size: int | None = None
    micro_tokens_per_step: int | None = None
    effective_tokens_per_step: int | None = None
    selected_device_count: int | None = None
    process_count: int | None = None
    data_pipeline_backend: str | None = None
    data_pipeline_order: str | None = None
    data_pipeline_shuffle_seed: int | None = None
    data_document_aware: bool | None = None
    final_batch_het: float | None = None
    avg_batch_het: float | None = None
    moe_balance_policy: str | None = None
    z_loss_weight: float | None = None
    final_router_max_vio: float | None = None
    final_router_mean_load_cv: float | None = None
    final_router_dead_experts_count: float | None = None
    final_router_mean_importance_cv: float | None = None
    final_router_mean_importance_entropy: float | None = None
    final_optimizer_groups: list[dict[str, Any]] | None = None
    final_optimizer_grad_norm_max_group: str | None = None
    final_optimizer_update_norm_max_group: str | None = None
    final_optimizer_update_param_ratio_max: float | None = None
    final_optimizer_update_param_ratio_mean: float | None = None
    final_optimizer_groups_with_zero_grad: int | None = None
    final_optimizer_groups_with_zero_update: int | None = None
    final_optimizer_nonfinite_group_count: int | None = None
    final_optimizer_nonfinite_groups: list[str] | None = None
    final_optimizer_route_backend_counts: dict[str, int] | None = None
    final_moe_router_layers: list[dict[str, Any]] | None = None
    global_device_count: int | None = None
    process_index: int | None = None
    single_process: bool | None = None
    data_pipeline_version: str | None = None
    data_pipeline_worker_count: int | None = None
    data_pipeline_worker_buffer_size: int | None = None
    data_pipeline_prefetch: bool | None = None
    data_pipeline_state_schema_version: int | None = None
    data_document_count: int | None = None
    data_document_offsets_path: str | None = None
    data_document_offsets_sha256: str | None = None
    data_document_buffer_size: int | None = None
    data_document_refill_size: int | None = None


COMPLETED_EVENT_FIELDS = (
    "target_tokens", "total_wall_sec", "final_train_tokens_per_sec", "avg_train_tokens_per_sec",
    "steady_train_tokens_per_sec", "final_mfu", "avg_mfu", "final_batch_het", "avg_batch_het", "execution_mode",
    "metrics_scope", "artifact_writer", "model_remat", "data_axis_size", "gradient_accumulation_steps",
    "effective_global_batch_size", "effective_tokens_per_step", "per_device_batch_size", "selected_device_count",
    "data_pipeline_backend", "data_pipeline_order", "data_pipeline_shuffle_seed", "data_pipeline_worker_count",
    "data_pipeline_worker_buffer_size", "data_pipeline_prefetch", "data_document_buffer_size",
    "data_document_refill_size", "moe_balance_policy", "z_loss_weight", "final_moe_router_layers",
    "final_router_max_vio", "final_router_mean_load_cv", "final_router_dead_experts_count",
    "final_router_mean_importance_cv", "final_router_mean_importance_entropy", "final_optimizer_groups",
    "final_optimizer_grad_norm_max_group", "final_optimizer_update_norm_max_group",
    "final_optimizer_update_param_ratio_max", "final_optimizer_update_param_ratio_mean",
    "final_optimizer_groups_with_zero_grad", "final_optimizer_groups_with_zero_update",
    "final_optimizer_nonfinite_group_count", "final_optimizer_nonfinite_groups",
    "final_optimizer_route_backend_counts")


def _noop_progress(event: str, payload: dict[str, Any]) -> None:
    return None


def should_log(step: int, tokens_seen: int, spec: RunSpec) -> bool:
    return step % spec.training.log_every_steps == 0 or tokens_seen >= spec.training.target_tokens


def metrics_row(trainer: Trainer, metrics: StepMetrics, spec: RunSpec) -> dict[str, Any]:
    """One ``metrics/train.jsonl`` row (field list: reference runtime/training.py:930-1019)."""

    prov = trainer.last_provenance
    token_count = int(metrics.token_count)
    loss = metrics.loss_sum / max(token_count, 1)
    mb_losses = None
    if metrics.microbatch_loss_sums and metrics.microbatch_token_counts:
        mb_losses = [s / max(c, 1.0) for s, c in zip(metrics.microbatch_loss_sums, metrics.microbatch_token_counts)]
    z_loss = None if metrics.z_loss_sum is None else spec.training.loss.z_loss_weight * metrics.z_loss_sum / max(token_count, 1)
    total = loss + (z_loss or 0.0) + (metrics.aux_loss or 0.0)
    row: dict[str, Any] = {
        "schema_version": 1, "step": trainer.step, "tokens_seen": trainer.tokens_seen, "loss_sum": metrics.loss_sum,
        "token_count": token_count, "loss": loss, "lm_loss": loss, "lr": metrics.lr, "grad_norm": metrics.grad_norm,
        "param_norm": metrics.param_norm, "update_norm": metrics.update_norm, "total_loss": total, "z_loss": z_loss,
        "moe_aux_loss": metrics.moe_aux_loss, "aux_loss": metrics.aux_loss,
    }
    for key in ("router_max_vio", "router_load_min", "router_load_max", "router_load_entropy", "router_mean_load_cv",
                "router_std_load_cv", "router_mean_load_entropy", "router_min_load_entropy",
                "router_dead_experts_count", "router_experts_active_mean", "router_mean_importance_cv",
                "router_mean_importance_entropy", "smebu_bias_norm", "smebu_momentum_norm"):
        row[key] = metrics.router.get(key)
    row["microbatch_loss_mean"] = None if not mb_losses else sum(mb_losses) / len(mb_losses)
    row["microbatch_loss_max"] = None if not mb_losses else max(mb_losses)
    row["batch_het"] = None if not mb_losses else max(mb_losses) - sum(mb_losses) / len(mb_losses)
    row["clip_scale"] = metrics.router.get("clip_scale")
    if prov:
        row.update({"epoch": prov[0].epoch, "token_start": min(p.token_start for p in prov),
                    "token_end": max(p.token_end for p in prov), "examples": sum(p.examples for p in prov),
                    "target_tokens": sum(p.target_tokens for p in prov)})
        doc_ids = [d for p in prov if p.row_doc_ids is not None for d in p.row_doc_ids]
        aware = all(p.row_doc_ids is not None for p in prov)
        row.update({"document_aware": aware, "documents_touched": len(set(doc_ids)) if aware else None,
                    "document_min": min(doc_ids) if aware and doc_ids else None,
                    "document_max": max(doc_ids) if aware and doc_ids else None})
    else:
        t = spec.training
        row.update({"epoch": 0, "token_start": None, "token_end": None,
                    "examples": t.global_batch_size * t.gradient_accumulation_steps,
                    "target_tokens": t.global_batch_size * t.seq_len * t.gradient_accumulation_steps,
                    "document_aware": False, "documents_touched": None, "document_min": None, "document_max": None})
    from research_b200.optim.diagnostics import health_fields, router_layers_payload

    row["moe_router_layers"] = router_layers_payload(metrics.router_layers) if metrics.router_layers else None
    row["optimizer_groups"] = metrics.optimizer_groups or None
    row.update(health_fields(metrics.optimizer_groups))
    t = spec.training
    data_axis = trainer.mesh.size("data") * trainer.mesh.size("fsdp")
    row.update({
        "data_axis_size": data_axis, "global_batch_size": t.global_batch_size,
        "per_device_batch_size": t.global_batch_size // data_axis,
        "gradient_accumulation_steps": t.gradient_accumulation_steps, "micro_global_batch_size": t.global_batch_size,
        "effective_global_batch_size": t.global_batch_size * t.gradient_accumulation_steps,
        "micro_tokens_per_step": t.global_batch_size * t.seq_len, "effective_tokens_per_step": row["target_tokens"],
        "global_target_tokens": row["target_tokens"], "per_device_target_tokens": row["target_tokens"] // data_axis,
        "data_pipeline_backend": "blackwell_native" if spec.data.mode == "prepared" else "hf_streaming",
        "data_order": spec.data.order, "data_worker_count": spec.data.worker_count,
        "data_prefetch": spec.data.prefetch, "data_worker_buffer_size": spec.data.worker_buffer_size,
    })
    return row


def _nonfinite(row: Mapping[str, Any]) -> list[str]:
    bad = []
    for key in ("loss", "grad_norm", "param_norm", "update_norm"):
        v = row.get(key)
        if v is not None and not math.isfinite(float(v)):
            bad.append(key)
    return bad


def run_validation_eval(trainer: Trainer, spec: RunSpec, writer, step: int, tokens_seen: int,
                        progress: ProgressFn) -> dict[str, Any] | None:
    """Fresh pass over the head of the validation split (reference: runtime/training.py:813-927)."""

    if not spec.evals:
        return None
    if len(spec.evals) != 1 or spec.evals[0].name != "validation":
        raise ContractError("runtime supports exactly one eval named 'validation'")
    ev = spec.evals[0]
    writer.append_event({"schema_version": 1, "type": "eval_started", "run_id": spec.run_id, "created_at": utc_now(),
                         "step": step, "name": ev.name, "num_batches": ev.num_batches})
    start = time.perf_counter()
    try:
        result = trainer.evaluate(ev.num_batches)
    except Exception as exc:
        writer.append_event({"schema_version": 1, "type": "eval_failed", "run_id": spec.run_id,
                             "created_at": utc_now(), "step": step, "name": ev.name,
                             "error_type": type(exc).__name__, "error_message": str(exc)})
        raise
    eval_sec = time.perf_counter() - start
    row = {"schema_version": 1, "name": ev.name, "eval_name": ev.name, "step": step, "tokens_seen": tokens_seen,
           "loss_sum": result["loss_sum"], "token_count": int(result["token_count"]), "loss": result["loss"],
           "bpb": result.get("bpb"), "num_batches": result["num_batches"]}
    row.update({k: result.get(k) for k in ("token_start", "token_end", "examples", "target_tokens", "document_aware",
                                           "documents_touched", "document_min", "document_max")})
    row = enrich_eval_metrics(row, eval_sec=eval_sec)
    writer.append_eval_metrics(row)
    writer.append_event({"schema_version": 1, "type": "eval_completed", "run_id": spec.run_id,
                         "created_at": utc_now(), "step": step, "name": ev.name, "loss": row["loss"]})
    progress("eval", {"row": row})
    return row


def _host_state(trainer: Trainer, spec: RunSpec, wall_start_ns: int) -> tuple[dict[str, Any], dict[str, Any]]:
    dataset = trainer.data.state_to_json(trainer.data_state) if hasattr(trainer.data, "state_to_json") else \
        data_pipeline_state_to_dict(trainer.data_state)
    host = {"dataset": dataset, "last_checkpoint_step": trainer.step, "wallclock_start_ns": wall_start_ns,
            "run_id": spec.run_id}
    return dataset, host


def save_checkpoint(trainer: Trainer, spec: RunSpec, service: LocalCheckpointService, writer, index, row, eval_row,
                    reason: str, wall_start_ns: int, compat, progress: ProgressFn):
    start = time.perf_counter()
    # collective: every rank takes part, the arrays are assembled on the writer only, one parameter at a time
    tensors = iter_state_tensors(trainer, writer_only=True)
    dataset, host = _host_state(trainer, spec, wall_start_ns)
    metadata = checkpoint_metadata(spec, row, reason=reason, eval_row=eval_row, compat=compat)
    path = service.save(trainer.step, tensors, dataset, host, metadata)
    if trainer.mesh.world_size > 1:
        torch.distributed.barrier()
    sec = time.perf_counter() - start
    index = record_checkpoint(index, spec.dirs.run_dir, step=trainer.step, tokens_seen=trainer.tokens_seen,
                              checkpoint_path=path, reason=reason, train_loss=float(row["loss"]),
                              eval_loss=None if eval_row is None else float(eval_row["loss"]))
    service.set_protected_steps(index.protected_steps())
    writer.write_checkpoint_index(index.to_dict())
    writer.append_event({"schema_version": 1, "type": "checkpoint_saved", "run_id": spec.run_id,
                         "created_at": utc_now(), "step": trainer.step, "tokens_seen": trainer.tokens_seen,
                         "checkpoint_path": Path(path).as_posix(), "reason": reason, "checkpoint_sec": sec,
                         "data_pipeline_backend": "blackwell_native", "data_pipeline_order": spec.data.order,
                         "data_pipeline_shuffle_seed": spec.data.shuffle_seed})
    progress("checkpoint", {"step": trainer.step, "checkpoint_path": Path(path).as_posix(), "reason": reason,
                            "checkpoint_sec": sec, "eval_loss": None if eval_row is None else eval_row["loss"]})
    return index


def run_training(config_path: str | Path, *, resume: bool = False, progress: ProgressFn | None = None,
                 trainer_hook: Callable[[Trainer], None] | None = None) -> RunSummary:
    progress = progress or _noop_progress
    config_path = Path(config_path)
    spec = load_config(config_path)
    from research_b200.parallel.mesh import init_distributed

    rank, world = init_distributed()
    run_dir = spec.dirs.run_dir
    if resume:
        if not run_dir.is_dir():
            raise ContractError(f"cannot resume: run directory does not exist: {run_dir}")
    elif rank == 0:
        initialize_run(config_path)
    if world > 1:
        torch.distributed.barrier()
    writer = build_artifact_writer(spec, run_dir, is_writer=rank == 0, resume=resume)
    progress("start", {"spec": spec, "config_path": str(config_path), "resume": resume})
    moe = spec.model.trinity.moe if spec.model.trinity is not None else None
    writer.append_event({"schema_version": 1, "type": "training_started", "run_id": spec.run_id,
                         "created_at": utc_now(), "resume": resume, "config_path": config_path.as_posix(),
                         "world_size": world, "execution_mode": runtime_execution_mode(spec),
                         "parallelism_mode": spec.parallelism.mode, "metrics_scope": METRICS_SCOPE,
                         "artifact_writer": ARTIFACT_WRITER, "model_remat": spec.model.remat,
                         "gradient_accumulation_steps": spec.training.gradient_accumulation_steps,
                         "data_pipeline_backend": "blackwell_native" if spec.data.mode == "prepared" else "hf_streaming",
                         "data_pipeline_order": spec.data.order, "data_pipeline_shuffle_seed": spec.data.shuffle_seed,
                         "data_pipeline_worker_count": spec.data.worker_count,
                         "data_pipeline_worker_buffer_size": spec.data.worker_buffer_size,
                         "data_pipeline_prefetch": spec.data.prefetch,
                         "data_document_buffer_size": spec.data.document_buffer_size,
                         "data_document_refill_size": spec.data.document_refill_size,
                         "moe_balance_policy": None if moe is None else moe.balance.name,
                         "z_loss_weight": spec.training.loss.z_loss_weight})
    monitor = None
    if world > 1:
        from research_b200.runtime.watchdog import RankMonitor

        # every rank posts heartbeats to the process group's store; a rank that leaves marks itself failed there
        monitor = RankMonitor(torch.distributed.distributed_c10d._get_default_store(), rank, world,
                              directory=run_dir / "diagnostics" / "heartbeats", writer=writer, run_id=spec.run_id,
                              timeout_s=float(os.environ.get("RESEARCH_B200_RANK_TIMEOUT_S", "300")),
                              poll_s=float(os.environ.get("RESEARCH_B200_RANK_POLL_S", "2"))).start()
    try:
        summary = _run_initialized(spec, config_path, writer, resume, progress, trainer_hook, monitor)
    except Exception as exc:
        if monitor is not None:
            monitor.mark_failed(-1, f"{type(exc).__name__}: {exc}")
            monitor.stop()
        writer.append_event({"schema_version": 1, "type": "training_failed", "run_id": spec.run_id,
                             "created_at": utc_now(), "error_type": type(exc).__name__, "error_message": str(exc),
                             "error": str(exc)})
        writer.close()
        raise
    if monitor is not None:
        monitor.mark_done(summary.steps)
        monitor.stop()
    writer.write_summary(normalize(asdict(summary)))
    completed = normalize(asdict(summary))
    writer.append_event({"schema_version": 1, "type": "training_completed", "run_id": spec.run_id,
                         "created_at": utc_now(), "steps": summary.steps, "tokens_seen": summary.tokens_seen,
                         "final_loss": summary.final_loss,
                         # the run-level figures of the summary, so that the event stream alone tells how a run ended
                         **{k: completed[k] for k in COMPLETED_EVENT_FIELDS}})
    writer.close()
    progress("completed", {"summary": summary})
    return summary


def _run_initialized(spec: RunSpec, config_path: Path, writer, resume: bool, progress: ProgressFn,
                     trainer_hook, monitor=None) -> RunSummary:
    wall_start = time.perf_counter()
    wall_start_ns = time.time_ns()
    trainer = Trainer(spec)
    spec = trainer.spec
    if trainer_hook is not None:
        trainer_hook(trainer)
    run_dir = spec.dirs.run_dir
    policy = optimizer_policy_summary(trainer.optimizer_build, trainer.result.metadata)
    pipeline_description = trainer.data.describe()
    compat = build_resume_compat(spec, optimizer_policy=policy, data_pipeline=pipeline_description)
    runtime = build_runtime_diagnostics(spec, trainer, optimizer_policy=policy, data_pipeline=pipeline_description)
    writer.write_runtime_diagnostics(runtime)
    from research_b200.kernels.registry import require_kernel_plan_supported

    require_kernel_plan_supported(runtime["kernels"], spec)
    progress("initialized", {"spec": spec, "diagnostics": runtime, "run_dir": str(run_dir)})
    profiler = ProfilingManager(spec, run_dir, writer, enabled=trainer.is_writer)
    service = LocalCheckpointService(run_dir, is_writer=trainer.is_writer)
    index = load_checkpoint_index(run_dir)
    service.set_protected_steps(index.protected_steps())

    if resume:
        try:
            metadata = service.restore_latest_metadata()
            validate_resume_metadata(metadata, spec, compat=compat)
            restored = service.restore_latest()
            load_state_tensors(trainer, restored.tensors)
            validate_resume_compat(restored, spec, state_step=trainer.step, state_tokens=trainer.tokens_seen,
                                   compat=compat)
            trainer.data_state = trainer.data.state_from_json(restored.dataset_state)
            wall_start_ns = int(restored.host_state.get("wallclock_start_ns", wall_start_ns))
        except Exception as exc:
            writer.append_event({"schema_version": 1, "type": "checkpoint_restore_failed", "run_id": spec.run_id,
                                 "created_at": utc_now(), "error_type": type(exc).__name__,
                                 "error_message": str(exc)})
            raise
        profiler.check_resume(trainer.step)
        writer.append_event({"schema_version": 1, "type": "training_resumed", "run_id": spec.run_id,
                             "created_at": utc_now(), "checkpoint_step": restored.step, "step": trainer.step,
                             "tokens_seen": trainer.tokens_seen, "checkpoint_path": restored.path.as_posix()})
        progress("resumed", {"checkpoint_step": restored.step, "step": trainer.step,
                             "tokens_seen": trainer.tokens_seen, "checkpoint_path": restored.path.as_posix()})

    target = spec.training.target_tokens
    timer = PhaseTimer()
    rows: list[dict[str, Any]] = []
    last_row: dict[str, Any] | None = None
    last_eval_row: dict[str, Any] | None = None
    last_logged_step = -1
    last_checkpoint_step = index.latest_record.step if index.latest_record is not None else -1
    first = True
    while trainer.tokens_seen < target:
        next_step = trainer.step + 1
        with profiler.step(next_step), timer.phase("train_loop_step"):
            with timer.phase("data"), profiler.annotate("data"):
                batches = trainer.next_accumulated_batch()
            if first:
                progress("compile_start", {"phase": "train"})
                first = False
            diagnostics = should_log(next_step, trainer.tokens_seen + _step_tokens(spec), spec)
            if monitor is not None:
                monitor.check()          # a peer that left between steps is seen here, before the next launch
            with timer.phase("train_step"), profiler.annotate("train_step"):
                metrics = trainer.train_on(batches, diagnostics=diagnostics)
            if monitor is not None:
                monitor.beat(trainer.step)
        timings = timer.reset()
        row = metrics_row(trainer, metrics, spec)
        row = enrich_train_metrics(row, timings=timings, runtime=runtime,
                                   telemetry=device_telemetry(trainer.device) if diagnostics else None)
        last_row = row
        rows.append(row)
        bad = _nonfinite(row)
        if bad:
            writer.append_train_metrics(row)
            from research_b200.runtime.train_debug import find_nonfinite_leaves

            writer.append_event({"schema_version": 1, "type": "optimizer_nonfinite", "run_id": spec.run_id,
                                 "created_at": utc_now(), "step": trainer.step, "fields": bad,
                                 "leaves": find_nonfinite_leaves(trainer)})
            raise ContractError(f"non-finite training metrics at step {trainer.step}: {bad}")
        bad_groups = row.get("optimizer_nonfinite_groups") or []
        if bad_groups:
            from research_b200.runtime.train_debug import find_nonfinite_leaves

            writer.append_train_metrics(row)
            writer.append_event({"schema_version": 1, "type": "optimizer_nonfinite", "run_id": spec.run_id,
                                 "created_at": utc_now(), "step": trainer.step, "tokens_seen": trainer.tokens_seen,
                                 "optimizer_nonfinite_group_count": len(bad_groups),
                                 "optimizer_nonfinite_groups": list(bad_groups),
                                 "leaves": find_nonfinite_leaves(trainer)})
            progress("failed", {"row": row, "optimizer_nonfinite_groups": list(bad_groups)})
            raise ContractError(f"optimizer state became non-finite at step {trainer.step}: {', '.join(bad_groups)}")
        if should_log(trainer.step, trainer.tokens_seen, spec):
            writer.append_train_metrics(row)
            last_logged_step = trainer.step
            progress("train", {"row": row})
        checkpoint_due = trainer.step % spec.training.checkpoint_every_steps == 0
        eval_every = spec.training.eval_every_steps or (spec.evals[0].every_steps if spec.evals else None)
        eval_due = bool(spec.evals) and eval_every is not None and trainer.step % eval_every == 0
        eval_row = None
        if spec.evals and (eval_due or checkpoint_due):
            with profiler.annotate("eval"):
                eval_row = run_validation_eval(trainer, spec, writer, trainer.step, trainer.tokens_seen, progress)
            last_eval_row = eval_row
        if checkpoint_due:
            with profiler.annotate("checkpoint"):
                index = save_checkpoint(trainer, spec, service, writer, index, row, eval_row, "cadence",
                                        wall_start_ns, compat, progress)
            last_checkpoint_step = trainer.step
    if last_row is None:
        raise ContractError("training.target_tokens was already reached; nothing to do")
    if last_logged_step != trainer.step:
        writer.append_train_metrics(last_row)
        progress("train", {"row": last_row})
    final_eval = last_eval_row if (last_eval_row is not None and last_eval_row["step"] == trainer.step) else None
    if spec.evals and final_eval is None:
        final_eval = run_validation_eval(trainer, spec, writer, trainer.step, trainer.tokens_seen, progress)
    if last_checkpoint_step != trainer.step:
        index = save_checkpoint(trainer, spec, service, writer, index, last_row, final_eval, "final", wall_start_ns,
                                compat, progress)
    profiler.finish()
    service.close()
    diag = training_diagnostics_summary(rows)       # wall time and device fields are set on the summary below
    from research_b200.optim.diagnostics import HEALTH_KEYS

    # group norms exist on the steps that computed diagnostics (the logged ones): report the newest of them
    last_groups_row = next((r for r in reversed(rows) if r.get("optimizer_groups")), {})
    latest, best = index.latest_record, index.best_record
    t = spec.training
    data_axis = trainer.mesh.size("data") * trainer.mesh.size("fsdp")
    moe = spec.model.trinity.moe if spec.model.trinity is not None else None
    backend_counts: dict[str, int] = {}
    for a in trainer.optimizer_build.route_assignments:
        backend_counts[a.backend] = backend_counts.get(a.backend, 0) + 1
    return RunSummary(
        run_id=spec.run_id, run_dir=run_dir, status="completed", steps=trainer.step, tokens_seen=trainer.tokens_seen,
        target_tokens=target, final_loss=float(last_row["loss"]),
        final_eval_loss=None if final_eval is None else float(final_eval["loss"]),
        final_eval_token_count=None if final_eval is None else int(final_eval["token_count"]),
        final_eval_num_batches=None if final_eval is None else int(final_eval["num_batches"]),
        latest_checkpoint_path=None if latest is None else latest.checkpoint_path.as_posix(),
        best_eval_step=None if best is None else best.step, best_eval_loss=None if best is None else best.eval_loss,
        best_checkpoint_path=None if best is None else best.checkpoint_path.as_posix(),
        total_wall_sec=time.perf_counter() - wall_start, device_kind=device_kind(trainer.device),
        device_count=trainer.mesh.world_size, runtime_diagnostics_path="diagnostics/runtime.json",
        execution_mode=runtime_execution_mode(spec), metrics_scope=METRICS_SCOPE, artifact_writer=ARTIFACT_WRITER,
        model_remat=spec.model.remat, data_axis_size=data_axis, global_batch_size=t.global_batch_size,
        per_device_batch_size=t.global_batch_size // data_axis,
        gradient_accumulation_steps=t.gradient_accumulation_steps,
        effective_global_batch_size=t.global_batch_size * t.gradient_accumulation_steps,
        micro_tokens_per_step=t.global_batch_size * t.seq_len,
        effective_tokens_per_step=t.global_batch_size * t.seq_len * t.gradient_accumulation_steps,
        selected_device_count=trainer.mesh.world_size, process_count=trainer.mesh.world_size,
        data_pipeline_backend=pipeline_description.get("backend", "blackwell_native"),
        data_pipeline_order=spec.data.order, data_pipeline_shuffle_seed=spec.data.shuffle_seed,
        data_document_aware=bool(last_row.get("document_aware")),
        moe_balance_policy=None if moe is None else moe.balance.name, z_loss_weight=t.loss.z_loss_weight,
        final_router_max_vio=last_row.get("router_max_vio"),
        final_router_mean_load_cv=last_row.get("router_mean_load_cv"),
        final_router_dead_experts_count=last_row.get("router_dead_experts_count"),
        final_router_mean_importance_cv=last_row.get("router_mean_importance_cv"),
        final_router_mean_importance_entropy=last_row.get("router_mean_importance_entropy"),
        final_optimizer_groups=last_groups_row.get("optimizer_groups"),
        **{f"final_{k}": last_groups_row.get(k) for k in HEALTH_KEYS if k != "optimizer_route_backend_counts"},
        final_optimizer_route_backend_counts=backend_counts,
        final_moe_router_layers=next((r["moe_router_layers"] for r in reversed(rows) if r.get("moe_router_layers")),
                                     None),
        global_device_count=trainer.mesh.world_size, process_index=trainer.mesh.rank,
        single_process=trainer.mesh.world_size == 1,
        data_pipeline_version=pipeline_description.get("backend_version"),
        data_pipeline_worker_count=pipeline_description.get("worker_count"),
        data_pipeline_worker_buffer_size=pipeline_description.get("worker_buffer_size"),
        data_pipeline_prefetch=pipeline_description.get("prefetch"),
        data_pipeline_state_schema_version=pipeline_description.get("state_schema_version"),
        data_document_count=pipeline_description.get("document_count"),
        data_document_offsets_path=pipeline_description.get("document_offsets_path"),
        data_document_offsets_sha256=pipeline_description.get("document_offsets_sha256"),
        data_document_buffer_size=pipeline_description.get("document_buffer_size"),
        data_document_refill_size=pipeline_description.get("document_refill_size"), **diag,
    )


def _step_tokens(spec: RunSpec) -> int:
    t = spec.training
    return t.global_batch_size * t.seq_len * t.gradient_accumulation_steps
