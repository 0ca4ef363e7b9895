"""``diagnostics/runtime.json``, per-step timing / throughput / MFU enrichment, device telemetry.

Keeps the reference's payload keys (src/jaxtitan/runtime/diagnostics.py:180-311, 634-686) with ``packages`` /
``runtime`` describing torch, CUDA and NCCL instead of JAX.  ``mfu`` uses the reference's dense FLOP formula and the
nominal per-device peak (B200: 2.25e15); ``mfu_exact`` counts the parameters a token really visits.
"""

from __future__ import annotations

import platform
import sys
import time
from contextlib import contextmanager
from typing import Any, Mapping

import torch

from research_b200 import __version__
from research_b200.config.canonical import normalize
from research_b200.config.specs import RunSpec
from research_b200.runtime.flops import estimate_flops_per_token, estimate_flops_per_token_exact, peak_flops_for_device
from research_b200.services.artifacts import utc_now

METRICS_SCOPE = "global"
ARTIFACT_WRITER = "single_host"
EXECUTION_MODE = "one_process_per_gpu"


class PhaseTimer:
    """Accumulates wall-clock seconds per named phase of one step (reference: diagnostics.py:82-107)."""

    def __init__(self) -> None:
        self.seconds: dict[str, float] = {}

    @contextmanager
    def phase(self, name: str):
        start = time.perf_counter()
        try:
            yield
        finally:
            self.seconds[name] = self.seconds.get(name, 0.0) + time.perf_counter() - start

    def reset(self) -> dict[str, float]:
        out, self.seconds = self.seconds, {}
        return out


def device_kind(device: torch.device) -> str:
    if device.type == "cuda":
        return torch.cuda.get_device_name(device)
    return platform.processor() or "cpu"


def device_telemetry(device: torch.device) -> dict[str, Any]:
    out: dict[str, Any] = {"device_memory_used_bytes": None, "device_memory_peak_bytes": None,
                           "device_memory_limit_bytes": None, "nvml_memory_used_bytes": None,
                           "nvml_memory_total_bytes": None, "nvml_gpu_utilization": None,
                           "nvml_memory_utilization": None, "nvml_power_watts": None, "nvml_temperature_c": None}
    if device.type != "cuda":
        return out
    out["device_memory_used_bytes"] = int(torch.cuda.memory_allocated(device))
    out["device_memory_peak_bytes"] = int(torch.cuda.max_memory_allocated(device))
    out["device_memory_limit_bytes"] = int(torch.cuda.get_device_properties(device).total_memory)
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(device.index or 0)
        mem = pynvml.nvmlDeviceGetMemoryInfo(handle)
        util = pynvml.nvmlDeviceGetUtilizationRates(handle)
        out.update(nvml_memory_used_bytes=int(mem.used), nvml_memory_total_bytes=int(mem.total),
                   nvml_gpu_utilization=float(util.gpu), nvml_memory_utilization=float(util.memory),
                   nvml_power_watts=pynvml.nvmlDeviceGetPowerUsage(handle) / 1000.0,
                   nvml_temperature_c=float(pynvml.nvmlDeviceGetTemperature(handle, pynvml.NVML_TEMPERATURE_GPU)))
    except Exception:
        pass
    return out


def build_runtime_diagnostics(spec: RunSpec, trainer, *, optimizer_policy: Mapping[str, Any] | None = None,
                              data_pipeline: Mapping[str, Any] | None = None,
                              wandb: Mapping[str, Any] | None = None) -> dict[str, Any]:
    mesh = trainer.mesh
    t = spec.training
    kind = device_kind(trainer.device)
    peak = peak_flops_for_device(kind)
    micro_tokens = t.global_batch_size * t.seq_len
    data_axis = mesh.size("data") * mesh.size("fsdp")
    from research_b200.kernels.registry import kernel_plan

    payload = {
        "schema_version": 1,
        "created_at": utc_now(),
        "run_id": spec.run_id,
        "python": sys.version.split()[0],
        "packages": {"research_b200": __version__, "torch": torch.__version__,
                     "cuda": torch.version.cuda, "nccl": _nccl_version()},
        "runtime": {"backend": trainer.device.type, "world_size": mesh.world_size, "rank": mesh.rank,
                    "device_kind": kind, "selected_device_count": mesh.world_size,
                    "global_device_count": mesh.world_size, "process_count": mesh.world_size,
                    "process_index": mesh.rank, "single_process": mesh.world_size == 1,
                    "execution_mode": EXECUTION_MODE},
        "mesh": {"axis_names": list(mesh.axis_names), "axis_sizes": list(mesh.axis_sizes),
                 "device_count": mesh.world_size, "data_axis_size": data_axis,
                 "global_batch_size": t.global_batch_size, "per_device_batch_size": t.global_batch_size // data_axis,
                 "gradient_accumulation_steps": t.gradient_accumulation_steps,
                 "effective_global_batch_size": t.global_batch_size * t.gradient_accumulation_steps,
                 "micro_tokens_per_step": micro_tokens,
                 "effective_tokens_per_step": micro_tokens * t.gradient_accumulation_steps},
        "model": {"name": spec.model.name, "variant": spec.model.variant, "parameters": trainer.parameter_count(),
                  "remat": spec.model.remat, "compute_dtype": spec.model.compute_dtype,
                  "param_dtype": spec.model.param_dtype, "tied_embeddings": spec.model.tied_embeddings},
        "training": {"precision": t.precision, "seq_len": t.seq_len, "target_tokens": t.target_tokens,
                     "z_loss_weight": t.loss.z_loss_weight},
        "optimizer": normalize(optimizer_policy),
        "performance": {"flops_per_token": estimate_flops_per_token(spec.model, t.seq_len),
                        "flops_per_token_exact": estimate_flops_per_token_exact(spec.model, t.seq_len),
                        "peak_flops_per_device": peak,
                        "peak_flops_total": None if peak is None else peak * mesh.world_size},
        "compile": {"train": {"expected_batch_shape": [t.gradient_accumulation_steps, t.global_batch_size, t.seq_len],
                              "mode": "eager_kernels"}},
        "parallelism": {"mode": spec.parallelism.mode, "execution_mode": EXECUTION_MODE,
                        "tensor_parallel": spec.parallelism.tensor_parallel,
                        "context_parallel": spec.parallelism.context_parallel,
                        "expert_parallel": spec.parallelism.expert_parallel,
                        "expert_parallel_axis": trainer.execution.ep_axis_name,
                        "expert_parallel_dispatcher": trainer.execution.ep_dispatcher,
                        "sequence_parallel": trainer.execution.sp},
        "profiling": normalize(spec.profiling),
        "kernels": kernel_plan(spec, device=trainer.device),
        "sharding": trainer.store.describe(),
        "data_pipeline": normalize(data_pipeline),
        "wandb": normalize(wandb),
        "device_telemetry": device_telemetry(trainer.device),
        "metrics_scope": METRICS_SCOPE,
        "artifact_writer": ARTIFACT_WRITER,
    }
    return normalize(payload)


def _nccl_version() -> str | None:
    try:
        return ".".join(str(v) for v in torch.cuda.nccl.version())
    except Exception:
        return None


def _rate(count: float, seconds: float) -> float | None:
    return None if seconds <= 0 else count / seconds


def enrich_train_metrics(row: Mapping[str, Any], *, timings: Mapping[str, float], runtime: Mapping[str, Any],
                         telemetry: Mapping[str, Any] | None = None) -> dict[str, Any]:
    perf = runtime["performance"]
    data_sec = float(timings.get("data", 0.0))
    placement_sec = float(timings.get("placement", 0.0))
    dispatch_sec = float(timings.get("train_step", 0.0))
    sync_sec = float(timings.get("metrics_sync", 0.0))
    train_step_sec = dispatch_sec + sync_sec
    step_sec = float(timings.get("train_loop_step", data_sec + placement_sec + train_step_sec))
    tokens = int(row["target_tokens"])
    tps = _rate(tokens, train_step_sec)
    fps = None if tps is None else perf["flops_per_token"] * tps
    fps_exact = None if tps is None else perf["flops_per_token_exact"] * tps
    peak_total = perf["peak_flops_total"]
    out = dict(row)
    out.update({
        "parallelism_mode": runtime["parallelism"]["mode"], "execution_mode": EXECUTION_MODE,
        "metrics_scope": METRICS_SCOPE, "artifact_writer": ARTIFACT_WRITER,
        "data_sec": data_sec, "placement_sec": placement_sec, "train_dispatch_sec": dispatch_sec,
        "metrics_sync_sec": sync_sec, "train_step_sec": train_step_sec, "step_sec": step_sec,
        "tokens_per_sec": _rate(tokens, step_sec), "train_tokens_per_sec": tps,
        "examples_per_sec": _rate(int(row["examples"]), step_sec),
        "flops_per_token": perf["flops_per_token"], "flops_per_step": perf["flops_per_token"] * tokens,
        "flops_per_sec": fps, "peak_flops_per_device": perf["peak_flops_per_device"], "peak_flops_total": peak_total,
        "mfu": None if fps is None or not peak_total else 100.0 * fps / peak_total,
        "mfu_exact": None if fps_exact is None or not peak_total else 100.0 * fps_exact / peak_total,
    })
    out.update(telemetry or runtime.get("device_telemetry") or {})
    return normalize(out)


def training_diagnostics_summary(rows: list[Mapping[str, Any]]) -> dict[str, Any]:
    """Run-level averages; "steady" drops the first row (reference: diagnostics.py:703-733)."""

    def mean(key: str, subset) -> float | None:
        vals = [float(r[key]) for r in subset if r.get(key) is not None]
        return sum(vals) / len(vals) if vals else None

    steady = rows[1:] if len(rows) > 1 else rows
    return {
        "avg_train_tokens_per_sec": mean("train_tokens_per_sec", rows),
        "final_train_tokens_per_sec": rows[-1].get("train_tokens_per_sec") if rows else None,
        "steady_train_tokens_per_sec": mean("train_tokens_per_sec", steady),
        "avg_mfu": mean("mfu", rows),
        "final_mfu": rows[-1].get("mfu") if rows else None,
        "avg_batch_het": mean("batch_het", rows),
        "final_batch_het": rows[-1].get("batch_het") if rows else None,
    }
