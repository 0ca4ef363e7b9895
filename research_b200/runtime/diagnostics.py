"""``diagnostics/runtime.json``, per-step timing / throughput / MFU enrichment, device telemetry.

Keeps the reference's payload keys (src/jaxtitan/runtime/diagnostics.py:180-311, 634-686) with ``packages`` /
``runtime`` describing torch, CUDA and NCCL instead of JAX.  ``mfu`` uses the reference's dense FLOP formula and the
nominal per-device peak (B200: 2.25e15); ``mfu_exact`` counts the parameters a token really visits.
"""

from __future__ import annotations

import math
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
EXECUTION_MODE = "replicated_data_parallel"


class PhaseTimer:
    """Accumulates wall-clock seconds per named phase of one step (reference: diagnostics.py:82-107)."""

    def __init__(self) -> None:
        self.seconds: dict[str, float] = {}
        self._started_at = time.perf_counter()

    @contextmanager
    def phase(self, name: str):
        start = time.perf_counter()
        try:
            yield
        finally:
            self.seconds[name] = self.seconds.get(name, 0.0) + time.perf_counter() - start

    def add(self, name: str, seconds: float) -> None:
        self.seconds[name] = self.seconds.get(name, 0.0) + float(seconds)

    def get(self, name: str) -> float:
        return self.seconds.get(name, 0.0)

    def total_sec(self) -> float:
        """Wall-clock seconds since construction or the last :meth:`reset`."""

        return time.perf_counter() - self._started_at

    def to_dict(self) -> dict[str, float]:
        return dict(self.seconds)

    def reset(self) -> dict[str, float]:
        out, self.seconds = self.seconds, {}
        self._started_at = time.perf_counter()
        return out


def device_kind(device: torch.device) -> str:
    if device.type == "cuda":
        return torch.cuda.get_device_name(device)
    return platform.processor() or "cpu"


_NVML_UNSET = object()
TELEMETRY_KEYS = ("device_memory_used_bytes", "device_memory_peak_bytes", "device_memory_limit_bytes",
                  "gpu_memory_used_bytes", "gpu_memory_total_bytes", "gpu_utilization_pct",
                  "gpu_memory_utilization_pct", "gpu_power_w", "gpu_temperature_c")


def _load_nvml():
    try:
        import pynvml
    except Exception:
        return None
    return pynvml


def sample_nvml(indices, *, provider: Any = _NVML_UNSET) -> dict[str, Any]:
    """Board counters of the GPUs ``indices`` through NVML (read only): memory and power summed, utilisation averaged,
    the hottest temperature.  Every query may fail on its own; what cannot be read stays ``None``
    (reference: src/jaxtitan/runtime/diagnostics.py:806-861).  ``provider`` replaces the ``pynvml`` module in tests."""

    out: dict[str, Any] = {k: None for k in TELEMETRY_KEYS[3:]}
    nvml = _load_nvml() if provider is _NVML_UNSET else provider
    indices = list(indices)
    if nvml is None or not indices:
        return out
    try:
        nvml.nvmlInit()
        handles = [nvml.nvmlDeviceGetHandleByIndex(i) for i in indices]
    except Exception:
        return out
    used = total = 0
    power = 0.0
    gpu_util, mem_util, temps = [], [], []
    for h in handles:
        try:
            mem = nvml.nvmlDeviceGetMemoryInfo(h)
            used, total = used + int(mem.used), total + int(mem.total)
        except Exception:
            pass
        try:
            util = nvml.nvmlDeviceGetUtilizationRates(h)
            gpu_util.append(float(util.gpu))
            mem_util.append(float(util.memory))
        except Exception:
            pass
        try:
            power += float(nvml.nvmlDeviceGetPowerUsage(h)) / 1000.0
        except Exception:
            pass
        try:
            temps.append(float(nvml.nvmlDeviceGetTemperature(h, nvml.NVML_TEMPERATURE_GPU)))
        except Exception:
            pass
    if total:
        out["gpu_memory_used_bytes"], out["gpu_memory_total_bytes"] = used, total
    if gpu_util:
        out["gpu_utilization_pct"] = sum(gpu_util) / len(gpu_util)
        out["gpu_memory_utilization_pct"] = sum(mem_util) / len(mem_util)
    if power:
        out["gpu_power_w"] = power
    if temps:
        out["gpu_temperature_c"] = max(temps)
    return out


def sample_device_telemetry(device: torch.device, *, nvml_provider: Any = _NVML_UNSET) -> dict[str, Any]:
    """Allocator figures of this process and NVML counters of its GPU; explicit nulls where there is no GPU."""

    out: dict[str, Any] = {k: None for k in TELEMETRY_KEYS}
    if device.type != "cuda":
        if nvml_provider is not _NVML_UNSET:
            out.update(sample_nvml([0], provider=nvml_provider))
        return out
    out["device_memory_used_bytes"] = int(torch.cuda.memory_allocated(device))
    out["device_memory_peak_bytes"] = int(torch.cuda.max_memory_allocated(device))
    out["device_memory_limit_bytes"] = int(torch.cuda.get_device_properties(device).total_memory)
    out.update(sample_nvml([device.index or 0], provider=nvml_provider))
    return out


device_telemetry = sample_device_telemetry


def runtime_execution_mode(spec: RunSpec) -> str:
    """Artifact-facing name of how the run is laid out: the state mode plus the activation axes in use
    (reference: diagnostics.py:736-750)."""

    extra = [name for name, on in (("ep", spec.parallelism.expert_parallel), ("tp", spec.parallelism.tensor_parallel),
                                   ("cp", spec.parallelism.context_parallel)) if on]
    if spec.parallelism.mode in ("zero2", "fsdp"):
        return "+".join([spec.parallelism.mode, *extra])
    return "+".join([EXECUTION_MODE, *extra])


def moe_balance_payload(spec: RunSpec) -> dict[str, Any]:
    trinity = spec.model.trinity
    if trinity is None or trinity.moe is None:
        return {"name": "none"}
    b = trinity.moe.balance
    return {"name": b.name, "load_lr": b.load_lr, "momentum": b.momentum, "clamp": b.clamp,
            "sequence_aux_loss_weight": b.sequence_aux_loss_weight}


def batch_summary(spec: RunSpec, data_axis: int) -> dict[str, int]:
    t = spec.training
    micro = t.global_batch_size * t.seq_len
    step = micro * t.gradient_accumulation_steps
    return {"global_batch_size": t.global_batch_size, "micro_global_batch_size": t.global_batch_size,
            "effective_global_batch_size": t.global_batch_size * t.gradient_accumulation_steps,
            "gradient_accumulation_steps": t.gradient_accumulation_steps,
            "per_device_batch_size": t.global_batch_size // data_axis,
            "micro_tokens_per_step": micro, "effective_tokens_per_step": step, "global_tokens_per_step": step,
            "per_device_tokens_per_step": step // data_axis}


def mesh_summary(spec: RunSpec, mesh) -> dict[str, Any]:
    data_axis = mesh.size("data") * mesh.size("fsdp")
    out = {"axis_names": list(mesh.axis_names), "axis_sizes": list(mesh.axis_sizes),
           "data_axis_size": data_axis, "data_replica_axis_size": mesh.size("data"),
           "fsdp_axis_size": mesh.size("fsdp"), "ep_axis_size": mesh.size("ep"), "tp_axis_size": mesh.size("tp"),
           "cp_axis_size": mesh.size("cp"), "expert_fsdp_axis_size": mesh.size("expert_fsdp"),
           "global_mesh_size": math.prod(int(n) for n in mesh.axis_sizes),
           "device_count": mesh.world_size, "selected_device_count": mesh.world_size,
           "rank": mesh.rank, "coords": dict(mesh.coords)}
    out.update(batch_summary(spec, data_axis))
    return out


def parallelism_summary(spec: RunSpec, mesh, execution) -> dict[str, Any]:
    """What each activation axis does in this run, in words a dashboard can group by
    (reference: diagnostics.py:315-423; the values name this stack's strategies)."""

    from research_b200.config.specs import resolve_expert_fsdp_axis, resolve_expert_parallel_axis

    par = spec.parallelism
    sizes = mesh.sizes
    ep = resolve_expert_parallel_axis(par, sizes)
    efsdp = resolve_expert_fsdp_axis(par, sizes)
    moe = spec.model.trinity.moe if spec.model.trinity is not None else None
    data_axis = mesh.size("data") * mesh.size("fsdp")
    tp, cp = par.tensor_parallel, par.context_parallel
    vocab_parallel = bool(getattr(execution, "vocab_parallel", False))
    fused = bool(getattr(execution, "fused", False)) and mesh.device.type == "cuda"
    return {
        "schema_version": 1, "mode": par.mode, "tensor_parallel": tp, "context_parallel": cp,
        "expert_parallel": par.expert_parallel,
        "tensor_parallel_policy": {
            "enabled": tp, "axis": "tp" if tp else None, "axis_size": mesh.size("tp") if tp else 1,
            "residual_stream": "replicated" if not tp else ("cp_sequence_parallel" if cp else "sequence_parallel"),
            "sequence_parallel": {"enabled": bool(execution.sp),
                                  "activation_spec": "batch,tp_sequence,hidden" if execution.sp else None},
            "embedding": "replicated",
            "lm_head": "replicated" if not tp else ("vocab_parallel" if vocab_parallel else "token_parallel"),
            "loss_parallel": {"enabled": tp,
                              "mode": None if not tp else ("exact_vocab_parallel" if vocab_parallel
                                                           else "token_parallel_fused_cross_entropy")},
            "linears": None if not tp else ("all_gather_gemm_and_gemm_reduce_scatter_kernels" if fused
                                            else "library_collectives"),
            "routed_experts": "not_tensor_parallel_sharded",
            "optimizer": "muon_routes_to_dist_muon" if tp else None,
        },
        "context_parallel_policy": {
            "enabled": cp, "axis": "cp" if cp else None, "axis_size": mesh.size("cp") if cp else 1,
            "attention": None if not cp else execution.cp_attention,
            "sequence_layout": "zigzag" if cp else None,
            "activation_spec": "batch,cp_sequence,hidden" if cp else None,
            "batch_sharding": "batch,cp_sequence" if cp else None,
        },
        "expert_parallel_policy": {
            "enabled": par.expert_parallel, "axis": ep.axis, "axis_size": ep.axis_size,
            "axis_sharing": ep.axis_sharing, "expert_fsdp_axis": efsdp.axis,
            "expert_fsdp_axis_size": efsdp.axis_size, "expert_fsdp_axis_sharing": efsdp.axis_sharing,
            "num_experts": None if moe is None else moe.num_experts,
            "experts_per_rank": None if moe is None or not par.expert_parallel else moe.num_experts // ep.axis_size,
            "dispatcher_backend": execution.ep_dispatcher if par.expert_parallel else None,
        },
        "execution_mode": runtime_execution_mode(spec), "metrics_scope": METRICS_SCOPE,
        "artifact_writer": ARTIFACT_WRITER, "single_process": mesh.world_size == 1,
        "process": {"count": mesh.world_size, "index": mesh.rank, "model": "one_process_per_gpu"},
        "devices": {"selected": mesh.world_size, "local": mesh.world_size, "global": mesh.world_size,
                    "addressable": 1},
        "mesh": {"axis_names": list(mesh.axis_names), "axis_sizes": list(mesh.axis_sizes),
                 "data_axis_size": data_axis, "fsdp_axis_size": mesh.size("fsdp"), "ep_axis_size": mesh.size("ep"),
                 "tp_axis_size": mesh.size("tp"), "cp_axis_size": mesh.size("cp"),
                 "tensor_parallel_axis": "tp" if tp else None, "context_parallel_axis": "cp" if cp else None,
                 "expert_parallel_axis": ep.axis, "expert_parallel_axis_size": ep.axis_size,
                 "expert_parallel_axis_sharing": ep.axis_sharing, "expert_fsdp_axis": efsdp.axis,
                 "expert_fsdp_axis_size": efsdp.axis_size},
        "batch": batch_summary(spec, data_axis),
        "host_artifacts": {"writer": ARTIFACT_WRITER, "records": METRICS_SCOPE},
        # kept at the top level for readers of earlier artifacts
        "expert_parallel_axis": execution.ep_axis_name, "expert_parallel_dispatcher": execution.ep_dispatcher,
        "sequence_parallel": bool(execution.sp),
    }


def compile_contract_summary(spec: RunSpec, mesh) -> dict[str, Any]:
    """The fixed input contract of a train and an eval step: shapes, which mesh axes split which batch dimension,
    and whether the step updates the state in place (reference: diagnostics.py:274-312; there is no tracing compiler
    here, the contract is what the step functions check on entry)."""

    t = spec.training
    rows = [a for a in ("data", "fsdp") if mesh.size(a) > 1]
    seq = ["cp"] if mesh.size("cp") > 1 and spec.parallelism.context_parallel else []
    split = {name: {"rows": rows, "sequence": seq} for name in ("input_ids", "target_ids", "loss_mask", "doc_ids")}
    return {
        "schema_version": 1, "mode": "eager_kernels",
        "train": {"donate_state": True,
                  "expected_batch_shape": [t.gradient_accumulation_steps, t.global_batch_size, t.seq_len],
                  "input_shardings": split},
        "eval": {"donate_state": False, "expected_batch_shape": [t.global_batch_size, t.seq_len],
                 "input_shardings": split},
    }


def build_runtime_diagnostics(spec: RunSpec, trainer, *, optimizer_policy: Mapping[str, Any] | None = None,
                              data_pipeline: Mapping[str, Any] | None = None,
                              wandb: Mapping[str, Any] | None = None) -> dict[str, Any]:
    mesh = trainer.mesh
    t = spec.training
    kind = device_kind(trainer.device)
    peak = peak_flops_for_device(kind)
    from research_b200.kernels.registry import kernel_plan

    payload = {
        "schema_version": 1,
        "created_at": utc_now(),
        "run_id": spec.run_id,
        "python": {"version": platform.python_version(), "implementation": platform.python_implementation(),
                   "executable": sys.executable},
        "packages": {"research_b200": __version__, "torch": torch.__version__,
                     "cuda": torch.version.cuda, "nccl": _nccl_version()},
        "runtime": {"backend": trainer.device.type, "world_size": mesh.world_size, "rank": mesh.rank,
                    "device_kind": kind, "selected_device_count": mesh.world_size,
                    "global_device_count": mesh.world_size, "process_count": mesh.world_size,
                    "process_index": mesh.rank, "single_process": mesh.world_size == 1,
                    "execution_mode": runtime_execution_mode(spec)},
        "mesh": mesh_summary(spec, mesh),
        "model": {"name": spec.model.name, "variant": spec.model.variant, "parameters": trainer.parameter_count(),
                  "parameter_leaves": len(trainer.result.metadata), "seq_len": t.seq_len,
                  "global_batch_size": t.global_batch_size,
                  "effective_global_batch_size": t.global_batch_size * t.gradient_accumulation_steps,
                  "gradient_accumulation_steps": t.gradient_accumulation_steps,
                  "remat": spec.model.remat, "compute_dtype": spec.model.compute_dtype,
                  "param_dtype": spec.model.param_dtype, "tied_embeddings": spec.model.tied_embeddings,
                  "moe_balance": moe_balance_payload(spec)},
        "training": {"precision": t.precision, "seq_len": t.seq_len, "target_tokens": t.target_tokens,
                     "z_loss_weight": t.loss.z_loss_weight, "loss": {"z_loss_weight": t.loss.z_loss_weight}},
        "optimizer": normalize(optimizer_policy),
        "performance": {"device_kind": kind, "device_count": mesh.world_size,
                        "flops_per_token": estimate_flops_per_token(spec.model, t.seq_len),
                        "flops_per_token_exact": estimate_flops_per_token_exact(spec.model, t.seq_len),
                        "peak_flops_per_device": peak,
                        "peak_flops_total": None if peak is None else peak * mesh.world_size},
        "compile": compile_contract_summary(spec, mesh),
        "parallelism": parallelism_summary(spec, mesh, trainer.execution),
        "profiling": normalize(spec.profiling),
        "kernels": kernel_plan(spec, device=trainer.device),
        "sharding": trainer.store.describe(),
        "data_pipeline": normalize(data_pipeline),
        "wandb": normalize(wandb),
        "device_telemetry": sample_device_telemetry(trainer.device),
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
    """Timing, throughput, MFU and telemetry fields of a train row.  ``timings`` takes the phase names of
    :class:`PhaseTimer` (``data``, ``placement``, ``train_step``, ``metrics_sync``, ``train_loop_step``) or the
    reference's ``*_sec`` names (diagnostics.py:634-686)."""

    def sec(short: str, long: str, default: float = 0.0) -> float:
        return float(timings.get(long, timings.get(short, default)))

    perf = runtime["performance"]
    parallelism = runtime.get("parallelism") or {"mode": "ddp", "execution_mode": EXECUTION_MODE}
    data_sec = sec("data", "data_sec")
    placement_sec = sec("placement", "placement_sec")
    dispatch_sec = sec("train_step", "train_dispatch_sec")
    sync_sec = sec("metrics_sync", "metrics_sync_sec")
    train_step_sec = float(timings.get("train_step_sec", dispatch_sec + sync_sec))
    step_sec = sec("train_loop_step", "step_sec", data_sec + placement_sec + train_step_sec)
    tokens = int(row["target_tokens"])
    tps = _rate(tokens, train_step_sec)
    fps = None if tps is None else perf["flops_per_token"] * tps
    exact = perf.get("flops_per_token_exact")
    fps_exact = None if tps is None or exact is None else exact * tps
    peak_total = perf["peak_flops_total"]
    out = dict(row)
    out.update({
        "parallelism_mode": parallelism["mode"],
        "execution_mode": parallelism.get("execution_mode", EXECUTION_MODE),
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
    source = telemetry or runtime.get("device_telemetry") or {}
    out.update({k: source.get(k) for k in TELEMETRY_KEYS})
    return normalize(out)


def enrich_eval_metrics(row: Mapping[str, Any], *, eval_sec: float) -> dict[str, Any]:
    """Validation timing and throughput fields (reference: diagnostics.py:689-700)."""

    out = dict(row)
    out.update({"eval_sec": eval_sec, "eval_tokens_per_sec": _rate(int(row["target_tokens"]), eval_sec),
                "eval_examples_per_sec": _rate(int(row["examples"]), eval_sec)})
    return normalize(out)


def _number(value: Any) -> float | None:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        return None
    return float(value)


def _mean(values) -> float | None:
    vals = [v for v in (_number(x) for x in values) if v is not None]
    return sum(vals) / len(vals) if vals else None


def training_diagnostics_summary(rows: list[Mapping[str, Any]], *, total_wall_sec: float | None = None,
                                 runtime: Mapping[str, Any] | None = None) -> dict[str, Any]:
    """Run-level averages over the rows of a run; "steady" leaves out the first row, which carries the one-time
    start-up cost, and is null for a single row (reference: diagnostics.py:703-733)."""

    final = rows[-1] if rows else {}
    steady = rows[1:] if len(rows) >= 2 else ()
    out = {
        "avg_train_tokens_per_sec": _mean(r.get("train_tokens_per_sec") for r in rows),
        "final_train_tokens_per_sec": _number(final.get("train_tokens_per_sec")),
        "steady_train_tokens_per_sec": _mean(r.get("train_tokens_per_sec") for r in steady),
        "avg_mfu": _mean(r.get("mfu") for r in rows),
        "final_mfu": _number(final.get("mfu")),
        "avg_batch_het": _mean(r.get("batch_het") for r in rows),
        "final_batch_het": _number(final.get("batch_het")),
    }
    if total_wall_sec is not None:
        out["total_wall_sec"] = float(total_wall_sec)
    if runtime is not None:
        perf = runtime["performance"]
        out.update({"device_kind": perf.get("device_kind"), "device_count": perf.get("device_count"),
                    "runtime_diagnostics_path": "diagnostics/runtime.json",
                    "execution_mode": (runtime.get("parallelism") or {}).get("execution_mode", EXECUTION_MODE),
                    "metrics_scope": METRICS_SCOPE, "artifact_writer": ARTIFACT_WRITER})
    return out
