"""Offline analysis of profiling runs: steady-window medians, paired deltas, GPU kernel categories.

Same measurement policy as the reference analyzer (src/jaxtitan/runtime/profile_analysis.py:68-97, 141-324): every
directory below ``root`` that holds ``metrics/train.jsonl`` is a run; the steady window starts after
``max(warmup_steps + 1, trace_end_step + 1)`` and skips steps that ran an eval or a checkpoint; scalars are reduced
with the median; runs are paired by name (``..._muon`` vs ``..._adamw``, same prefix) for percentage deltas.  Where
the reference categorises XLA/HLO ops and Perfetto GPU:0 events, this one categorises CUDA kernels of a Chrome /
Perfetto trace written by ``torch.profiler`` (GEMM, attention, NCCL, element-wise, optimizer, other) and counts
collectives by NCCL kernel name.
"""

from __future__ import annotations

import json
import re
import statistics
from collections import Counter, defaultdict
from pathlib import Path
from typing import Any, Mapping

from research_b200.errors import ContractError

PROFILE_ANALYSIS_SCHEMA_VERSION = 1
_EXCLUDED_EVENT_TYPES = {"checkpoint_saved", "eval_completed"}
_SCALARS = ("train_step_sec", "step_sec", "data_sec", "train_tokens_per_sec", "tokens_per_sec", "mfu", "mfu_exact",
            "loss", "grad_norm")
_KERNEL_CATEGORIES = (
    ("nccl", re.compile(r"nccl|AllReduce|AllGather|ReduceScatter|SendRecv|all_to_all", re.I)),
    ("gemm", re.compile(r"gemm|cutlass|cublas|sm100_xmma|matmul", re.I)),
    ("attention", re.compile(r"attn|attention|flash|fmha", re.I)),
    ("optimizer", re.compile(r"adamw|muon|sumsq|newton", re.I)),
    ("norm_rope_act", re.compile(r"rmsnorm|qknorm|rope|swiglu|sigmoid_gate|embedding|ce_fwd", re.I)),
    ("elementwise", re.compile(r"elementwise|vectorized|copy|fill|reduce_kernel|index", re.I)),
)


def discover_profile_runs(root: str | Path) -> list[Path]:
    root = Path(root)
    found = {p.parent.parent for p in root.rglob("metrics/train.jsonl") if p.is_file()}
    return sorted(found, key=lambda p: p.as_posix())


def _read_jsonl(path: Path) -> list[dict[str, Any]]:
    rows = []
    if not path.is_file():
        return rows
    for line in path.read_text().splitlines():
        if line.strip():
            rows.append(json.loads(line))
    return rows


def categorize_kernel(name: str) -> str:
    for cat, pattern in _KERNEL_CATEGORIES:
        if pattern.search(name):
            return cat
    return "other"


def summarize_trace(path: Path) -> dict[str, Any]:
    """Per-category GPU kernel time and NCCL collective counts from a Chrome-trace JSON."""

    try:
        raw = json.loads(path.read_text())
    except (OSError, json.JSONDecodeError) as exc:
        raise ContractError(f"failed to read trace {path}: {exc}") from exc
    events = raw.get("traceEvents", raw) if isinstance(raw, Mapping) else raw
    time_us: Counter[str] = Counter()
    counts: Counter[str] = Counter()
    collectives: Counter[str] = Counter()
    top: Counter[str] = Counter()
    for ev in events:
        if not isinstance(ev, Mapping) or ev.get("ph") != "X":
            continue
        cat = str(ev.get("cat", "")).lower()
        if "kernel" not in cat and cat != "gpu_memcpy":
            continue
        name = str(ev.get("name", ""))
        dur = float(ev.get("dur", 0.0))
        k = categorize_kernel(name)
        time_us[k] += dur
        counts[k] += 1
        top[name[:96]] += dur
        if k == "nccl":
            for kind in ("AllGather", "ReduceScatter", "AllReduce", "SendRecv", "Broadcast"):
                if kind.lower() in name.lower():
                    collectives[kind] += 1
    total = sum(time_us.values())
    return {"trace": path.name, "gpu_time_us": dict(sorted(time_us.items())), "kernel_counts": dict(sorted(counts.items())),
            "gpu_time_share": {k: (v / total if total else 0.0) for k, v in sorted(time_us.items())},
            "collective_counts": dict(sorted(collectives.items())),
            "top_kernels": [{"name": n, "time_us": t} for n, t in top.most_common(10)], "total_gpu_time_us": total}


def _analyze_run(run_dir: Path, warmup_steps: int) -> dict[str, Any]:
    rows = _read_jsonl(run_dir / "metrics" / "train.jsonl")
    events = _read_jsonl(run_dir / "events.jsonl")
    profiling = {}
    prof_path = run_dir / "diagnostics" / "profiling.json"
    if prof_path.is_file():
        profiling = json.loads(prof_path.read_text())
    runtime = {}
    rt_path = run_dir / "diagnostics" / "runtime.json"
    if rt_path.is_file():
        runtime = json.loads(rt_path.read_text())
    trace_end = int(profiling.get("trace_end_step") or 0) if profiling.get("enabled") else 0
    start = max(warmup_steps + 1, trace_end + 1)
    excluded = {int(e["step"]) for e in events if e.get("type") in _EXCLUDED_EVENT_TYPES and "step" in e}
    steady = [r for r in rows if int(r.get("step", 0)) >= start and int(r.get("step", 0)) not in excluded]
    medians = {}
    for key in _SCALARS:
        vals = [float(r[key]) for r in steady if r.get(key) is not None]
        medians[key] = statistics.median(vals) if vals else None
    traces = [summarize_trace(p) for p in sorted((run_dir / "profiles").glob("*.json"))] if (run_dir / "profiles").is_dir() else []
    return {
        "run_id": run_dir.name, "path": run_dir.as_posix(), "rows": len(rows),
        "steady": {"start_step": start, "end_step": int(steady[-1]["step"]) if steady else None, "rows": len(steady),
                   "excluded_steps": sorted(excluded), "medians": medians},
        "device_kind": (runtime.get("runtime") or {}).get("device_kind"),
        "device_count": (runtime.get("mesh") or {}).get("device_count"),
        "optimizer": (runtime.get("optimizer") or {}).get("name"),
        "parallelism": runtime.get("parallelism"), "traces": traces,
    }


def _paired_comparisons(runs: list[dict[str, Any]]) -> list[dict[str, Any]]:
    by_id = {r["run_id"]: r for r in runs}
    out = []
    for rid, run in sorted(by_id.items()):
        for cand_tag, base_tag, kind in (("muon", "adamw", "optimizer"), ("distributed", "duplicated", "muon_tp_mode"),
                                         ("fused", "nccl", "transport")):
            if cand_tag not in rid:
                continue
            base_id = rid.replace(cand_tag, base_tag)
            base = by_id.get(base_id)
            if base is None or base_id == rid:
                continue
            def delta(key):
                a, b = run["steady"]["medians"].get(key), base["steady"]["medians"].get(key)
                return None if not a or not b else (a - b) / b
            out.append({"kind": kind, "candidate": rid, "baseline": base_id,
                        "train_step_delta": delta("train_step_sec"), "step_delta": delta("step_sec"),
                        "tokens_per_sec_delta": delta("train_tokens_per_sec")})
    return out


def analyze_profile_root(root: str | Path, *, warmup_steps: int = 2) -> dict[str, Any]:
    root = Path(root)
    if warmup_steps < 0:
        raise ContractError(f"profile warmup steps must be non-negative, got {warmup_steps}")
    if not root.is_dir():
        raise ContractError(f"profile analysis root is not a directory: {root}")
    run_dirs = discover_profile_runs(root)
    if not run_dirs:
        raise ContractError(f"profile analysis found no metrics/train.jsonl below {root}")
    runs = sorted((_analyze_run(d, warmup_steps) for d in run_dirs), key=lambda r: r["run_id"])
    hardware: dict[str, list[str]] = defaultdict(list)
    for r in runs:
        hardware[f"{r['device_count']}x{r['device_kind']}"].append(r["run_id"])
    return {
        "schema_version": PROFILE_ANALYSIS_SCHEMA_VERSION, "source": root.name,
        "measurement_policy": {"warmup_steps": warmup_steps, "steady_start": "max(warmup_steps + 1, trace_end_step + 1)",
                               "excluded_event_types": sorted(_EXCLUDED_EVENT_TYPES), "scalar_reducer": "median",
                               "trace_device": "cuda kernels of torch.profiler traces"},
        "run_count": len(runs), "hardware": dict(sorted(hardware.items())), "runs": runs,
        "comparisons": _paired_comparisons(runs),
    }
