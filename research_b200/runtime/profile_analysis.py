"""Offline analysis of profiling runs: steady-window medians, paired deltas, GPU kernel categories.

Same measurement policy as the reference analyzer (src/jaxtitan/runtime/profile_analysis.py:68-97, 141-324): every
directory below ``root`` that holds ``metrics/train.jsonl`` is a run; the steady window starts after
``max(warmup_steps + 1, trace_end_step + 1)`` and skips steps that ran an eval or a checkpoint; scalars are reduced
with the median; runs are paired by name (``..._muon`` vs ``..._adamw``, same prefix) for percentage deltas.  Where
the reference categorises XLA/HLO ops and Perfetto GPU:0 events, this one categorises CUDA kernels of a Chrome /
Perfetto trace written by ``torch.profiler`` (GEMM, attention, NCCL, element-wise, optimizer, other; plain or gzipped
JSON) and counts collectives by NCCL kernel name.  Runs are also paired by structure - same model signature and
layout with ``muon`` against ``adamw``, and a layout against the one it extends (``tp`` over ``ddp``, ``fsdp+tp`` and
``zero2+tp`` over ``tp``, ``tp+ep`` over ``ep``).  The rows inside the traced window are reduced separately and their
relative distance from the steady window is the cost of tracing ("tax").  A run whose final summary says it did not
complete, or that ended with non-finite optimizer groups, is refused.  There is no compiler IR to summarise here: the
reference's HLO section has no counterpart and ``hlo`` is always null.
"""

from __future__ import annotations

import gzip
import json
import math
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


def _load_trace(path: Path) -> Any:
    try:
        if path.suffix == ".gz":
            with gzip.open(path, "rt", encoding="utf-8") as handle:
                return json.load(handle)
        return json.loads(path.read_text())
    except (OSError, json.JSONDecodeError, EOFError) as exc:
        raise ContractError(f"failed to read trace {path}: {exc}") from exc


def summarize_trace(path: Path) -> dict[str, Any]:
    """Per-category GPU kernel time and NCCL collective counts from a Chrome-trace JSON (``.json`` or ``.json.gz``)."""

    raw = _load_trace(path)
    events = raw.get("traceEvents", raw) if isinstance(raw, Mapping) else raw
    if not isinstance(events, list):
        raise ContractError(f"trace must contain a traceEvents array: {path}")
    time_us: Counter[str] = Counter()
    counts: Counter[str] = Counter()
    longest: dict[str, float] = {}
    collectives: Counter[str] = Counter()
    top: Counter[str] = Counter()
    top_counts: Counter[str] = Counter()
    for ev in events:
        if not isinstance(ev, Mapping) or ev.get("ph") != "X":
            continue
        cat = str(ev.get("cat", "")).lower()
        if "kernel" not in cat and cat != "gpu_memcpy":
            continue
        name = str(ev.get("name", ""))
        dur = ev.get("dur", 0.0)
        if not isinstance(dur, (int, float)) or dur < 0:
            continue
        dur = float(dur)
        k = "memcpy" if cat == "gpu_memcpy" else categorize_kernel(name)
        time_us[k] += dur
        counts[k] += 1
        longest[k] = max(longest.get(k, 0.0), dur)
        top[name[:96]] += dur
        top_counts[name[:96]] += 1
        if k == "nccl":
            for kind in ("AllGather", "ReduceScatter", "AllReduce", "SendRecv", "Broadcast"):
                if kind.lower() in name.lower():
                    collectives[kind] += 1
    total = sum(time_us.values())
    return {"trace": path.name, "gpu_time_us": dict(sorted(time_us.items())), "kernel_counts": dict(sorted(counts.items())),
            "gpu_time_share": {k: (v / total if total else 0.0) for k, v in sorted(time_us.items())},
            "max_kernel_us": dict(sorted(longest.items())),
            "collective_counts": dict(sorted(collectives.items())),
            "top_kernels": [{"name": n, "time_us": t, "count": top_counts[n]} for n, t in top.most_common(20)],
            "event_count": int(sum(counts.values())), "total_gpu_time_us": total}


def model_signature(model: Any) -> str:
    """A model's structural fields as canonical JSON: two runs with the same signature train the same network
    (``variant`` and ``remat`` do not change it)."""

    if not isinstance(model, Mapping):
        return "unknown"
    return json.dumps({k: v for k, v in model.items() if k not in ("variant", "remat")}, sort_keys=True,
                      separators=(",", ":"))


def layout_name(resolved: Mapping[str, Any]) -> str:
    par = resolved.get("parallelism") or {}
    axes = [str(par["mode"])] if par.get("mode") in ("fsdp", "zero2") else []
    axes += [name for name, key in (("tp", "tensor_parallel"), ("cp", "context_parallel"), ("ep", "expert_parallel"))
             if par.get(key)]
    return "+".join(axes) if axes else "ddp"


def _medians(rows) -> dict[str, float | None]:
    rows = list(rows)
    out = {}
    for key in _SCALARS:
        vals = [float(r[key]) for r in rows if isinstance(r.get(key), (int, float)) and not isinstance(r.get(key), bool)
                and math.isfinite(float(r[key]))]
        out[key] = statistics.median(vals) if vals else None
    return out


def relative_delta(candidate: Any, baseline: Any) -> float | None:
    if not isinstance(candidate, (int, float)) or not isinstance(baseline, (int, float)) or baseline == 0:
        return None
    return float(candidate) / float(baseline) - 1.0


def _optional_json(path: Path) -> dict[str, Any]:
    if not path.is_file():
        return {}
    try:
        raw = json.loads(path.read_text())
    except (OSError, json.JSONDecodeError) as exc:
        raise ContractError(f"failed to read {path}: {exc}") from exc
    if not isinstance(raw, dict):
        raise ContractError(f"{path} must be a JSON object")
    return raw


def _analyze_run(run_dir: Path, warmup_steps: int) -> dict[str, Any]:
    rows = _read_jsonl(run_dir / "metrics" / "train.jsonl")
    events = _read_jsonl(run_dir / "events.jsonl")
    runtime = _optional_json(run_dir / "diagnostics" / "runtime.json")
    resolved = _optional_json(run_dir / "config" / "resolved.json")
    final = _optional_json(run_dir / "summaries" / "final.json")
    profiling = _optional_json(run_dir / "diagnostics" / "profiling.json") or dict(runtime.get("profiling") or {})
    run_id = final.get("run_id") if isinstance(final.get("run_id"), str) and final.get("run_id") else run_dir.name
    if final and final.get("status") not in (None, "completed"):
        raise ContractError(f"profile run {run_id} is not completed: status={final.get('status')!r}")
    if int(final.get("final_optimizer_nonfinite_group_count") or 0) != 0:
        raise ContractError(f"profile run {run_id} contains nonfinite optimizer groups")

    def step_of(value):
        return int(value) if isinstance(value, int) and not isinstance(value, bool) else None

    traced = bool(profiling.get("enabled"))
    trace_start = step_of(profiling.get("trace_start_step")) if traced else None
    trace_end = step_of(profiling.get("trace_end_step")) if traced else None
    start = max(warmup_steps + 1, (trace_end or 0) + 1)
    excluded = {int(e["step"]) for e in events if e.get("type") in _EXCLUDED_EVENT_TYPES and step_of(e.get("step")) is not None}
    steady = [r for r in rows if int(r.get("step", 0)) >= start and int(r.get("step", 0)) not in excluded]
    medians = _medians(steady)
    window = []
    if trace_start is not None and trace_end is not None:
        window = [r for r in rows if trace_start <= int(r.get("step", -1)) <= trace_end]
    window_medians = _medians(window) if window else None
    profiles = run_dir / "profiles"
    trace_files = sorted(list(profiles.glob("*.json")) + list(profiles.glob("*.json.gz"))) if profiles.is_dir() else []
    traces = [summarize_trace(p) for p in trace_files]
    model = resolved.get("model") or {}
    return {
        "run_id": run_id, "path": run_dir.as_posix(), "rows": len(rows),
        "status": final.get("status"),
        "model": {"name": (runtime.get("model") or {}).get("name", model.get("name")),
                  "parameters": (runtime.get("model") or {}).get("parameters"),
                  "signature": model_signature(model) if model else "unknown"},
        "layout": layout_name(resolved) if resolved else layout_name({"parallelism": runtime.get("parallelism")}),
        "steady": {"start_step": start, "end_step": int(steady[-1]["step"]) if steady else None, "rows": len(steady),
                   "row_count": len(steady), "excluded_steps": sorted(excluded), "medians": medians},
        "trace_window": {"start_step": trace_start, "end_step": trace_end, "row_count": len(window),
                         "medians": window_medians,
                         "tax": None if window_medians is None else {k: relative_delta(window_medians.get(k), medians.get(k))
                                                                     for k in _SCALARS}},
        "device_kind": (runtime.get("runtime") or {}).get("device_kind"),
        "device_count": (runtime.get("mesh") or {}).get("device_count"),
        "hardware": {"backend": (runtime.get("runtime") or {}).get("backend"),
                     "device_kind": (runtime.get("runtime") or {}).get("device_kind"),
                     "device_count": (runtime.get("mesh") or {}).get("device_count"),
                     "mesh": (runtime.get("parallelism") or {}).get("mesh")},
        "optimizer": (runtime.get("optimizer") or {}).get("name") or (resolved.get("optimizer") or {}).get("name"),
        "parallelism": runtime.get("parallelism"), "traces": traces, "trace": traces[0] if traces else None,
        "hlo": None,
    }


_LAYOUT_BASELINES = {"tp": "ddp", "fsdp+tp": "tp", "zero2+tp": "tp", "tp+ep": "ep", "fsdp+tp+ep": "fsdp+ep",
                     "cp": "ddp", "fsdp+cp": "fsdp"}


def _comparison(kind: str, base: Mapping[str, Any], cand: Mapping[str, Any]) -> dict[str, Any]:
    b, c = base["steady"]["medians"], cand["steady"]["medians"]
    return {"kind": kind, "candidate": cand["run_id"], "baseline": base["run_id"],
            "train_step_delta": relative_delta(c.get("train_step_sec"), b.get("train_step_sec")),
            "step_delta": relative_delta(c.get("step_sec"), b.get("step_sec")),
            "tokens_per_sec_delta": relative_delta(c.get("train_tokens_per_sec"), b.get("train_tokens_per_sec"))}


def _paired_comparisons(runs: list[dict[str, Any]]) -> list[dict[str, Any]]:
    by_id = {r["run_id"]: r for r in runs}
    seen: set[tuple[str, str, str]] = set()
    out = []

    def add(kind, base, cand):
        key = (kind, cand["run_id"], base["run_id"])
        if base["run_id"] != cand["run_id"] and key not in seen:
            seen.add(key)
            out.append(_comparison(kind, base, cand))

    # by name: the same run id with one tag exchanged
    for rid, run in sorted(by_id.items()):
        for cand_tag, base_tag, kind in (("muon", "adamw", "optimizer"), ("distributed", "duplicated", "muon_tp_mode"),
                                         ("fused", "nccl", "transport")):
            if cand_tag in rid and rid.replace(cand_tag, base_tag) in by_id:
                add(kind, by_id[rid.replace(cand_tag, base_tag)], run)
    # by structure: the same network, and either the optimizer or the layout differs
    by_key = {(r["model"]["signature"], r["layout"], r["optimizer"]): r for r in runs
              if r["model"]["signature"] != "unknown"}
    for (signature, layout, optimizer), run in sorted(by_key.items(), key=lambda kv: kv[1]["run_id"]):
        if optimizer == "muon" and (signature, layout, "adamw") in by_key:
            add("optimizer", by_key[(signature, layout, "adamw")], run)
        base_layout = _LAYOUT_BASELINES.get(layout)
        if base_layout is not None and (signature, base_layout, optimizer) in by_key:
            add("layout", by_key[(signature, base_layout, optimizer)], run)
    return sorted(out, key=lambda item: (item["kind"], item["candidate"], item["baseline"]))


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


def profile_analysis_to_json(payload: Mapping[str, Any]) -> str:
    return json.dumps(payload, sort_keys=True, separators=(",", ":"), allow_nan=False)


def format_profile_analysis(payload: Mapping[str, Any]) -> str:
    """The table a person reads: one line per run with its steady medians, then the paired deltas
    (reference: profile_analysis.py:114-138)."""

    def ms(v):
        return "n/a" if v is None else f"{1000.0 * float(v):.2f}"

    def num(v):
        return "n/a" if v is None else f"{float(v):,.0f}"

    def pct(v):
        return "n/a" if v is None else f"{100.0 * float(v):+.1f}%"

    lines = [f"profile analysis: runs={payload['run_count']} source={payload['source']}", "",
             f"{'run':<47} {'steps':>7} {'train ms':>11} {'step ms':>10} {'tok/s':>10}"]
    for run in payload["runs"]:
        m = run["steady"]["medians"]
        span = f"{run['steady']['start_step']}-{run['steady']['end_step']}"
        lines.append(f"{run['run_id']:<47} {span:>7} {ms(m.get('train_step_sec')):>11} {ms(m.get('step_sec')):>10} "
                     f"{num(m.get('train_tokens_per_sec')):>10}")
        tax = (run.get("trace_window") or {}).get("tax")
        if tax and tax.get("train_step_sec") is not None:
            lines.append(f"{'':<47} traced steps {run['trace_window']['start_step']}-{run['trace_window']['end_step']}: "
                         f"train {pct(tax['train_step_sec'])}")
        trace = run.get("trace")
        if trace and trace["total_gpu_time_us"] > 0:
            shares = " ".join(f"{k}={100.0 * v:.0f}%" for k, v in sorted(trace["gpu_time_share"].items(),
                                                                          key=lambda kv: -kv[1]) if v >= 0.005)
            lines.append(f"{'':<47} gpu time: {shares}")
    if payload["comparisons"]:
        lines += ["", "paired deltas:"]
        for item in payload["comparisons"]:
            lines.append(f"  {item['kind']} {item['candidate']} vs {item['baseline']}: "
                         f"train={pct(item['train_step_delta'])} step={pct(item['step_delta'])} "
                         f"tok/s={pct(item['tokens_per_sec_delta'])}")
    return "\n".join(lines)
