"""Baseline-relative run score and the run registry ledger (the legacy scoring tools of the reference).

Formulas restated from the reference's scoring document (docs/scoring.md:1-260; implementation in
src/research/utils/run_score.py and run_registry.py): ``RunScore = 25 * (0.40 Quality + 0.25 TrainingEfficiency +
0.20 InferenceEfficiency + 0.15 Health)``; the first three are ratios to a baseline run with every component
clamped to [0.5, 1.5], Health is an absolute reliability score in [0, 1].  A run that lacks a required input is
returned unscored rather than filled with neutral values.  ``bits_per_byte`` is the tokenizer-independent quality
metric: nats / (ln 2 * bytes).
"""

from __future__ import annotations

import json
import math
from pathlib import Path
from typing import Any, Mapping

BASE_SCORE = 25.0
WEIGHTS = {"quality": 0.40, "training_efficiency": 0.25, "inference_efficiency": 0.20, "health": 0.15}
QUALITY_WEIGHTS = {"core": 0.50, "native_val_bpb": 0.23, "domain_mean_bpb": 0.17, "domain_worst_bpb": 0.05,
                   "epiplexity": 0.05}
TRAINING_WEIGHTS = {"mfu": 0.50, "quality_per_compute": 0.30, "tokens_per_peak_flop": 0.20}
INFERENCE_WEIGHTS = {"decode": 0.55, "prefill": 0.30, "ttft": 0.15}


def bits_per_byte(nats_sum: float, byte_count: float) -> float:
    """Summed negative log-likelihood in nats over the text's raw bytes -> bits per byte."""

    if byte_count <= 0:
        raise ValueError("byte_count must be positive")
    return float(nats_sum) / (math.log(2.0) * float(byte_count))


def _clamp(x: float, lo: float = 0.5, hi: float = 1.5) -> float:
    return max(lo, min(hi, x))


def _need(row: Mapping[str, Any], keys) -> list[str]:
    return [k for k in keys if row.get(k) is None]


def quality(run: Mapping[str, Any], base: Mapping[str, Any]) -> float:
    parts = {
        "core": (run["core"] + 1.0) / (base["core"] + 1.0),                       # CORE can be negative
        "native_val_bpb": base["final_val_bpb"] / run["final_val_bpb"],           # lower is better
        "domain_mean_bpb": base["domain_mean_bpb"] / run["domain_mean_bpb"],
        "domain_worst_bpb": base["domain_worst_bpb"] / run["domain_worst_bpb"],
        "epiplexity": run["train_epiplexity_bpb_auc_per_byte"] / base["train_epiplexity_bpb_auc_per_byte"],
    }
    return sum(QUALITY_WEIGHTS[k] * _clamp(v) for k, v in parts.items())


def training_efficiency(run: Mapping[str, Any], base: Mapping[str, Any], run_quality: float,
                        base_quality: float = 1.0) -> float:
    run_compute = run["flops_per_token"] * run["tokens_seen"]
    base_compute = base["flops_per_token"] * base["tokens_seen"]
    parts = {
        "mfu": run["steady_train_mfu"] / base["steady_train_mfu"],
        "quality_per_compute": (run_quality / run_compute) / (base_quality / base_compute),
        "tokens_per_peak_flop": (run["steady_train_tokens_per_sec"] / run["peak_flops_total"])
        / (base["steady_train_tokens_per_sec"] / base["peak_flops_total"]),
    }
    return sum(TRAINING_WEIGHTS[k] * _clamp(v) for k, v in parts.items())


def inference_efficiency(run: Mapping[str, Any], base: Mapping[str, Any]) -> float:
    parts = {
        "decode": run["decode_tokens_per_sec"] / base["decode_tokens_per_sec"],
        "prefill": run["prefill_tokens_per_sec"] / base["prefill_tokens_per_sec"],
        "ttft": base["ttft_sec"] / run["ttft_sec"],                               # lower is better
    }
    return sum(INFERENCE_WEIGHTS[k] * _clamp(v) for k, v in parts.items())


def health(run: Mapping[str, Any]) -> float:
    h = 1.0
    status = run.get("status", "complete")
    if status == "failed" or run.get("nan_count", 0) > 0:
        return 0.0
    if status == "incomplete":
        h = min(h, 0.25)
    if status == "unstable":
        h = min(h, 0.75)
    h -= min(0.25, 0.05 * run.get("loss_spike_count", 0))
    h -= min(0.15, 0.03 * run.get("grad_norm_spike_count", 0))
    best, final = run.get("best_val_bpb"), run.get("final_val_bpb")
    if best and final:
        h -= min(0.20, max(0.0, final - best) / best)
    return max(0.0, min(1.0, h))


REQUIRED = ("core", "final_val_bpb", "domain_mean_bpb", "domain_worst_bpb", "train_epiplexity_bpb_auc_per_byte",
            "steady_train_mfu", "flops_per_token", "peak_flops_total", "tokens_seen", "steady_train_tokens_per_sec",
            "decode_tokens_per_sec", "prefill_tokens_per_sec", "ttft_sec")


def run_score(run: Mapping[str, Any], base: Mapping[str, Any]) -> dict[str, Any]:
    """Score ``run`` against ``base``.  Returns the components; ``score`` is None (with the reason) when unscored."""

    if run.get("status") == "failed":
        return {"score": None, "unscored_reason": "failed run", "health": 0.0}
    missing = _need(run, REQUIRED) + [f"baseline.{k}" for k in _need(base, REQUIRED)]
    if missing:
        return {"score": None, "unscored_reason": "missing " + ", ".join(missing), "health": health(run)}
    q = quality(run, base)
    t = training_efficiency(run, base, q)
    inf = inference_efficiency(run, base)
    h = health(run)
    total = BASE_SCORE * (WEIGHTS["quality"] * q + WEIGHTS["training_efficiency"] * t
                          + WEIGHTS["inference_efficiency"] * inf + WEIGHTS["health"] * h)
    return {"score": total, "quality": q, "training_efficiency": t, "inference_efficiency": inf, "health": h}


# --------------------------------------------------------------------------------------------------
# registry: one JSON line per run, upserted by run name
# --------------------------------------------------------------------------------------------------
def load_registry(path: str | Path) -> list[dict[str, Any]]:
    path = Path(path)
    if not path.exists():
        return []
    return [json.loads(line) for line in path.read_text(encoding="utf-8").splitlines() if line.strip()]


def register_run(summary: Mapping[str, Any], path: str | Path) -> Path:
    """Insert or replace the row whose ``run_name`` matches; rows keep their order of first registration."""

    path = Path(path)
    if "run_name" not in summary:
        raise ValueError("a run summary needs a run_name")
    rows = load_registry(path)
    for i, row in enumerate(rows):
        if row.get("run_name") == summary["run_name"]:
            rows[i] = dict(summary)
            break
    else:
        rows.append(dict(summary))
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(path.suffix + ".tmp")
    tmp.write_text("".join(json.dumps(r, sort_keys=True) + "\n" for r in rows), encoding="utf-8")
    tmp.replace(path)
    return path


def format_registry(rows: list[Mapping[str, Any]]) -> str:
    if not rows:
        return "no registered runs"
    cols = (("run_name", 28), ("status", 10), ("score", 8), ("tokens_seen", 12), ("best_val_loss", 10),
            ("latest_decode_tokens_per_sec", 9), ("avg_mfu", 8))

    def fmt(v):
        if v is None:
            return "-"
        if isinstance(v, float):
            return f"{v:.0f}" if abs(v) >= 1000 else f"{v:.4f}"
        return str(v)

    head = " ".join(f"{name[:w]:<{w}}" for name, w in cols)
    lines = [head, "-" * len(head)]
    for row in rows:
        lines.append(" ".join(f"{fmt(row.get(name))[:w]:<{w}}" for name, w in cols))
    return "\n".join(lines)
