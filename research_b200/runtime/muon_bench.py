"""Distributed-Muon benchmark and selector: candidate executions per leaf class on the current tensor-parallel
group, their correctness envelope against the duplicated path, and the timing that picks between them.

What is measured follows the reference selector (src/jaxtitan/runtime/muon_bench.py:69-187 leaf classes, production
buckets and the one-factor calibration lattice; 520-533 eligible executions; 536-643 candidate check; 655-700 timing;
829-852 replica difference): for every case each eligible execution runs five Muon steps on perturbed gradients and
must stay finite, keep the momentum bit-identical to the duplicated path (it does not depend on the orthogonaliser),
give the same bits when run twice, leave all replicas equal, and keep the update and the parameter within
``6e-4`` / ``1.25e-3`` per ``1e-3`` of learning rate of the duplicated path.  Candidates are then timed round-robin
and the fastest one that passed is the selection.  The process group the command runs in plays the tensor-parallel
group (one rank: every execution degenerates to the local iteration, which still exercises the code).

``jaxtitan profile bench muon`` prints the report and, with ``--artifact-dir``, writes ``manifest.json`` with one entry
per case (``runtime/validation_matrix.py: analyze_muon_bench`` gates it).
"""

from __future__ import annotations

import json
import math
import time
from dataclasses import dataclass
from pathlib import Path
from statistics import median
from typing import Any

import torch
import torch.distributed as dist

from research_b200.optim import distributed_ns as dns
from research_b200.optim import orthogonalize as orth

BENCH_LR = 0.02
CALIBRATION_LR = 1e-3
UPDATE_ENVELOPE = 6e-4             # at the calibration learning rate
PARAM_ENVELOPE = 1.25e-3
UPDATE_ATOL = UPDATE_ENVELOPE * BENCH_LR / CALIBRATION_LR
PARAM_ATOL = PARAM_ENVELOPE * BENCH_LR / CALIBRATION_LR
WEIGHT_DECAY = 0.01
STABILITY_LIMIT = 0.05             # median absolute deviation over the median of a candidate's timings
SELECTION_MIN_SPEEDUP = 1.05       # what a distributed execution must gain over the duplicated one to be selected
SELECTION_TIE_FRACTION = 0.03


def benchmark_contract() -> dict[str, Any]:
    """The numerical and measurement policy of the selector, as data (reference: muon_bench.py:854-874)."""

    return {"correctness_steps": 5, "benchmark_learning_rate": BENCH_LR,
            "reference_calibration_learning_rate": CALIBRATION_LR, "reference_update_atol": UPDATE_ENVELOPE,
            "reference_parameter_atol": PARAM_ENVELOPE, "tolerance_scaling": "linear_with_learning_rate",
            "update_atol": UPDATE_ATOL, "parameter_atol": PARAM_ATOL, "candidate_order": "rotating",
            "timing_reducer": "median", "tail_percentile": 95,
            "stability_metric": "median_abs_deviation_over_median", "stability_limit": STABILITY_LIMIT,
            "selection_min_speedup": SELECTION_MIN_SPEEDUP, "selection_tie_fraction": SELECTION_TIE_FRACTION,
            "timing_is_production_acceptance_gate": False}


@dataclass(frozen=True)
class Leaf:
    role: str
    shape: tuple[int, int]          # logical [in, out]
    tp_partition_dim: int           # logical axis the group splits


@dataclass(frozen=True)
class BucketCase:
    name: str
    leaf: Leaf
    leaf_count: int
    kind: str


CURRENT_LEAVES = (
    Leaf("attention_kv", (1024, 256), 1), Leaf("attention_q_gate", (1024, 1024), 1),
    Leaf("attention_o", (1024, 1024), 0), Leaf("shared_mlp_gate_up", (1024, 2048), 1),
    Leaf("shared_mlp_down", (2048, 1024), 0), Leaf("dense_mlp_gate_up", (1024, 4096), 1),
    Leaf("dense_mlp_down", (4096, 1024), 0),
)
PRODUCTION_BUCKETS = tuple(BucketCase(f"{leaf.role}_bucket{n}", leaf, n, "production_bucket")
                           for leaf, n in zip(CURRENT_LEAVES, (24, 12, 12, 20, 10, 24, 12)))


def calibration_bucket_cases() -> tuple[BucketCase, ...]:
    """One-factor lattice around (width 1024, aspect 2, 12 leaves), both split orientations."""

    points = ((256, 2, 12), (1024, 2, 12), (2048, 2, 12), (1024, 1, 12), (1024, 4, 12), (1024, 2, 1), (1024, 2, 24))
    cases = []
    for short, aspect, count in points:
        for canonical in (0, 1):
            orientation = "row" if canonical == 0 else "column"
            cases.append(BucketCase(f"calibration_w{short}_r{aspect}_{orientation}_bucket{count}",
                                    Leaf("calibration", (short, short * aspect), canonical), count,
                                    "calibration_bucket"))
    return tuple(cases)


def eligible_executions(shape: tuple[int, int], tp_partition_dim: int, tp_size: int) -> tuple[str, ...]:
    transpose = shape[0] > shape[1]
    canonical = 1 - tp_partition_dim if transpose else tp_partition_dim
    if canonical == 1:
        return ("duplicated", "distributed_direct")
    out = ["duplicated", "distributed_large_gram"]
    if max(shape) % tp_size == 0:
        out.append("distributed_exchange")
    return tuple(out)


def collective_operand_model(shape: tuple[int, int], execution: str, tp_size: int) -> dict[str, Any]:
    """Bytes each rank contributes to the collectives of one orthogonalisation."""

    elements, short, long = math.prod(shape), min(shape), max(shape)
    if execution == "duplicated":
        return {"kind": "logical_matrix_gather", "gather_local_operand_bytes_per_rank": elements * 2 // tp_size,
                "gather_result_bytes_per_rank": elements * 2}
    g = long if execution == "distributed_large_gram" else short
    out = {"kind": "norm_folded_into_five_gram_reductions", "gram_dimension": g,
           "gram_operand_bytes_per_rank_per_step": g * g * 4, "gram_steps": orth.MUON_NS_STEPS}
    if execution == "distributed_exchange":
        out["exchange_operand_bytes_per_rank_each_direction"] = elements * 2 // tp_size
        out["exchange_directions"] = 2
    return out


class _Candidate:
    """One execution of one case: local shards of ``count`` equal leaves and the Muon step over them."""

    def __init__(self, leaf: Leaf, count: int, execution: str, group, device: torch.device, reducer):
        self.leaf, self.count, self.execution, self.group, self.reducer = leaf, count, execution, group, reducer
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        rows, cols = leaf.shape
        self.storage_axis = 1 - leaf.tp_partition_dim            # storage is [out, in] = logical transposed
        transpose = rows > cols
        canonical = 1 - leaf.tp_partition_dim if transpose else leaf.tp_partition_dim
        self.plans = [dns.MuonLeafPlan(f"{leaf.role}.{i}", leaf.shape, leaf.tp_partition_dim, transpose, canonical,
                                       "distributed", execution, None, 0, True) for i in range(count)]
        g = torch.Generator(device="cpu").manual_seed(1234)
        shard = lambda t: t.chunk(self.world, dim=self.storage_axis)[self.rank].contiguous().to(device)  # noqa: E731
        self.params = [shard(torch.randn(cols, rows, generator=g) * 0.02) for _ in range(count)]
        self.grads = [shard(torch.randn(cols, rows, generator=g) * 0.01) for _ in range(count)]
        self.momentum = [torch.zeros_like(p) for p in self.params]
        self.timings: list[float] = []

    def _orthogonalise(self, inputs: list[torch.Tensor]) -> list[torch.Tensor]:
        if self.execution == "duplicated":
            outs = []
            for u in inputs:
                parts = [torch.empty_like(u) for _ in range(self.world)]
                dist.all_gather(parts, u.contiguous(), group=self.group)
                full = orth.zeropower_via_newton_schulz(torch.cat(parts, dim=self.storage_axis))
                outs.append(full.chunk(self.world, dim=self.storage_axis)[self.rank].contiguous())
            return outs
        return dns.bucketed_distributed_zeropower(inputs, self.plans, [self.storage_axis] * self.count, self.group,
                                                  self.reducer)

    def step(self, params, grads, momentum):
        """One Muon step: returns ``(next params, updates, next momentum)`` (lists of local shards)."""

        nxt_m, inputs = [], []
        for g, m in zip(grads, momentum):
            m2 = orth.MUON_MOMENTUM * m + (1.0 - orth.MUON_MOMENTUM) * g
            nxt_m.append(m2)
            inputs.append(((1.0 - orth.MUON_MOMENTUM) * g + orth.MUON_MOMENTUM * m2).to(torch.bfloat16))
        outs = self._orthogonalise(inputs)
        scale = BENCH_LR * orth.rms_match_scale(self.leaf.shape)
        updates = [-scale * o.float() - BENCH_LR * WEIGHT_DECAY * p for o, p in zip(outs, params)]
        return [p + u for p, u in zip(params, updates)], updates, nxt_m

    def replica_difference(self, tensors: list[torch.Tensor]) -> float:
        """Largest difference between what the ranks reconstruct as the whole matrices (0 when they agree)."""

        worst = 0.0
        for t in tensors:
            parts = [torch.empty_like(t) for _ in range(self.world)]
            dist.all_gather(parts, t.contiguous(), group=self.group)
            full = torch.cat(parts, dim=self.storage_axis).float()
            hi, lo = full.clone(), full.clone()
            dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=self.group)
            dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=self.group)
            worst = max(worst, float((hi - lo).abs().max()))
        return worst


def _sync(device: torch.device) -> None:
    if device.type == "cuda":
        torch.cuda.synchronize(device)


def _max_abs(a: list[torch.Tensor], b: list[torch.Tensor], group) -> float:
    worst = torch.zeros(1, device=a[0].device)
    for x, y in zip(a, b):
        worst = torch.maximum(worst, (x.float() - y.float()).abs().max().reshape(1))
    dist.all_reduce(worst, op=dist.ReduceOp.MAX, group=group)
    return float(worst.item())


def _all_ranks(flag: bool, group, device) -> bool:
    t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
    return bool(int(t.item()))


def check_candidates(candidates: list[_Candidate]) -> dict[str, dict[str, Any]]:
    """Five steps on perturbed gradients; every execution against ``duplicated``."""

    group, device = candidates[0].group, candidates[0].params[0].device
    state = {c.execution: (c.params, c.momentum) for c in candidates}
    maxima = {c.execution: {"max_update_abs_error": 0.0, "max_parameter_abs_error": 0.0, "momentum_exact": True,
                            "finite": True, "replica_max_abs_error": 0.0} for c in candidates}
    for k in range(5):
        outputs = {}
        for c in candidates:
            params, momentum = state[c.execution]
            grads = [g + torch.sin(g * (k + 1)) * (0.03 * k) for g in c.grads]
            nxt_p, upd, nxt_m = c.step(params, grads, momentum)
            outputs[c.execution] = (nxt_p, upd, nxt_m)
            state[c.execution] = (nxt_p, nxt_m)
            row = maxima[c.execution]
            row["finite"] = row["finite"] and _all_ranks(all(torch.isfinite(t).all().item() for t in nxt_p + upd),
                                                         group, device)
            row["replica_max_abs_error"] = max(row["replica_max_abs_error"], c.replica_difference(nxt_p))
        ref_p, ref_u, ref_m = outputs["duplicated"]
        for c in candidates:
            p, u, m = outputs[c.execution]
            row = maxima[c.execution]
            row["max_update_abs_error"] = max(row["max_update_abs_error"], _max_abs(u, ref_u, group))
            row["max_parameter_abs_error"] = max(row["max_parameter_abs_error"], _max_abs(p, ref_p, group))
            row["momentum_exact"] = row["momentum_exact"] and _all_ranks(
                all(torch.equal(x, y) for x, y in zip(m, ref_m)), group, device)
    for c in candidates:
        row = maxima[c.execution]
        a, b = c.step(c.params, c.grads, c.momentum), c.step(c.params, c.grads, c.momentum)
        row["deterministic"] = _all_ranks(all(torch.equal(x, y) for xs, ys in zip(a, b) for x, y in zip(xs, ys)),
                                          group, device)
        row["correctness_gate"] = bool(
            row["finite"] and row["momentum_exact"] and row["deterministic"] and row["replica_max_abs_error"] == 0.0
            and row["max_update_abs_error"] <= UPDATE_ATOL and row["max_parameter_abs_error"] <= PARAM_ATOL)
        row["max_update_abs_error_per_lr"] = row["max_update_abs_error"] / BENCH_LR
        row["max_parameter_abs_error_per_lr"] = row["max_parameter_abs_error"] / BENCH_LR
    return maxima


def time_candidates(candidates: list[_Candidate], *, warmup: int, iters: int) -> None:
    """Round-robin timing (each iteration visits every candidate, starting one further each time)."""

    device = candidates[0].params[0].device
    current = {c.execution: (c.params, c.momentum) for c in candidates}
    for c in candidates:
        p, m = current[c.execution]
        for _ in range(warmup):
            p, _, m = c.step(p, c.grads, m)
        current[c.execution] = (p, m)
    _sync(device)
    for it in range(iters):
        for off in range(len(candidates)):
            c = candidates[(it + off) % len(candidates)]
            p, m = current[c.execution]
            dist.barrier(group=c.group)
            _sync(device)
            t0 = time.perf_counter()
            p, _, m = c.step(p, c.grads, m)
            _sync(device)
            ms = torch.tensor([(time.perf_counter() - t0) * 1e3], dtype=torch.float64, device=device)
            dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=c.group)          # the slowest rank counts
            c.timings.append(float(ms.item()))
            current[c.execution] = (p, m)


def timing_summary(values: list[float]) -> dict[str, float]:
    ordered = sorted(values)
    centre = float(median(ordered))
    pos = 0.95 * (len(ordered) - 1)
    lo, hi = int(pos), min(int(pos) + 1, len(ordered) - 1)
    return {"median": centre, "p50": centre, "p95": float(ordered[lo] * (1 - (pos - lo)) + ordered[hi] * (pos - lo)),
            "min": float(ordered[0]), "max": float(ordered[-1]),
            "median_abs_deviation": float(median(sorted(abs(v - centre) for v in ordered)))}


def benchmark_case(leaf: Leaf, count: int, name: str, kind: str, group, device, reducer, *, warmup: int,
                   iters: int) -> dict[str, Any]:
    world = dist.get_world_size(group)
    rows, cols = leaf.shape
    if leaf.shape[leaf.tp_partition_dim] % world:
        return {"case": name, "kind": kind, "skipped": f"split side {leaf.shape[leaf.tp_partition_dim]} not divisible "
                                                       f"by {world} ranks"}
    executions = eligible_executions(leaf.shape, leaf.tp_partition_dim, world)
    candidates = [_Candidate(leaf, count, e, group, device, reducer) for e in executions]
    checks = check_candidates(candidates)
    time_candidates(candidates, warmup=warmup, iters=iters)
    transpose = rows > cols
    canonical = 1 - leaf.tp_partition_dim if transpose else leaf.tp_partition_dim
    rows_out = []
    for c in candidates:
        rows_out.append({"execution": c.execution, **checks[c.execution], "timing_ms": timing_summary(c.timings),
                         "collectives": collective_operand_model(leaf.shape, c.execution, world)})
    for r in rows_out:
        t = r["timing_ms"]
        r["stability"] = t["median_abs_deviation"] / t["median"] if t["median"] > 0 else None
        r["stable"] = r["stability"] is not None and r["stability"] <= STABILITY_LIMIT
    passing = [r for r in rows_out if r["correctness_gate"]]
    best = min(passing, key=lambda r: r["timing_ms"]["median"]) if passing else None
    duplicated = next(r for r in rows_out if r["execution"] == "duplicated")
    reason = None if best is None else "fastest_passing_candidate"
    if best is not None and best is not duplicated and duplicated["correctness_gate"]:
        # a distributed execution replaces the exact duplicated one only for a clear gain
        gain = duplicated["timing_ms"]["median"] / max(best["timing_ms"]["median"], 1e-9)
        if gain < SELECTION_MIN_SPEEDUP:
            best, reason = duplicated, "gain_below_selection_min_speedup"
    return {
        "case": name, "kind": kind, "role": leaf.role, "logical_shape": list(leaf.shape),
        "tp_partition_dim": leaf.tp_partition_dim, "leaf_count": count,
        "policy_features": {"short_dimension": min(leaf.shape), "long_dimension": max(leaf.shape),
                            "aspect_ratio": max(leaf.shape) / min(leaf.shape), "canonical_tp_dim": canonical,
                            "tp_size": world, "leaf_count": count,
                            "aggregate_matrix_elements": math.prod(leaf.shape) * count},
        "candidates": rows_out, "selected": None if best is None else best["execution"],
        "selection_reason": reason,
        "speedup_vs_duplicated": None if best is None else
        duplicated["timing_ms"]["median"] / max(best["timing_ms"]["median"], 1e-9),
    }


def benchmark_muon(*, warmup: int = 2, iters: int = 5, artifact_dir: str | Path | None = None,
                   cases: str = "auto") -> dict[str, Any]:
    """Run the selector on the current process group.  ``cases``: ``leaves`` (the 7 leaf classes), ``buckets``
    (+ production buckets), ``all`` (+ the calibration lattice); ``auto`` = ``all`` on CUDA, ``leaves`` on CPU with
    leaf dimensions divided by 8 so that it finishes in seconds."""

    from research_b200.ops import functional as Fn

    from research_b200.parallel.mesh import init_distributed

    init_distributed()            # under torchrun: the ranks of this launch form the tensor-parallel group
    device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    started_group = False
    if not dist.is_initialized():
        import os

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29577")
        dist.init_process_group("nccl" if device.type == "cuda" else "gloo", rank=0, world_size=1)
        started_group = True
    group = dist.group.WORLD
    world = dist.get_world_size(group)
    if cases == "auto":
        cases = "all" if device.type == "cuda" else "leaves"
    shrink = 1 if device.type == "cuda" else 8
    scale = lambda leaf: Leaf(leaf.role, (leaf.shape[0] // shrink, leaf.shape[1] // shrink), leaf.tp_partition_dim)  # noqa: E731
    reducer = None
    if device.type == "cuda" and Fn.native_enabled() and world > 1:
        from research_b200.parallel.symmetric import build_collectively

        reducer = build_collectively(group, lambda: dns.ArenaReducer(group, dns.GRAM_BUCKET_MAX_BYTES // 2 + 65536,
                                                                     device), "symmetric arena for the Muon benchmark")
    reducer = reducer or dns.TorchReducer(group)
    rows = [benchmark_case(scale(leaf), 1, leaf.role, "leaf", group, device, reducer, warmup=warmup, iters=iters)
            for leaf in CURRENT_LEAVES]
    if cases in ("buckets", "all"):
        extra = PRODUCTION_BUCKETS + (calibration_bucket_cases() if cases == "all" else ())
        for bc in extra:
            payload = bc.leaf_count * min(bc.leaf.shape) ** 2 * 2
            if payload > dns.GRAM_BUCKET_MAX_BYTES and bc.kind == "production_bucket":
                pass          # larger than one bucket on purpose: the plan would split it, the benchmark keeps it whole
            rows.append(benchmark_case(scale(bc.leaf), bc.leaf_count, bc.name, bc.kind, group, device, reducer,
                                       warmup=warmup, iters=iters))
    report = {
        "schema_version": 2, "component": "muon", "device": str(device), "tp_size": world,
        "transport": type(reducer).__name__, "benchmark_learning_rate": BENCH_LR,
        "envelope": {"update_atol": UPDATE_ATOL, "parameter_atol": PARAM_ATOL,
                     "calibration": {"lr": CALIBRATION_LR, "update": UPDATE_ENVELOPE, "parameter": PARAM_ENVELOPE}},
        "gram_bucket_max_bytes": dns.GRAM_BUCKET_MAX_BYTES, "contract": benchmark_contract(), "cases": rows,
        "selection": {r["case"]: r.get("selected") for r in rows if "skipped" not in r},
        "all_selected_pass": all(r.get("selected") is not None for r in rows if "skipped" not in r),
    }
    if artifact_dir is not None and dist.get_rank(group) == 0:
        root = Path(artifact_dir)
        root.mkdir(parents=True, exist_ok=True)
        (root / "manifest.json").write_text(json.dumps(report, indent=1, sort_keys=True))
    if started_group:
        dist.destroy_process_group()
    return report
