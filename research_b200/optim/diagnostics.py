"""Per-group optimizer diagnostics: gradient / update / parameter norms of every ``tag:backend`` group, the
health roll-up derived from them, and the per-layer router summary.

Payload fields and roll-up rules follow the reference (src/jaxtitan/steps/train.py:480-566 group templates and
norms; src/jaxtitan/runtime/training.py:1175-1268 payload and health fields, 1277-1313 router layers).  The
norms are computed on steps that log: every rank sums the squares of the elements it holds (its range of a sharded
section, its tensor- or expert-parallel slice), one packed reduction per mesh axis adds the pieces, and the result
rides to the host in the step's single device-to-host read.
"""

from __future__ import annotations

import math
from typing import Any

import numpy as np
import torch
import torch.distributed as dist


def group_templates(assignments, metadata) -> tuple[list[dict[str, Any]], dict[str, int]]:
    """One template per ``(tag, backend)`` in route order, and the group index of every logical parameter."""

    shapes = {m.name: m.shape for m in metadata}
    groups: list[dict[str, Any]] = []
    by_key: dict[tuple[str, str], int] = {}
    index_of: dict[str, int] = {}
    for a in assignments:
        key = (a.tag, a.backend)
        if key not in by_key:
            by_key[key] = len(groups)
            groups.append({"group": f"{a.tag}:{a.backend}", "tag": a.tag, "backend": a.backend, "leaf_count": 0,
                           "parameter_count": 0, "weight_decay_enabled_count": 0, "auto_resolved_count": 0})
        g = groups[by_key[key]]
        g["leaf_count"] += 1
        g["parameter_count"] += int(math.prod(shapes.get(a.name, ())))
        g["weight_decay_enabled_count"] += int(bool(a.weight_decay))
        g["auto_resolved_count"] += int(bool(a.auto_resolved))
        index_of[a.name] = by_key[key]
    return groups, index_of


def _flat_ranges(meta, param_shape) -> list[tuple[int, int]]:
    """Element ranges, inside the flattened storage parameter, that hold one logical parameter."""

    numel = int(math.prod(param_shape))
    if meta.rows is None:
        return [(0, numel)]
    a, b = meta.rows
    cols = int(param_shape[-1])
    if len(param_shape) == 3:
        per = int(param_shape[1]) * cols
        return [(e * per + a * cols, e * per + b * cols) for e in range(int(param_shape[0]))]
    return [(a * cols, b * cols)]


def group_square_sums(optimizer, before: list[torch.Tensor | None], sumsq) -> torch.Tensor:
    """``[groups, 3]`` sums of squares (gradient, update, parameter) over the whole model.

    ``before[i]`` is the fp32 master copy of section ``i`` from before the update (``None`` for frozen sections);
    ``sumsq(x, out, index)`` accumulates ``sum(x^2)`` into ``out[index]``."""

    store = optimizer.store
    groups = len(optimizer.group_templates)
    dev = store.device
    per_section = []
    for i, sec in enumerate(store.sections):
        acc = torch.zeros(groups * 3, dtype=torch.float32, device=dev)
        per_section.append(acc)
        if sec.backend == "frozen" or before[i] is None:
            continue
        lo, hi = store.local_master_range(sec)
        update = (sec.master - before[i]).contiguous()
        for e in sec.entries:
            for meta in e.metas:
                g = optimizer.group_index.get(meta.name)
                if g is None:
                    continue
                for a, b in _flat_ranges(meta, e.param.shape):
                    a2, b2 = max(e.offset + a, lo), min(e.offset + b, hi)
                    if b2 <= a2:
                        continue
                    sumsq(store.grad_arena[a2:b2], acc, 3 * g)
                    sumsq(update[a2 - lo:b2 - lo], acc, 3 * g + 1)
                    sumsq(sec.master[a2 - lo:b2 - lo], acc, 3 * g + 2)
    axes: dict[str, list[int]] = {}
    for i, sec in enumerate(store.sections):
        for axis in optimizer._sum_axes(sec):
            axes.setdefault(axis, []).append(i)
    for axis, idx in axes.items():
        group = optimizer.mesh.group(axis)
        if group is None:
            continue
        packed = torch.stack([per_section[i] for i in idx])
        dist.all_reduce(packed, group=group)
        for row, i in enumerate(idx):
            per_section[i] = packed[row]
    total = torch.stack(per_section).sum(dim=0) if per_section else torch.zeros(groups * 3, device=dev)
    return total.view(groups, 3)


def _safe_ratio(num: float, den: float) -> float:
    return 0.0 if den <= 0.0 else num / den


def groups_payload(templates: list[dict[str, Any]], squares) -> list[dict[str, Any]]:
    """Rows of ``optimizer_groups`` from the templates and the ``[groups, 3]`` sums of squares (host values)."""

    sq = np.asarray(squares, dtype=np.float64).reshape(len(templates), 3)
    rows = []
    for t, (g2, u2, p2) in zip(templates, sq):
        grad, update, param = (float(np.sqrt(v)) if v >= 0 or np.isnan(v) else float("nan") for v in (g2, u2, p2))
        upr, gpr = _safe_ratio(update, param), _safe_ratio(grad, param)
        rows.append({
            "group": t["group"], "tag": t["tag"], "backend": t["backend"],
            "parameter_count": int(t["parameter_count"]), "leaf_count": int(t["leaf_count"]),
            "grad_norm": grad, "update_norm": update, "param_norm": param,
            "grad_param_ratio": gpr, "update_param_ratio": upr,
            "grad_norm_finite": math.isfinite(grad), "update_norm_finite": math.isfinite(update),
            "param_norm_finite": math.isfinite(param), "grad_param_ratio_finite": math.isfinite(gpr),
            "update_param_ratio_finite": math.isfinite(upr),
            "weight_decay_enabled_count": int(t["weight_decay_enabled_count"]),
            "auto_resolved_count": int(t["auto_resolved_count"]),
        })
    return rows


HEALTH_KEYS = ("optimizer_grad_norm_max_group", "optimizer_update_norm_max_group", "optimizer_update_param_ratio_max",
               "optimizer_update_param_ratio_mean", "optimizer_groups_with_zero_grad",
               "optimizer_groups_with_zero_update", "optimizer_nonfinite_group_count", "optimizer_nonfinite_groups",
               "optimizer_route_backend_counts")


def health_fields(groups: list[dict[str, Any]] | None) -> dict[str, Any]:
    """The roll-up of one step's groups that goes into the train row, the summary and ``run inspect``."""

    if not groups:
        return {k: None for k in HEALTH_KEYS}
    fin = math.isfinite
    finite_grad = [g for g in groups if fin(g["grad_norm"])]
    finite_update = [g for g in groups if fin(g["update_norm"])]
    ratios = [g["update_param_ratio"] for g in groups if fin(g["update_param_ratio"])]
    bad = [g["group"] for g in groups
           if not all(fin(g[k]) for k in ("grad_norm", "update_norm", "param_norm", "grad_param_ratio",
                                          "update_param_ratio"))]
    backends: dict[str, int] = {}
    for g in groups:
        backends[g["backend"]] = backends.get(g["backend"], 0) + int(g["leaf_count"])
    return {
        "optimizer_grad_norm_max_group": max(finite_grad, key=lambda g: g["grad_norm"])["group"] if finite_grad else None,
        "optimizer_update_norm_max_group":
            max(finite_update, key=lambda g: g["update_norm"])["group"] if finite_update else None,
        "optimizer_update_param_ratio_max": max(ratios) if ratios else None,
        "optimizer_update_param_ratio_mean": float(np.mean(ratios)) if ratios else None,
        "optimizer_groups_with_zero_grad": sum(1 for g in groups if g["grad_norm"] <= 0.0),
        "optimizer_groups_with_zero_update": sum(1 for g in groups if g["update_norm"] <= 0.0),
        "optimizer_nonfinite_group_count": len(bad),
        "optimizer_nonfinite_groups": bad,
        "optimizer_route_backend_counts": dict(sorted(backends.items())),
    }


def _percent(values: np.ndarray) -> np.ndarray:
    total = float(values.sum())
    return np.zeros_like(values, dtype=np.float64) if total <= 0.0 else values / total * 100.0


def _cv(values: np.ndarray) -> float:
    mean = float(values.mean()) if values.size else 0.0
    return 0.0 if mean <= 0.0 else float(values.std() / mean * 100.0)


def _entropy(values: np.ndarray) -> float:
    total = float(values.sum())
    if total <= 0.0:
        return 0.0
    p = values / total
    p = p[p > 0.0]
    return float(-(p * np.log(p)).sum())


def router_layers_payload(layers: list[dict[str, Any]]) -> list[dict[str, Any]]:
    """``moe_router_layers`` rows: per-layer expert counts and importance with load / importance quantiles (in
    percent of the layer's total), coefficient of variation, entropy and the number of active experts."""

    rows = []
    for item in layers:
        counts = np.asarray(item["counts"].tolist() if torch.is_tensor(item["counts"]) else item["counts"], dtype=np.float64)
        imp = np.asarray(item["importance"].tolist() if torch.is_tensor(item["importance"]) else item["importance"],
                         dtype=np.float64)
        load_pct, imp_pct = _percent(counts), _percent(imp)
        q = lambda v, x: float(np.quantile(v, x)) if v.size else 0.0  # noqa: E731
        rows.append({
            "layer_index": int(item["layer_index"]), "total_assignments": float(counts.sum()),
            "expert_counts": [int(v) for v in counts.tolist()],
            "load_min": q(load_pct, 0.0), "load_p10": q(load_pct, 0.10), "load_p50": q(load_pct, 0.50),
            "load_p90": q(load_pct, 0.90), "load_max": q(load_pct, 1.0), "load_cv": _cv(counts),
            "load_entropy": _entropy(counts), "experts_active": int(np.count_nonzero(counts > 0.0)),
            "importance": [float(v) for v in imp.tolist()],
            "importance_min": q(imp_pct, 0.0), "importance_p10": q(imp_pct, 0.10), "importance_p50": q(imp_pct, 0.50),
            "importance_p90": q(imp_pct, 0.90), "importance_max": q(imp_pct, 1.0), "importance_cv": _cv(imp),
            "importance_entropy": _entropy(imp),
        })
    return rows
