"""Optimizer construction: tag-based routing, backend resolution, policy summary.

Routing follows the reference (src/jaxtitan/optim/build.py:36-65, 412-467, 672-747): with ``optimizer.name =
"muon"`` the hidden matrices (attention q/k/v/o/gate, MLP and shared-expert gate/up/down, routed expert stacks)
go to the matrix optimizer and everything else (embedding, lm_head, norms, router) falls back to AdamW with
b1/b2/eps = 0.9/0.999/1e-8; weight decay applies to everything except ``expert_bias``.

Backend resolution differs where the hardware design differs: the reference turns Muon into Dion2 whenever
the optimizer state is FSDP-sharded (build.py:682-685) because a sharded leaf cannot be orthogonalised locally.
Here sharded sections assign *whole matrices* to owners, so ``muon`` stays Muon under ``zero2``/``fsdp``
("owner-distributed Muon"); ``optimizer.name = "dion"`` selects Dion2 explicitly.  Tensor-parallel shards use
``dist_muon`` in ``duplicated`` or ``distributed`` mode as in the reference.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from research_b200.config.specs import OptimizerSpec
from research_b200.errors import ContractError
from research_b200.models.build import NORM_TAGS, ROUTED_EXPERT_TAGS, ParamMeta
from research_b200.optim.orthogonalize import dion2_policy_constants, muon_policy_constants
from research_b200.optim.schedules import build_lr_schedule

ADAMW_B1 = 0.9
ADAMW_B2 = 0.999
ADAMW_EPS = 1e-8
SUPPORTED_RUNTIME_BACKENDS = ("adamw", "dion", "muon")
MUON_MATRIX_TAGS = frozenset({
    "attention_q", "attention_k", "attention_v", "attention_o", "attention_gate", "mlp_gate", "mlp_up", "mlp_down",
    "moe_shared_gate", "moe_shared_up", "moe_shared_down",
})
MUON_TAGS = MUON_MATRIX_TAGS | ROUTED_EXPERT_TAGS


@dataclass(frozen=True)
class RouteAssignment:
    path: tuple[str, ...]
    tag: str
    backend: str                     # adamw | muon | dist_muon | dion2
    weight_decay: bool
    requested_backend: str
    auto_resolved: bool
    resolution_reason: str | None
    fallback_reason: str | None
    matrix_axis: int | None          # logical axis that is split (tp for dist_muon, fsdp policy axis for dion2)

    @property
    def name(self) -> str:
        return ".".join(self.path)


@dataclass
class OptimizerBuildResult:
    spec: OptimizerSpec
    schedule: Callable[[int], float]
    adamw_fallback_schedule: Callable[[int], float] | None
    route_assignments: tuple[RouteAssignment, ...]
    description: str
    muon_execution_plans: tuple = ()          # one MuonLeafPlan per tensor-parallel-sharded Muon matrix

    def backend_by_name(self) -> dict[str, str]:
        """Storage-level backend per logical parameter: adamw | muon | dion2 (dist_muon is a muon mode)."""

        return {a.name: ("muon" if a.backend == "dist_muon" else a.backend) for a in self.route_assignments}

    def weight_decay_by_name(self) -> dict[str, bool]:
        """Whether decoupled weight decay applies, per logical parameter (reference mask: optim/build.py:506-518)."""

        return {a.name: a.weight_decay for a in self.route_assignments}


def _fallback_reason(spec: OptimizerSpec, item: ParamMeta, backend: str, explicit: bool) -> str | None:
    if spec.name not in ("muon", "dion") or backend != "adamw":
        return None
    if explicit:
        return "route_rule"
    if item.tag in ("embedding", "lm_head"):
        return item.tag
    if item.tag in NORM_TAGS:
        return "norm"
    if item.tag == "moe_expert_bias":
        return "expert_bias"
    if len(item.shape) != 2:
        return "rank_not_two"
    return "not_hidden_matrix"


def route_assignments(spec: OptimizerSpec, metadata: tuple[ParamMeta, ...], *, tp_size: int = 1) -> tuple[RouteAssignment, ...]:
    known_tags = {m.tag for m in metadata}
    seen = set()
    for m in metadata:
        if m.path in seen:
            raise ContractError(f"optimizer metadata contains duplicate parameter path {m.name!r}")
        seen.add(m.path)
    rules = {}
    for rule in spec.route_rules:
        if rule.tag not in known_tags:
            raise ContractError(f"optimizer route tag {rule.tag!r} does not match any model parameter metadata tag")
        if rule.tag in rules:
            raise ContractError(f"optimizer route tag {rule.tag!r} is configured more than once")
        if rule.transform not in SUPPORTED_RUNTIME_BACKENDS:
            raise ContractError(
                f"optimizer route transform {rule.transform!r} has no runtime adapter yet; "
                f"supported runtime backends: {sorted(SUPPORTED_RUNTIME_BACKENDS)}"
            )
        rules[rule.tag] = rule
    out = []
    for m in metadata:
        rule = rules.get(m.tag)
        if rule is not None:
            requested = rule.transform
        elif spec.name in ("muon", "dion") and m.tag in MUON_TAGS:
            requested = spec.name
        else:
            requested = "adamw"
        backend, axis, reason = requested, None, None
        if requested == "dion":
            backend, axis, reason = "dion2", m.fsdp_axis, "explicit_dion"
            if m.tag in ROUTED_EXPERT_TAGS:
                axis = 2 if m.tag in ("moe_gate", "moe_up") else 1
        elif requested == "muon" and m.tag in MUON_MATRIX_TAGS and tp_size > 1 and m.tp_axis is not None:
            backend, axis, reason = "dist_muon", m.tp_axis, "tp_sharded_matrix_muon"
        if backend in ("muon", "dist_muon", "dion2") and len(m.shape) not in (2, 3):
            raise ContractError(f"parameter {m.name!r} with shape {m.shape} cannot use matrix optimizer {backend}")
        wd = (m.tag != "moe_expert_bias") if rule is None else bool(rule.weight_decay and m.tag != "moe_expert_bias")
        out.append(RouteAssignment(m.path, m.tag, backend, wd, requested, backend != requested, reason,
                                   _fallback_reason(spec, m, backend, rule is not None), axis))
    return tuple(out)


def describe_optimizer(spec: OptimizerSpec) -> str:
    clip = "none" if spec.grad_clip_norm is None else f"{spec.grad_clip_norm:g}"
    sch = spec.schedule
    total = "none" if sch.total_steps is None else str(sch.total_steps)
    stable = "none" if sch.stable_steps is None else str(sch.stable_steps)
    fb = spec.adamw_fallback_schedule
    fb_text = "none" if fb is None else f"{fb.name}:peak_lr={fb.peak_lr:g}:warmup_steps={fb.warmup_steps}"
    suffix = f" muon_tp_mode={spec.muon_tp_mode}" if spec.name in ("muon", "dion") else ""
    return (
        f"{spec.name} schedule={sch.name} peak_lr={sch.peak_lr:g} warmup_steps={sch.warmup_steps} "
        f"total_steps={total} min_lr_ratio={sch.min_lr_ratio:g} stable_steps={stable} "
        f"adamw_fallback_schedule={fb_text} weight_decay={spec.weight_decay:g} grad_clip_norm={clip} "
        f"adamw_b1={ADAMW_B1:g} adamw_b2={ADAMW_B2:g} adamw_eps={ADAMW_EPS:g}{suffix}"
    )


def build_optimizer(spec: OptimizerSpec, metadata: tuple[ParamMeta, ...], *, tp_size: int = 1) -> OptimizerBuildResult:
    if spec.name not in SUPPORTED_RUNTIME_BACKENDS:
        raise ContractError(
            f"optimizer.name {spec.name!r} is valid config but has no runtime adapter yet; "
            f"supported runtime backends: {sorted(SUPPORTED_RUNTIME_BACKENDS)}"
        )
    assignments = route_assignments(spec, tuple(metadata), tp_size=tp_size)
    schedule = build_lr_schedule(spec.schedule)
    fallback = None if spec.adamw_fallback_schedule is None else build_lr_schedule(spec.adamw_fallback_schedule)
    from research_b200.optim.distributed_ns import build_muon_execution_plans

    plans = build_muon_execution_plans(assignments, tuple(metadata), tp_size=tp_size, requested_mode=spec.muon_tp_mode)
    return OptimizerBuildResult(spec, schedule, fallback, assignments, describe_optimizer(spec), plans)


def _muon_plan_summary(result: OptimizerBuildResult) -> dict[str, Any] | None:
    if not result.muon_execution_plans:
        return None
    from research_b200.optim.distributed_ns import summarize_plans

    return summarize_plans(result.muon_execution_plans)


def schedule_payload(spec) -> dict[str, Any] | None:
    if spec is None:
        return None
    return {"name": spec.name, "peak_lr": spec.peak_lr, "warmup_steps": spec.warmup_steps,
            "total_steps": spec.total_steps, "min_lr_ratio": spec.min_lr_ratio, "stable_steps": spec.stable_steps}


def distributed_policy_payload(name: str) -> dict[str, str]:
    """How each optimizer family lives with sharded state here (reference: optim/build.py:470-487, whose Muon turns
    into Dion2 under FSDP; here whole matrices go to owner ranks instead)."""

    if name == "adamw":
        return {"optimizer_state": "elementwise_shard_safe", "gradient_update": "elementwise_shard_safe",
                "zero2_fsdp": "supported"}
    if name == "muon":
        return {"optimizer_state": "whole_matrices_on_owner_ranks_or_tp_sharded_dist_muon",
                "gradient_update": "muon_on_the_owner_rank_dist_muon_for_tp",
                "zero2_fsdp": "owner_distributed_muon"}
    if name == "dion":
        return {"optimizer_state": "whole_matrices_on_owner_ranks", "gradient_update": "dion2_on_the_owner_rank",
                "zero2_fsdp": "owner_distributed_dion2"}
    return {"optimizer_state": "unknown", "gradient_update": "unknown", "zero2_fsdp": "unsupported"}


def route_distributed_policy(backend: str, *, muon_tp_mode: str) -> str:
    if backend == "adamw":
        return "elementwise_shard_safe"
    if backend in ("muon", "dion2"):
        return "complete_matrix_or_per_expert_complete_matrix"
    if backend == "dist_muon":
        return "duplicated_full_logical_matrix" if muon_tp_mode == "duplicated" else "sharded_gram_collectives"
    return "unknown"


def dist_muon_policy_payload(spec: OptimizerSpec) -> dict[str, Any]:
    """What the tensor-parallel Muon mode promises (reference: optim/build.py:332-359)."""

    common = {"requested_mode": spec.muon_tp_mode,
              "newton_schulz_precision": muon_policy_constants().get("newton_schulz_precision"),
              "replicated_model_axis_reduction": "mean", "auto_selected_for": "tp_sharded_muon_matrix_routes"}
    if spec.muon_tp_mode == "duplicated":
        return {**common, "distributed_policy": "duplicated_full_logical_matrix", "exact": True,
                "approximation": "none", "execution": "duplicated",
                "performance": "single_bf16_logical_matrix_gather",
                "numerical_contract": "accepted_bfloat16_reference"}
    return {**common, "distributed_policy": "sharded_gram_collectives", "exact": False,
            "approximation": "floating_point_reduction_order", "execution": "distributed",
            "performance": "one_norm_plus_five_gram_reductions_with_optional_exchange",
            "numerical_contract": "deterministic_close_not_bitwise"}


def optimizer_policy_summary(result: OptimizerBuildResult, metadata: tuple[ParamMeta, ...] | None = None) -> dict[str, Any]:
    """Stable payload for ``diagnostics/runtime.json`` and the resume fingerprint
    (sections of the reference's payload: optim/build.py:231-329)."""

    by_backend: dict[str, int] = {}
    fallbacks: dict[str, int] = {}
    groups: dict[tuple[str, str], int] = {}
    for a in result.route_assignments:
        by_backend[a.backend] = by_backend.get(a.backend, 0) + 1
        groups[(a.tag, a.backend)] = groups.get((a.tag, a.backend), 0) + 1
        if a.fallback_reason is not None:
            fallbacks[a.fallback_reason] = fallbacks.get(a.fallback_reason, 0) + 1
    spec = result.spec
    shapes = {} if metadata is None else {m.path: list(m.shape) for m in metadata}
    plan_summary = _muon_plan_summary(result)
    dist_muon = dist_muon_policy_payload(spec)
    if plan_summary is not None:
        dist_muon["leaf_execution_plans"] = plan_summary["leaves"]
    return {
        "name": spec.name,
        "requested_name": spec.name,
        "description": result.description,
        "schedule": schedule_payload(spec.schedule),
        "adamw_fallback_schedule": schedule_payload(spec.adamw_fallback_schedule),
        "supported_runtime_backends": sorted(SUPPORTED_RUNTIME_BACKENDS),
        "internal_runtime_backends": ["dion2", "dist_muon"],
        "distributed_policy": distributed_policy_payload(spec.name),
        "adamw": {"b1": ADAMW_B1, "b2": ADAMW_B2, "eps": ADAMW_EPS, "distributed_policy": "elementwise_shard_safe"},
        "muon": None if spec.name != "muon" else {
            **muon_policy_constants(), "tp_mode": spec.muon_tp_mode,
            "distributed_policy": "owner_distributed_complete_matrices",
            "rank3_expert_policy": "per_expert_full_matrix",
            "hidden_matrix_tags": sorted(MUON_MATRIX_TAGS), "routed_expert_matrix_tags": sorted(ROUTED_EXPERT_TAGS),
            "fallback_tags": ["embedding", "lm_head", *sorted(NORM_TAGS)]},
        "dion2": None if spec.name != "dion" else {**dion2_policy_constants(),
                                                    "distributed_policy": "owner_distributed_complete_matrices"},
        "dist_muon": dist_muon,
        "auto_routing": {"muon_sharded_matrix_backend": "muon", "muon_tp_sharded_matrix_backend": "dist_muon",
                         "active": any(a.auto_resolved for a in result.route_assignments)},
        "muon_tp_mode": spec.muon_tp_mode,
        "muon_tp_execution": plan_summary,
        "backend_parameter_counts": dict(sorted(by_backend.items())),
        "route_counts": dict(sorted(by_backend.items())),
        "fallback_counts": dict(sorted(fallbacks.items())),
        "groups": [{"tag": t, "backend": b, "parameters": n} for (t, b), n in sorted(groups.items())],
        "routes": [
            {"path": a.name, "tag": a.tag, "backend": a.backend, "weight_decay": a.weight_decay,
             "requested_backend": a.requested_backend, "auto_resolved": a.auto_resolved,
             "resolution_reason": a.resolution_reason, "fallback_reason": a.fallback_reason,
             "matrix_axis": a.matrix_axis, "logical_shape": shapes.get(a.path),
             "distributed_policy": route_distributed_policy(a.backend, muon_tp_mode=spec.muon_tp_mode)}
            for a in result.route_assignments
        ],
    }
