"""Optimizers: routing by parameter tag, AdamW, Muon, Dion2, schedules, the distributed Newton-Schulz plans."""

from research_b200._lazy import lazy_exports

__getattr__, __dir__, __all__ = lazy_exports(__name__, {
    "MuonLeafPlan": ("research_b200.optim.distributed_ns", "MuonLeafPlan"),
    "Optimizer": ("research_b200.optim.optimizer", "Optimizer"),
    "OptimizerBuildResult": ("research_b200.optim.build", "OptimizerBuildResult"),
    "OptimizerTransform": ("research_b200.optim.optimizer", "Optimizer"),
    "RouteAssignment": ("research_b200.optim.build", "RouteAssignment"),
    "build_lr_schedule": ("research_b200.optim.schedules", "build_lr_schedule"),
    "build_muon_execution_plans": ("research_b200.optim.distributed_ns", "build_muon_execution_plans"),
    "build_optimizer": ("research_b200.optim.build", "build_optimizer"),
    "describe_optimizer": ("research_b200.optim.build", "describe_optimizer"),
    "dion2_policy_constants": ("research_b200.optim.orthogonalize", "dion2_policy_constants"),
    "muon_policy_constants": ("research_b200.optim.orthogonalize", "muon_policy_constants"),
    "optimizer_policy_summary": ("research_b200.optim.build", "optimizer_policy_summary"),
    "polar_express": ("research_b200.optim.orthogonalize", "polar_express"),
    "route_assignments": ("research_b200.optim.build", "route_assignments"),
    "select_dion2_slices": ("research_b200.optim.orthogonalize", "select_dion2_slices"),
    "zeropower_via_newton_schulz": ("research_b200.optim.orthogonalize", "zeropower_via_newton_schulz"),
})
