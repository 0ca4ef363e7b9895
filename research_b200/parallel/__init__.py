"""Mesh axes as process groups, the parameter store (DDP / ZeRO-2 / FSDP), symmetric arenas, TP / CP / EP paths."""

from research_b200._lazy import lazy_exports

__getattr__, __dir__, __all__ = lazy_exports(__name__, {
    "MeshContext": ("research_b200.parallel.mesh", "MeshContext"),
    "ParamStore": ("research_b200.parallel.sharding", "ParamStore"),
    "SymmetricArena": ("research_b200.parallel.symmetric", "SymmetricArena"),
    "build_mesh_context": ("research_b200.parallel.mesh", "build_mesh_context"),
    "execution_context_for": ("research_b200.parallel.mesh", "execution_context_for"),
    "init_distributed": ("research_b200.parallel.mesh", "init_distributed"),
    "require_single_node_runtime": ("research_b200.parallel.mesh", "require_single_node_runtime"),
    "validate_runtime_mesh_spec": ("research_b200.parallel.mesh", "validate_runtime_mesh_spec"),
})
