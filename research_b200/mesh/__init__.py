"""The reference's ``mesh`` package under its own name: mesh context, batch placement, the sharding plan.

What JAX expresses as a sharding plan over one process is here one process per GPU: ``MeshContext`` holds the
process groups of the named axes, ``ParamStore`` is the plan of where parameters, gradients and optimizer state
live, and a batch is placed by slicing the rows and sequence positions of this rank and staging them on the device.
"""

from research_b200._lazy import lazy_exports

__getattr__, __dir__, __all__ = lazy_exports(__name__, {
    "MeshContext": ("research_b200.parallel.mesh", "MeshContext"),
    "build_mesh_context": ("research_b200.parallel.mesh", "build_mesh_context"),
    "init_distributed": ("research_b200.parallel.mesh", "init_distributed"),
    "execution_context_for": ("research_b200.parallel.mesh", "execution_context_for"),
    "require_single_node_runtime": ("research_b200.parallel.mesh", "require_single_node_runtime"),
    "require_single_process_runtime": ("research_b200.parallel.mesh", "require_single_node_runtime"),
    "validate_runtime_mesh_spec": ("research_b200.parallel.mesh", "validate_runtime_mesh_spec"),
    "ShardingPlan": ("research_b200.parallel.sharding", "ParamStore"),
    "build_sharding_plan": ("research_b200.parallel.sharding", "ParamStore"),
    "ParamStore": ("research_b200.parallel.sharding", "ParamStore"),
    "BatchSharding": ("research_b200.steps.train", "BatchStager"),
    "place_batch": ("research_b200.steps.train", "local_batch_slices"),
    "local_batch_slices": ("research_b200.steps.train", "local_batch_slices"),
})
