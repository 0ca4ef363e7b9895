"""The sm_100a kernel library: in-tree build with a source-keyed cache, registry, per-run kernel plan, benches."""

from research_b200._lazy import lazy_exports

__getattr__, __dir__, __all__ = lazy_exports(__name__, {
    "benchmark_kernel": ("research_b200.kernels.bench", "benchmark_kernel"),
    "build_all": ("research_b200.kernels.build", "build_all"),
    "compile_kernel_plan": ("research_b200.kernels.registry", "compile_kernel_plan"),
    "enrich_kernel_plan_with_cache": ("research_b200.kernels.registry", "enrich_kernel_plan_with_cache"),
    "format_compile_result": ("research_b200.kernels.registry", "format_compile_result"),
    "format_kernel_plan": ("research_b200.kernels.registry", "format_kernel_plan"),
    "format_kernel_registry": ("research_b200.kernels.registry", "format_kernel_registry"),
    "kernel_plan": ("research_b200.kernels.registry", "kernel_plan"),
    "kernel_plan_to_json": ("research_b200.kernels.registry", "kernel_plan_to_json"),
    "kernel_registry": ("research_b200.kernels.registry", "kernel_registry"),
    "kernel_registry_payload": ("research_b200.kernels.registry", "kernel_registry_payload"),
    "load_cache_manifest": ("research_b200.kernels.registry", "load_cache_manifest"),
    "require_kernel_plan_supported": ("research_b200.kernels.registry", "require_kernel_plan_supported"),
})
