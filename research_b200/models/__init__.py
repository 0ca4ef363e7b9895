"""Decoder and Trinity (MoE) models, parameter metadata, the execution policy of the activation axes."""

from research_b200._lazy import lazy_exports

__getattr__, __dir__, __all__ = lazy_exports(__name__, {
    "AuxLoss": ("research_b200.models.output", "AuxLoss"),
    "DecoderModel": ("research_b200.models.transformer", "TransformerLM"),
    "ExecutionContext": ("research_b200.models.execution", "ExecutionContext"),
    "ModelBuildResult": ("research_b200.models.build", "ModelBuildResult"),
    "ModelExecutionContext": ("research_b200.models.execution", "ExecutionContext"),
    "ModelOutput": ("research_b200.models.output", "ModelOutput"),
    "ParamMeta": ("research_b200.models.build", "ParamMeta"),
    "ParamMetadata": ("research_b200.models.build", "ParamMeta"),
    "RouterStats": ("research_b200.models.output", "RouterStats"),
    "SparseMoE": ("research_b200.models.moe", "SparseMoE"),
    "TransformerLM": ("research_b200.models.transformer", "TransformerLM"),
    "TrinityModel": ("research_b200.models.transformer", "TransformerLM"),
    "apply_model": ("research_b200.models.build", "apply_model"),
    "build_model": ("research_b200.models.build", "build_model"),
    "count_parameters": ("research_b200.models.build", "count_parameters"),
    "dtype_from_name": ("research_b200.models.build", "dtype_from_name"),
    "layout_policy": ("research_b200.models.build", "layout_policy"),
})
