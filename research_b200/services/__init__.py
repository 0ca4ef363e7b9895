"""Host services: run artifacts, checkpoints, the optional W&B mirror."""

from research_b200._lazy import lazy_exports

__getattr__, __dir__, __all__ = lazy_exports(__name__, {
    "ArtifactWriter": ("research_b200.services.artifacts", "LocalArtifactWriter"),
    "CheckpointRestore": ("research_b200.services.checkpoints", "CheckpointRestore"),
    "CheckpointService": ("research_b200.services.checkpoints", "LocalCheckpointService"),
    "LocalArtifactWriter": ("research_b200.services.artifacts", "LocalArtifactWriter"),
    "LocalCheckpointService": ("research_b200.services.checkpoints", "LocalCheckpointService"),
    "LocalOrbaxCheckpointService": ("research_b200.services.checkpoints", "LocalCheckpointService"),
    "MirroredArtifactWriter": ("research_b200.services.wandb", "WandbMirroredWriter"),
    "NullArtifactWriter": ("research_b200.services.artifacts", "NullArtifactWriter"),
    "WandbMirroredWriter": ("research_b200.services.wandb", "WandbMirroredWriter"),
    "build_artifact_writer": ("research_b200.services.artifacts", "build_artifact_writer"),
    "initialize_run": ("research_b200.services.artifacts", "initialize_run"),
    "namespaced_metrics": ("research_b200.services.wandb", "namespaced_metrics"),
    "read_array": ("research_b200.services.checkpoints", "read_array"),
    "wandb_run_id": ("research_b200.services.wandb", "wandb_run_id"),
    "write_array": ("research_b200.services.checkpoints", "write_array"),
})
