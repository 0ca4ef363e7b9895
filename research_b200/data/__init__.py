"""Prepared-token data: manifest validation, memmap token access, deterministic pipelines, synthetic sets."""

from research_b200.data.manifest import (
    PreparedDatasetManifest,
    dataset_manifest_sha256,
    dataset_manifest_summary,
    load_dataset_manifest,
    validate_dataset_manifest,
)
from research_b200.data.pipeline import (
    BatchProvenance,
    DataPipelineState,
    PipelineBatch,
    PreparedTokenDocumentBufferPipeline,
    PreparedTokenWindowPipeline,
    TokenReader,
    TrainingDataPipeline,
    build_prepared_token_pipeline,
    data_pipeline_compat_payload,
    data_pipeline_state_from_mapping,
    data_pipeline_state_to_dict,
    read_token_range,
)
from research_b200.data.synthetic import generate_synthetic_dataset, write_prepared_dataset

__all__ = [
    "BatchProvenance", "DataPipelineState", "PipelineBatch", "PreparedDatasetManifest",
    "PreparedTokenDocumentBufferPipeline", "PreparedTokenWindowPipeline", "TokenReader", "TrainingDataPipeline",
    "build_prepared_token_pipeline", "data_pipeline_compat_payload", "data_pipeline_state_from_mapping",
    "data_pipeline_state_to_dict", "dataset_manifest_sha256", "dataset_manifest_summary",
    "generate_synthetic_dataset", "load_dataset_manifest", "read_token_range", "validate_dataset_manifest",
    "write_prepared_dataset",
]
