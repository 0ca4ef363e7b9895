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


# names that resolve on first use (prepare, inspect and streaming pull in tokenizers and, for streaming, ``datasets``)
from research_b200._lazy import lazy_exports as _lazy_exports

_EAGER = tuple(__all__)
__getattr__, __dir__, __all__ = _lazy_exports(__name__, {
    "DATA_PIPELINE_BACKEND": ("research_b200.data.pipeline", "BACKEND"),
    "DATA_PIPELINE_STATE_SCHEMA_VERSION": ("research_b200.data.pipeline", "STATE_SCHEMA_VERSION"),
    "DATA_PIPELINE_DEFAULT_ORDER": ("research_b200.data.pipeline", "DEFAULT_ORDER"),
    "DATA_PIPELINE_DEFAULT_WORKER_COUNT": ("research_b200.data.pipeline", "DEFAULT_WORKER_COUNT"),
    "DATA_PIPELINE_DEFAULT_WORKER_BUFFER_SIZE": ("research_b200.data.pipeline", "DEFAULT_WORKER_BUFFER_SIZE"),
    "DATA_PIPELINE_DEFAULT_PREFETCH": ("research_b200.data.pipeline", "DEFAULT_PREFETCH"),
    "backend_version": ("research_b200.data.pipeline", "backend_version"),
    "open_document_offsets": ("research_b200.data.pipeline", "open_document_offsets"),
    "PreparedTokenDataSource": ("research_b200.data.pipeline", "TokenReader"),
    "PreparedTokenGrainPipeline": ("research_b200.data.pipeline", "PreparedTokenWindowPipeline"),
    "TokenShard": ("research_b200.data.manifest", "TokenShard"),
    "TokenSplit": ("research_b200.data.manifest", "TokenSplit"),
    "DocumentTable": ("research_b200.data.manifest", "DocumentTable"),
    "prepared_dataset_manifest_to_dict": ("research_b200.data.manifest", "prepared_dataset_manifest_to_dict"),
    "prepared_dataset_manifest_to_json": ("research_b200.data.manifest", "prepared_dataset_manifest_to_json"),
    "HF_STREAMING_BACKEND": ("research_b200.data.streaming", "STREAM_BACKEND"),
    "HFStreamingTextPipeline": ("research_b200.data.streaming", "HFStreamingTextPipeline"),
    "build_hf_streaming_pipeline": ("research_b200.data.streaming", "build_hf_streaming_pipeline"),
    "hf_streaming_compat_payload": ("research_b200.data.streaming", "hf_streaming_compat_payload"),
    "datasets_version": ("research_b200.data.streaming", "datasets_version"),
    "PrepareConfig": ("research_b200.data.prepare", "PrepareConfig"),
    "PrepareOutputConfig": ("research_b200.data.prepare", "PrepareOutputConfig"),
    "PrepareSourceConfig": ("research_b200.data.prepare", "PrepareSourceConfig"),
    "PrepareTokenizerConfig": ("research_b200.data.prepare", "PrepareTokenizerConfig"),
    "PrepareTokenizationConfig": ("research_b200.data.prepare", "PrepareTokenizationConfig"),
    "TOKEN_BYTES_FILENAME": ("research_b200.data.prepare", "TOKEN_BYTES_FILENAME"),
    "DOCUMENT_OFFSETS_FILENAME": ("research_b200.data.prepare", "DOCUMENT_OFFSETS_FILENAME"),
    "load_prepare_config": ("research_b200.data.prepare", "load_prepare_config"),
    "prepare_config_from_mapping": ("research_b200.data.prepare", "prepare_config_from_mapping"),
    "prepare_dataset": ("research_b200.data.prepare", "prepare_dataset"),
    "prepare_result_to_dict": ("research_b200.data.prepare", "prepare_result_to_dict"),
    "prepare_result_to_json": ("research_b200.data.prepare", "prepare_result_to_json"),
    "format_prepare_result": ("research_b200.data.prepare", "format_prepare_result"),
    "build_token_bytes": ("research_b200.data.prepare", "build_token_bytes"),
    "load_hf_texts": ("research_b200.data.prepare", "load_hf_texts"),
    "load_tokenizer": ("research_b200.data.prepare", "load_tokenizer"),
    "inspect_dataset": ("research_b200.data.inspect", "inspect_dataset"),
    "inspect_dataset_manifest": ("research_b200.data.inspect", "inspect_dataset_manifest"),
    "data_config_snippet": ("research_b200.data.inspect", "data_config_snippet"),
    "data_inspection_to_dict": ("research_b200.data.inspect", "data_inspection_to_dict"),
    "data_inspection_to_json": ("research_b200.data.inspect", "data_inspection_to_json"),
    "format_data_inspection": ("research_b200.data.inspect", "format_data_inspection"),
}, eager=_EAGER)
