"""TOML run contract: loading, validation, canonical JSON and hashes."""

from research_b200.config.canonical import (
    canonical_json,
    load_resolved_config,
    resolved_config_sha256,
    run_spec_from_resolved,
    run_spec_to_dict,
    run_spec_to_json,
    source_config_sha256,
)
from research_b200.config.loader import load_config, run_spec_from_mapping
from research_b200.config.validate import validate_run_spec

__all__ = [
    "canonical_json",
    "load_config",
    "load_resolved_config",
    "resolved_config_sha256",
    "run_spec_from_mapping",
    "run_spec_from_resolved",
    "run_spec_from_resolved_mapping",
    "run_spec_to_dict",
    "run_spec_to_json",
    "source_config_sha256",
    "validate_run_spec",
]

run_spec_from_resolved_mapping = run_spec_from_resolved       # the reference's name for it
