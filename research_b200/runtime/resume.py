"""Resume compatibility: what must not change between a checkpoint and the run that resumes it.

The payload covers seed, the full model and optimizer specs with the optimizer policy summary, mesh, parallelism
and the policies derived from it, the data identity (manifest path + sha256, tokenizer, pipeline description) and
the training contract; its canonical-JSON sha256 is the ``runtime_fingerprint`` stored with every checkpoint.
``target_tokens`` (only when the schedule's ``total_steps`` is explicit), ``log_every_steps`` and
``checkpoint_every_steps`` may change (reference: src/jaxtitan/runtime/resume.py:33-256).
"""

from __future__ import annotations

from dataclasses import dataclass
from hashlib import sha256
from typing import Any, Mapping

from research_b200.config.canonical import canonical_json, normalize
from research_b200.config.specs import RunSpec, resolve_expert_fsdp_axis, resolve_expert_parallel_axis
from research_b200.errors import ContractError

RESUME_METADATA_SCHEMA_VERSION = 1
RESUME_COMPAT_VERSION = 1


@dataclass(frozen=True)
class ResumeCompat:
    payload: dict[str, Any]
    runtime_fingerprint: str


def _hash(payload: Any) -> str:
    return sha256(canonical_json(payload).encode("utf-8")).hexdigest()


def build_resume_compat(spec: RunSpec, *, optimizer_policy: Mapping[str, Any] | None = None,
                        data_pipeline: Mapping[str, Any] | None = None) -> ResumeCompat:
    from research_b200.runtime.trainer import with_runtime_schedule_steps

    spec = with_runtime_schedule_steps(spec)
    sizes = spec.mesh.sizes
    ep = resolve_expert_parallel_axis(spec.parallelism, sizes)
    efsdp = resolve_expert_fsdp_axis(spec.parallelism, sizes)
    if data_pipeline is None and spec.data.mode == "prepared" and spec.data.train_manifest is not None:
        from research_b200.data.pipeline import data_pipeline_compat_payload

        d, t = spec.data, spec.training
        data_pipeline = data_pipeline_compat_payload(
            d.train_manifest, tokenizer_id=d.tokenizer_id, split="train", seq_len=t.seq_len,
            batch_size=t.global_batch_size, order=d.order, shuffle_seed=d.shuffle_seed,
            document_buffer_size=d.document_buffer_size, document_refill_size=d.document_refill_size)
    payload = {
        "compat_version": RESUME_COMPAT_VERSION,
        "seed": spec.seed,
        "model": normalize(spec.model),
        "optimizer": {"spec": normalize(spec.optimizer),
                      "policy": None if optimizer_policy is None else _policy_identity(optimizer_policy)},
        "mesh": normalize(spec.mesh),
        "parallelism": {
            "spec": normalize(spec.parallelism),
            "tensor_parallel": {"enabled": spec.parallelism.tensor_parallel, "axis_size": sizes.get("tp", 1),
                                "sequence_parallel": spec.parallelism.tensor_parallel and not spec.parallelism.context_parallel},
            "context_parallel": {"enabled": spec.parallelism.context_parallel, "axis_size": sizes.get("cp", 1),
                                 "attention": "ring_exact"},
            "expert_parallel": normalize(ep),
            "expert_fsdp": normalize(efsdp),
        },
        "data": {"mode": spec.data.mode, "tokenizer_id": spec.data.tokenizer_id,
                 "hf_streaming": normalize(spec.data.hf_streaming), "pipeline": normalize(data_pipeline)},
        "training": {
            "precision": spec.training.precision, "seq_len": spec.training.seq_len,
            "global_batch_size": spec.training.global_batch_size,
            "gradient_accumulation_steps": spec.training.gradient_accumulation_steps,
            "eval_every_steps": spec.training.eval_every_steps,
            "evals": normalize(spec.evals), "grad_clip_norm": spec.training.grad_clip_norm,
            "loss": normalize(spec.training.loss),
        },
    }
    return ResumeCompat(payload, _hash(payload))


def _policy_identity(policy: Mapping[str, Any]) -> dict[str, Any]:
    return {k: normalize(policy.get(k)) for k in ("name", "adamw", "muon", "dion2", "muon_tp_mode",
                                                  "backend_parameter_counts", "groups")}


def checkpoint_metadata(spec: RunSpec, row: Mapping[str, Any], *, reason: str,
                        eval_row: Mapping[str, Any] | None = None, compat: ResumeCompat | None = None) -> dict[str, Any]:
    compat = compat or build_resume_compat(spec)
    for key in ("step", "tokens_seen", "loss"):
        if key not in row:
            raise ContractError(f"checkpoint metrics row is missing {key!r}")
    return {
        "schema_version": RESUME_METADATA_SCHEMA_VERSION,
        "compat_version": RESUME_COMPAT_VERSION,
        "run_id": spec.run_id,
        "checkpoint": {"step": int(row["step"]), "tokens_seen": int(row["tokens_seen"]), "reason": reason},
        "metrics": {"train_loss": float(row["loss"]),
                    "eval_loss": None if eval_row is None else float(eval_row["loss"])},
        "runtime_fingerprint": compat.runtime_fingerprint,
        "compatibility": compat.payload,
        "mutable_controls": {"target_tokens": spec.training.target_tokens,
                             "log_every_steps": spec.training.log_every_steps,
                             "checkpoint_every_steps": spec.training.checkpoint_every_steps},
    }


def _first_mismatch(stored: Any, current: Any, path: str = "compatibility") -> str:
    if isinstance(stored, Mapping) and isinstance(current, Mapping):
        for key in sorted(set(stored) | set(current)):
            if stored.get(key) != current.get(key):
                return _first_mismatch(stored.get(key), current.get(key), f"{path}.{key}")
        return path
    if isinstance(stored, list) and isinstance(current, list) and len(stored) == len(current):
        for i, (a, b) in enumerate(zip(stored, current)):
            if a != b:
                return _first_mismatch(a, b, f"{path}[{i}]")
    return f"{path}: checkpoint={stored!r} current={current!r}"


def validate_resume_metadata(metadata: Mapping[str, Any], current_spec: RunSpec, *,
                             compat: ResumeCompat | None = None) -> None:
    for key, want in (("schema_version", RESUME_METADATA_SCHEMA_VERSION), ("compat_version", RESUME_COMPAT_VERSION)):
        if metadata.get(key) != want:
            raise ContractError(f"resume metadata {key} must be {want}, got {metadata.get(key)!r}")
    if metadata.get("run_id") != current_spec.run_id:
        raise ContractError(
            f"resume metadata run_id mismatch: checkpoint={metadata.get('run_id')!r} current={current_spec.run_id!r}"
        )
    current = compat or build_resume_compat(current_spec)
    stored_payload = metadata.get("compatibility")
    if not isinstance(stored_payload, Mapping):
        raise ContractError("resume metadata compatibility must be an object")
    fingerprint = metadata.get("runtime_fingerprint")
    if not isinstance(fingerprint, str) or not fingerprint:
        raise ContractError("resume metadata runtime_fingerprint must be a non-empty string")
    if fingerprint != _hash(normalize(stored_payload)):
        raise ContractError("resume metadata runtime_fingerprint does not match compatibility payload")
    if fingerprint != current.runtime_fingerprint:
        raise ContractError(f"resume compatibility mismatch at {_first_mismatch(normalize(stored_payload), current.payload)}")
    checkpoint = metadata.get("checkpoint")
    if not isinstance(checkpoint, Mapping):
        raise ContractError("resume metadata checkpoint must be an object")
    for key in ("step", "tokens_seen"):
        if not isinstance(checkpoint.get(key), int) or isinstance(checkpoint.get(key), bool):
            raise ContractError(f"resume metadata checkpoint.{key} must be an integer")


def validate_resume_compat(restored, current_spec: RunSpec, *, state_step: int, state_tokens: int,
                           compat: ResumeCompat | None = None) -> None:
    validate_resume_metadata(restored.metadata, current_spec, compat=compat)
    ck = restored.metadata["checkpoint"]
    if restored.step != ck["step"]:
        raise ContractError(f"resume checkpoint step mismatch: manager={restored.step} metadata={ck['step']}")
    if state_step != ck["step"]:
        raise ContractError(f"resume checkpoint step mismatch: train_state={state_step} metadata={ck['step']}")
    if state_tokens != ck["tokens_seen"]:
        raise ContractError(
            f"resume checkpoint tokens_seen mismatch: train_state={state_tokens} metadata={ck['tokens_seen']}"
        )
    if restored.host_state.get("dataset") != restored.dataset_state:
        raise ContractError("resume checkpoint host_state.dataset does not match dataset_state")
