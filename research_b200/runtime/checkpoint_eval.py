"""``eval checkpoint``: validation loss of a retained checkpoint -> ``evals/checkpoints/<step>.json``
(reference: src/jaxtitan/runtime/checkpoint_eval.py:24-96).

The payload carries the reference's sections (``checkpoint``, ``eval``, ``data``) and, at the top level, the figures a
script usually wants (``loss``, ``bpb``, ``token_count``, ``checkpoint_step``).
"""

from __future__ import annotations

import json
import time
from pathlib import Path
from typing import Any, Mapping

from research_b200.config.canonical import normalize
from research_b200.errors import ContractError
from research_b200.infer.checkpoint import restore_inference_checkpoint
from research_b200.runtime.diagnostics import enrich_eval_metrics
from research_b200.services.artifacts import LocalArtifactWriter, utc_now

PROVENANCE_KEYS = ("token_start", "token_end", "examples", "target_tokens", "document_aware", "documents_touched",
                   "document_min", "document_max")


def evaluate_checkpoint(run_dir: str | Path, selector: str) -> dict[str, Any]:
    run_dir = Path(run_dir)
    ck = restore_inference_checkpoint(run_dir, selector)
    spec = ck.spec
    ev = next((e for e in spec.evals if e.name == "validation"), None)
    if ev is None:
        raise ContractError("checkpoint eval requires [[evals]] name = 'validation'")
    manifest_path = spec.data.validation_manifest or spec.data.train_manifest
    if manifest_path is None:
        raise ContractError("checkpoint eval requires a prepared validation manifest")
    start = time.perf_counter()
    result = ck.trainer.evaluate(ev.num_batches)
    sec = time.perf_counter() - start
    if result["num_batches"] < ev.num_batches:
        raise ContractError(f"validation split ended before eval.num_batches={ev.num_batches} completed")
    row = {"schema_version": 1, "step": ck.record.step, "tokens_seen": ck.record.tokens_seen, "eval_name": ev.name,
           "loss_sum": result["loss_sum"], "token_count": int(result["token_count"]), "loss": result["loss"],
           "bpb": result.get("bpb"), "num_batches": result["num_batches"],
           **{k: result.get(k) for k in PROVENANCE_KEYS}}
    row = enrich_eval_metrics(row, eval_sec=sec)
    from research_b200.data.manifest import validate_dataset_manifest

    payload = {
        "schema_version": 1, "status": "completed", "created_at": utc_now(), "run_id": spec.run_id,
        "selector": selector, "checkpoint": ck.describe(), "eval": row,
        "data": {"manifest_path": Path(manifest_path).as_posix(),
                 "manifest_sha256": validate_dataset_manifest(manifest_path).manifest_sha256},
        "checkpoint_step": ck.record.step, "checkpoint_path": ck.record.checkpoint_path.as_posix(),
        "tokens_seen": ck.record.tokens_seen, "name": ev.name, "loss": row["loss"], "bpb": row["bpb"],
        "loss_sum": row["loss_sum"], "token_count": row["token_count"], "num_batches": row["num_batches"],
        "eval_sec": sec, "eval_tokens_per_sec": row["eval_tokens_per_sec"],
        "train_loss_at_checkpoint": ck.record.train_loss, "eval_loss_at_checkpoint": ck.record.eval_loss,
    }
    payload = normalize(payload)
    if ck.trainer.is_writer:
        path = LocalArtifactWriter(run_dir).write_checkpoint_eval(ck.record.step, payload)
        payload["artifact_path"] = path.relative_to(run_dir).as_posix()
    return payload


def checkpoint_eval_to_json(payload: Mapping[str, Any]) -> str:
    return json.dumps(normalize(payload), sort_keys=True, separators=(",", ":"))


def format_checkpoint_eval(payload: Mapping[str, Any]) -> str:
    ck, row = payload.get("checkpoint"), payload.get("eval")
    if not isinstance(ck, Mapping) or not isinstance(row, Mapping):
        raise ContractError("checkpoint eval payload needs checkpoint and eval objects")
    bpb = "" if row.get("bpb") is None else f" bpb={row['bpb']:.4f}"
    return (f"evaluated checkpoint step={ck['step']} path={ck['path']} loss={row['loss']}{bpb} "
            f"tokens={row['token_count']} batches={row['num_batches']}")
