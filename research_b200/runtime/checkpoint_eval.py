"""``eval checkpoint``: validation loss of a retained checkpoint -> ``evals/checkpoints/<step>.json``
(reference: src/jaxtitan/runtime/checkpoint_eval.py:24-96)."""

from __future__ import annotations

import time
from pathlib import Path
from typing import Any

from research_b200.errors import ContractError
from research_b200.infer.checkpoint import restore_inference_checkpoint
from research_b200.services.artifacts import LocalArtifactWriter, utc_now


def evaluate_checkpoint(run_dir: str | Path, selector: str) -> dict[str, Any]:
    run_dir = Path(run_dir)
    ck = restore_inference_checkpoint(run_dir, selector)
    spec = ck.spec
    if not spec.evals:
        raise ContractError("the run config has no [[evals]] section; nothing to evaluate")
    ev = spec.evals[0]
    start = time.perf_counter()
    result = ck.trainer.evaluate(ev.num_batches)
    sec = time.perf_counter() - start
    payload = {
        "schema_version": 1, "created_at": utc_now(), "run_id": spec.run_id, "selector": selector,
        "checkpoint_step": ck.record.step, "checkpoint_path": ck.record.checkpoint_path.as_posix(),
        "tokens_seen": ck.record.tokens_seen, "name": ev.name, "loss": result["loss"], "bpb": result.get("bpb"), "loss_sum": result["loss_sum"],
        "token_count": int(result["token_count"]), "num_batches": result["num_batches"], "eval_sec": sec,
        "eval_tokens_per_sec": None if sec <= 0 else result["token_count"] / sec,
        "train_loss_at_checkpoint": ck.record.train_loss, "eval_loss_at_checkpoint": ck.record.eval_loss,
    }
    if ck.trainer.is_writer:
        path = LocalArtifactWriter(run_dir).write_checkpoint_eval(ck.record.step, payload)
        payload["artifact_path"] = path.relative_to(run_dir).as_posix()
    return payload
