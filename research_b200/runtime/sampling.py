"""``sample checkpoint``: token sampling from a retained checkpoint -> ``samples/checkpoints/<step>.jsonl`` with
prompt / generated / full ids and log-probabilities (reference: src/jaxtitan/runtime/sampling.py:20-100)."""

from __future__ import annotations

from pathlib import Path
from typing import Any

import torch

from research_b200.errors import ContractError
from research_b200.infer.checkpoint import restore_inference_checkpoint
from research_b200.infer.generation import generate_tokens
from research_b200.services.artifacts import LocalArtifactWriter, utc_now


def parse_prompt_ids(text: str, vocab_size: int) -> list[int]:
    """Strict parsing of a comma-separated id list: integers only, no blanks, inside the vocabulary."""

    if not isinstance(text, str) or not text.strip():
        raise ContractError("--prompt-ids must be a non-empty comma-separated list of token ids")
    ids = []
    for part in text.split(","):
        token = part.strip()
        if not token or not (token.isdigit()):
            raise ContractError(f"--prompt-ids contains an invalid token id {part!r}")
        value = int(token)
        if value >= vocab_size:
            raise ContractError(f"prompt token id {value} is outside the vocabulary of size {vocab_size}")
        ids.append(value)
    return ids


def sample_checkpoint(run_dir: str | Path, selector: str, *, prompt_ids: str, max_new_tokens: int,
                      temperature: float = 1.0, top_k: int | None = None) -> dict[str, Any]:
    run_dir = Path(run_dir)
    ck = restore_inference_checkpoint(run_dir, selector)
    spec = ck.spec
    prompt = parse_prompt_ids(prompt_ids, spec.model.vocab_size)
    page_size = spec.generation.page_size if spec.generation is not None else 128
    result = generate_tokens(ck.model, torch.tensor([prompt], dtype=torch.int64), max_new_tokens=max_new_tokens,
                             temperature=temperature, top_k=top_k, seed=ck.trainer.rng.sample & 0x7FFFFFFF,
                             page_size=page_size)
    row = {
        "schema_version": 1, "created_at": utc_now(), "run_id": spec.run_id, "selector": selector,
        "checkpoint_step": ck.record.step, "checkpoint_path": ck.record.checkpoint_path.as_posix(),
        "prompt_ids": result.prompt_ids[0], "generated_ids": result.generated_ids[0], "full_ids": result.full_ids[0],
        "logprobs": result.logprobs[0], "max_new_tokens": max_new_tokens, "temperature": temperature, "top_k": top_k,
        "sampler": "greedy" if top_k == 1 else "categorical",
    }
    if ck.trainer.is_writer:
        path = LocalArtifactWriter(run_dir).append_checkpoint_sample(ck.record.step, row)
        row["artifact_path"] = path.relative_to(run_dir).as_posix()
    return row
