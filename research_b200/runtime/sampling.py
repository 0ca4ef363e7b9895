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


def parse_prompt_ids(value, vocab_size: int | None = None) -> list[int]:
    """Strict parsing of a comma-separated id list, or validation of a sequence of ints: base-10 integers only, no
    blanks, non-negative and, when ``vocab_size`` is given, inside the vocabulary
    (reference: src/jaxtitan/runtime/sampling.py:82-136)."""

    if isinstance(value, str):
        if not value.strip():
            raise ContractError("--prompt-ids must be a non-empty comma-separated list of token ids")
        ids = []
        for part in value.split(","):
            token = part.strip()
            if not token or not token.isdigit():
                raise ContractError(f"--prompt-ids contains an invalid token id {part!r}")
            ids.append(int(token))
    else:
        ids = list(value)
        if not ids:
            raise ContractError("prompt_ids must contain at least one token id")
        for token in ids:
            if isinstance(token, bool) or not isinstance(token, int):
                raise ContractError("prompt_ids must be integers")
            if token < 0:
                raise ContractError(f"prompt_ids must be non-negative, got {token}")
    if vocab_size is not None:
        for token in ids:
            if token >= vocab_size:
                raise ContractError(f"prompt token id {token} is outside the vocabulary of size {vocab_size}")
    return ids


def sample_checkpoint(run_dir: str | Path, selector: str, *, prompt_ids, max_new_tokens: int,
                      temperature: float = 1.0, top_k: int | None = None) -> dict[str, Any]:
    run_dir = Path(run_dir)
    prompt = parse_prompt_ids(prompt_ids)                    # a malformed prompt fails before anything is restored
    ck = restore_inference_checkpoint(run_dir, selector)
    spec = ck.spec
    parse_prompt_ids(prompt, spec.model.vocab_size)
    if top_k is not None and top_k > spec.model.vocab_size:
        raise ContractError(f"generation.top_k={top_k} exceeds vocab size {spec.model.vocab_size}")
    page_size = spec.generation.page_size if spec.generation is not None else 128
    result = generate_tokens(ck.model, torch.tensor([prompt], dtype=torch.int64), max_new_tokens=max_new_tokens,
                             temperature=temperature, top_k=top_k, seed=ck.trainer.rng.sample & 0x7FFFFFFF,
                             page_size=page_size)
    m = spec.model
    row = {
        "schema_version": 1, "status": "completed", "created_at": utc_now(), "run_id": spec.run_id,
        "selector": selector, "checkpoint": ck.describe(selector),
        "model": {"name": m.name, "variant": m.variant, "vocab_size": m.vocab_size, "max_seq_len": m.max_seq_len},
        "sampling": {"max_new_tokens": max_new_tokens, "temperature": temperature, "top_k": top_k, "top_p": None},
        "checkpoint_step": ck.record.step, "checkpoint_path": ck.record.checkpoint_path.as_posix(),
        "prompt_ids": result.prompt_ids[0], "generated_ids": result.generated_ids[0], "full_ids": result.full_ids[0],
        "logprobs": result.logprobs[0], "max_new_tokens": max_new_tokens, "temperature": temperature, "top_k": top_k,
        "sampler": "greedy" if top_k == 1 else "categorical",
    }
    if ck.trainer.is_writer:
        path = LocalArtifactWriter(run_dir).append_checkpoint_sample(ck.record.step, row)
        row["artifact_path"] = path.relative_to(run_dir).as_posix()
    return row


def checkpoint_sample_to_json(payload) -> str:
    import json

    return json.dumps(payload, sort_keys=True, separators=(",", ":"))


def format_checkpoint_sample(payload) -> str:
    ck, sampling = payload.get("checkpoint"), payload.get("sampling")
    if not isinstance(ck, dict) or not isinstance(sampling, dict):
        raise ContractError("checkpoint sample payload needs checkpoint and sampling objects")
    return (f"sampled checkpoint step={ck['step']} path={ck['path']} generated={sampling['max_new_tokens']} "
            f"top_k={sampling['top_k']} ids={payload.get('generated_ids')}")
