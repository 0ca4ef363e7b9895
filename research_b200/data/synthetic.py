"""Seed-generated prepared-token datasets of a named shape (no network, no tokenizer needed).

Writes a complete manifest-v1 directory: uint32 shards, ``document_offsets.u64``, ``token_bytes.bin`` and
``manifest.json``.  Document lengths are geometric with a given mean, clipped to a range, token ids uniform
below the EOS id, and every document ends with EOS - the shape the smoke and benchmark configs name.
The writer mirrors what the reference's offline prepare step emits (src/jaxtitan/data/prepare.py:221-273,
408-418, 490-552).
"""

from __future__ import annotations

import json
from hashlib import sha256
from pathlib import Path

import numpy as np

from research_b200.errors import ContractError


def geometric_document_lengths(rng: np.random.Generator, count: int, mean: float, low: int, high: int) -> np.ndarray:
    lengths = rng.geometric(1.0 / float(mean), size=count)
    return np.clip(lengths, low, high).astype(np.int64)


def write_prepared_dataset(out_dir: str | Path, *, tokens: np.ndarray, document_offsets: np.ndarray | None,
                           tokenizer_id: str, vocab_size: int, eot_id: int | None, val_fraction: float = 0.05,
                           shard_tokens: int = 1 << 24, dataset_id: str = "synthetic", overwrite: bool = False) -> Path:
    """Write ``tokens`` (uint32) as a prepared dataset; the val split is the tail, cut at a document boundary."""

    out = Path(out_dir)
    if out.exists() and any(out.iterdir()) and not overwrite:
        raise ContractError(f"prepared dataset directory already exists: {out}")
    out.mkdir(parents=True, exist_ok=True)
    tokens = np.ascontiguousarray(tokens, dtype="<u4")
    n = int(tokens.shape[0])
    if n <= 1:
        raise ContractError("a prepared dataset needs at least two tokens")
    shards = []
    start = 0
    idx = 0
    while start < n:
        end = min(start + shard_tokens, n)
        name = f"tokens-{idx:05d}.bin"
        chunk = tokens[start:end]
        (out / name).write_bytes(chunk.tobytes())
        shards.append({"path": name, "start": start, "end": end, "tokens": end - start, "bytes": (end - start) * 4,
                       "sha256": sha256(chunk.tobytes()).hexdigest()})
        start = end
        idx += 1
    val_start = n - int(round(n * val_fraction))
    if document_offsets is not None:
        document_offsets = np.ascontiguousarray(document_offsets, dtype="<u8")
        pos = int(np.searchsorted(document_offsets, val_start, side="left"))
        val_start = int(document_offsets[min(pos, len(document_offsets) - 1)])
    val_start = min(max(val_start, 1), n)
    token_bytes = np.full((vocab_size,), 3, dtype="<u2")
    if eot_id is not None and 0 <= eot_id < vocab_size:
        token_bytes[eot_id] = 0
    (out / "token_bytes.bin").write_bytes(token_bytes.tobytes())
    files = {"token_bytes": {"path": "token_bytes.bin", "dtype": "uint16", "bytes": int(token_bytes.nbytes),
                             "sha256": sha256(token_bytes.tobytes()).hexdigest()}}
    manifest = {
        "schema_version": 1,
        "kind": "training_tokens",
        "dataset_id": dataset_id,
        "dtype": "uint32",
        "tokenizer": {"name": tokenizer_id, "vocab_size": int(vocab_size), "eot_id": eot_id},
        "num_tokens": n,
        "shards": shards,
        "splits": {"train": {"start": 0, "end": val_start, "tokens": val_start},
                   "val": {"start": val_start, "end": n, "tokens": n - val_start}},
        "files": files,
    }
    if document_offsets is not None:
        raw = document_offsets.tobytes()
        (out / "document_offsets.u64").write_bytes(raw)
        files["document_offsets"] = {"path": "document_offsets.u64", "dtype": "uint64", "bytes": len(raw),
                                     "sha256": sha256(raw).hexdigest()}
        manifest["documents"] = {"count": int(len(document_offsets) - 1)}
    path = out / "manifest.json"
    path.write_text(json.dumps(manifest, sort_keys=True, indent=1), encoding="utf-8")
    return path


def generate_synthetic_dataset(out_dir: str | Path, *, seed: int, num_documents: int, mean_length: float,
                               min_length: int, max_length: int, vocab_size: int, eos_id: int,
                               val_fraction: float = 0.05, tokenizer_id: str = "synthetic-uniform",
                               shard_tokens: int = 1 << 24, overwrite: bool = False) -> Path:
    """Documents ~ geometric(mean) clipped to [min, max]; ids uniform in [0, eos_id); EOS closes each document."""

    rng = np.random.default_rng(int(seed))
    lengths = geometric_document_lengths(rng, num_documents, mean_length, min_length, max_length)
    offsets = np.zeros(num_documents + 1, dtype=np.uint64)
    offsets[1:] = np.cumsum(lengths)
    total = int(offsets[-1])
    tokens = rng.integers(0, eos_id, size=total, dtype=np.uint32)
    tokens[(offsets[1:] - 1).astype(np.int64)] = eos_id
    return write_prepared_dataset(out_dir, tokens=tokens, document_offsets=offsets, tokenizer_id=tokenizer_id,
                                  vocab_size=vocab_size, eot_id=eos_id, val_fraction=val_fraction,
                                  shard_tokens=shard_tokens, dataset_id=f"synthetic-seed{seed}", overwrite=overwrite)
