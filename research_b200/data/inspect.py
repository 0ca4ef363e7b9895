"""``data inspect``: manifest summary plus a paste-ready ``[data]`` TOML block
(reference: src/jaxtitan/data/inspect.py:21-128)."""

from __future__ import annotations

from pathlib import Path
from typing import Any

import numpy as np

from research_b200.data.manifest import dataset_manifest_summary, validate_dataset_manifest
from research_b200.data.pipeline import open_document_offsets


def inspect_dataset(path: str | Path, *, tokenizer_id: str | None = None, verify_checksums: bool = False,
                    seq_len: int | None = None) -> dict[str, Any]:
    manifest = validate_dataset_manifest(path, tokenizer_id=tokenizer_id, verify_checksums=verify_checksums)
    report: dict[str, Any] = {"schema_version": 1, **dataset_manifest_summary(manifest),
                              "checksums_verified": bool(verify_checksums),
                              "shards": [{"path": s.path.as_posix(), "tokens": s.tokens, "bytes": s.bytes}
                                         for s in manifest.shards]}
    offsets = open_document_offsets(manifest)
    if offsets is not None:
        lengths = np.diff(np.asarray(offsets, dtype=np.int64))
        report["document_lengths"] = {"min": int(lengths.min()), "max": int(lengths.max()),
                                      "mean": float(lengths.mean()), "median": float(np.median(lengths))}
    if seq_len is not None:
        report["seq_len"] = seq_len
        report["train_records"] = max(0, (manifest.train_tokens - 1) // seq_len)
        report["val_records"] = max(0, (manifest.val_tokens - 1) // seq_len)
        report["train_document_buffer_records"] = manifest.train_tokens // (seq_len + 1)
    order = "document_buffer" if manifest.documents is not None else "sequential"
    lines = ["[data]", 'mode = "prepared"', f'train_manifest = "{manifest.manifest_path.as_posix()}"',
             f'tokenizer_id = "{manifest.tokenizer_id}"', f'order = "{order}"']
    if order == "document_buffer":
        lines += ["shuffle_seed = 0", "document_buffer_size = 128", "document_refill_size = 128"]
    report["data_toml"] = "\n".join(lines) + "\n"
    return report


def format_inspection(report: dict[str, Any]) -> str:
    out = [f"manifest: {report['manifest_path']}", f"tokenizer: {report['tokenizer_id']}",
           f"tokens: total {report['total_tokens']:,} | train {report['train_tokens']:,} | val {report['val_tokens']:,}",
           f"shards: {report['shard_count']}", f"document aware: {report['document_aware']} "
           f"(documents: {report['document_count']})"]
    if "seq_len" in report:
        out.append(f"records at seq_len {report['seq_len']}: train {report['train_records']:,} | val {report['val_records']:,}")
    out += ["", report["data_toml"].rstrip()]
    return "\n".join(out)
