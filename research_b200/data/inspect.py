"""``data inspect``: a read-only summary of a prepared-token manifest plus a paste-ready ``[data]`` TOML block
(reference: src/jaxtitan/data/inspect.py:21-162).

The JSON payload has the reference's sections - ``manifest``, ``source``, ``tokenizer``, ``tokens``, ``documents``,
``shards``, ``records``, ``data_config_toml`` - and, beside them, the flat manifest summary a run's ``manifest.json``
carries, per-shard sizes and the document length distribution.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any

import numpy as np

from research_b200.data.manifest import (PreparedDatasetManifest, dataset_manifest_summary,
                                         prepared_dataset_manifest_to_dict, validate_dataset_manifest)
from research_b200.data.pipeline import open_document_offsets
from research_b200.errors import ContractError


def record_count(tokens: int, seq_len: int) -> int:
    """Fixed windows of ``seq_len + 1`` tokens, ``seq_len`` apart, that fit in ``tokens``."""

    return max(0, (tokens - 1) // seq_len)


def data_config_snippet(manifest: PreparedDatasetManifest) -> str:
    """A ``[data]`` block for a training config that reads this dataset: ``document_buffer`` order when the dataset
    has document offsets, ``sequential`` otherwise."""

    lines = ["[data]", 'mode = "prepared"', f'train_manifest = "{manifest.manifest_path.as_posix()}"',
             f'tokenizer_id = "{manifest.tokenizer_id}"']
    if manifest.documents is None:
        lines.append('order = "sequential"')
    else:
        lines += ['order = "document_buffer"', "shuffle_seed = 123", "document_buffer_size = 8",
                  "document_refill_size = 8"]
    return "\n".join(lines)


def _read_raw(path: Path) -> dict[str, Any]:
    try:
        raw = json.loads(path.read_text(encoding="utf-8"))
    except OSError as exc:
        raise ContractError(f"failed to read prepared dataset manifest {path}: {exc}") from exc
    except json.JSONDecodeError as exc:
        raise ContractError(f"failed to parse prepared dataset manifest {path}: {exc}") from exc
    if not isinstance(raw, dict):
        raise ContractError(f"prepared dataset manifest must be a JSON object: {path}")
    return raw


def inspect_dataset(path: str | Path, *, tokenizer_id: str | None = None, verify_checksums: bool = False,
                    seq_len: int | None = None) -> dict[str, Any]:
    if seq_len is not None and seq_len <= 0:
        raise ContractError(f"data inspect --seq-len must be positive, got {seq_len}")
    manifest = validate_dataset_manifest(path, tokenizer_id=tokenizer_id, verify_checksums=verify_checksums)
    raw = _read_raw(manifest.manifest_path)
    source, tokenizer = raw.get("source"), raw.get("tokenizer")
    docs = manifest.documents
    report: dict[str, Any] = {
        "schema_version": 1,
        "manifest": prepared_dataset_manifest_to_dict(manifest),
        "source": source if isinstance(source, dict) else None,
        "tokenizer": tokenizer if isinstance(tokenizer, dict) else {"name": manifest.tokenizer_id},
        "tokens": {"total": manifest.num_tokens, "train": manifest.train_tokens, "val": manifest.val_tokens},
        "documents": {"count": None if docs is None else docs.count,
                      "offsets_path": None if docs is None else docs.path.as_posix(),
                      "offsets_sha256": None if docs is None else docs.sha256},
        "shards": {"count": manifest.shard_count, "bytes": sum(s.bytes for s in manifest.shards),
                   "checksums_present": all(s.sha256 is not None for s in manifest.shards),
                   "checksums_verified": bool(verify_checksums),
                   "files": [{"path": s.path.as_posix(), "tokens": s.tokens, "bytes": s.bytes}
                             for s in manifest.shards]},
        "records": None,
        "data_config_toml": data_config_snippet(manifest),
        **dataset_manifest_summary(manifest),
    }
    offsets = open_document_offsets(manifest)
    if offsets is not None:
        lengths = np.diff(np.asarray(offsets, dtype=np.int64))
        report["documents"]["lengths"] = {"min": int(lengths.min()), "max": int(lengths.max()),
                                          "mean": float(lengths.mean()), "median": float(np.median(lengths))}
    if seq_len is not None:
        report["records"] = {"seq_len": seq_len, "train": record_count(manifest.train_tokens, seq_len),
                             "val": record_count(manifest.val_tokens, seq_len),
                             # packed document rows carry seq_len + 1 tokens each and share none
                             "train_document_buffer_rows": manifest.train_tokens // (seq_len + 1)}
    return report


def _format_source(source: dict[str, Any]) -> str:
    if source.get("type") == "hf":
        return (f"type=hf dataset={source.get('dataset')} name={source.get('name')} split={source.get('split')} "
                f"text_column={source.get('text_column')}")
    if source:
        return (f"type={source.get('type')} files={source.get('resolved_file_count')} "
                f"bytes={source.get('resolved_total_bytes')} text_column={source.get('text_column')}")
    return "type=None dataset=None name=None split=None text_column=None"


def format_inspection(report: dict[str, Any]) -> str:
    tok, tokens, docs, shards = report["tokenizer"], report["tokens"], report["documents"], report["shards"]
    out = [f"manifest: {report['manifest_path']}",
           f"source: {_format_source(report['source'] or {})}",
           f"tokenizer: {tok.get('name')} append_eot={tok.get('append_eot')} eot={tok.get('eot_token')}",
           f"tokens: total={tokens['total']:,} train={tokens['train']:,} val={tokens['val']:,}",
           f"documents: count={docs['count']} offsets={docs['offsets_path']}",
           f"shards: count={shards['count']} bytes={shards['bytes']:,} checksums={shards['checksums_present']}"]
    if "lengths" in docs:
        ln = docs["lengths"]
        out.append(f"document lengths: min={ln['min']} median={ln['median']:.0f} mean={ln['mean']:.1f} max={ln['max']}")
    records = report["records"]
    if records is not None:
        out.append(f"records: seq_len={records['seq_len']} train={records['train']:,} val={records['val']:,}")
    out += ["", "training config:", report["data_config_toml"]]
    return "\n".join(out)


# the reference's names for the same operations (src/jaxtitan/data/inspect.py)
inspect_dataset_manifest = inspect_dataset
format_data_inspection = format_inspection


def data_inspection_to_dict(report: dict[str, Any]) -> dict[str, Any]:
    return dict(report)


def data_inspection_to_json(report: dict[str, Any]) -> str:
    return json.dumps(report, sort_keys=True, separators=(",", ":"))
