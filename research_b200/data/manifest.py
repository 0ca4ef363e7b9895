"""Prepared-token dataset manifest (schema v1): parsing, validation against the files on disk, hashing.

Same on-disk contract as the reference validator (src/jaxtitan/data/manifest.py:98-361): kind
``training_tokens``, dtype ``uint32``, contiguous little-endian shards, non-overlapping train/val
splits, ``files.token_bytes``, optional ``documents.count`` + ``files.document_offsets`` (uint64,
count + 1 entries, first 0, last ``num_tokens``, strictly increasing), relative paths only, and
``manifest_sha256`` = sha256 of the manifest file bytes.
"""

from __future__ import annotations

import json
from collections.abc import Mapping
from dataclasses import dataclass
from hashlib import sha256
from pathlib import Path
from typing import Any

import numpy as np

from research_b200.config.canonical import canonical_json, normalize
from research_b200.errors import ContractError

UINT32_BYTES = 4
UINT64_BYTES = 8


@dataclass(frozen=True, slots=True)
class TokenShard:
    path: Path
    start: int
    end: int
    tokens: int
    bytes: int
    sha256: str | None = None


@dataclass(frozen=True, slots=True)
class TokenSplit:
    start: int
    end: int
    tokens: int


@dataclass(frozen=True, slots=True)
class DocumentTable:
    path: Path
    dtype: str
    count: int
    bytes: int
    sha256: str | None = None


@dataclass(frozen=True, slots=True)
class PreparedDatasetManifest:
    manifest_path: Path
    schema_version: int
    kind: str
    dtype: str
    tokenizer_id: str
    num_tokens: int
    train: TokenSplit
    val: TokenSplit
    shards: tuple[TokenShard, ...]
    token_bytes_path: Path
    token_bytes_sha256: str | None
    documents: DocumentTable | None
    manifest_sha256: str

    @property
    def shard_count(self) -> int:
        return len(self.shards)

    @property
    def train_tokens(self) -> int:
        return self.train.tokens

    @property
    def val_tokens(self) -> int:
        return self.val.tokens

    @property
    def data_dir(self) -> Path:
        return self.manifest_path.parent


def file_sha256(path: Path) -> str:
    digest = sha256()
    with path.open("rb") as handle:
        while True:
            chunk = handle.read(1 << 20)
            if not chunk:
                break
            digest.update(chunk)
    return digest.hexdigest()


def dataset_manifest_sha256(path: str | Path) -> str:
    return file_sha256(Path(path))


def _fail(message: str) -> None:
    raise ContractError(message)


def _obj(value: Any, label: str) -> Mapping[str, Any]:
    if not isinstance(value, Mapping):
        _fail(f"prepared dataset manifest {label} must be an object")
    return value


def _req_str(raw: Mapping[str, Any], key: str, label: str) -> str:
    value = raw.get(key)
    if not isinstance(value, str) or not value:
        _fail(f"prepared dataset manifest {label}.{key} must be a non-empty string")
    return value


def _req_int(raw: Mapping[str, Any], key: str, label: str) -> int:
    value = raw.get(key)
    if not isinstance(value, int) or isinstance(value, bool):
        _fail(f"prepared dataset manifest {label}.{key} must be an integer")
    return value


def _inside(data_dir: Path, rel_value: str, label: str) -> Path:
    rel = Path(rel_value)
    if rel.is_absolute():
        _fail(f"prepared dataset {label} path must be relative, got {rel_value!r}")
    full = data_dir / rel
    if not full.resolve().is_relative_to(data_dir.resolve()):
        _fail(f"prepared dataset {label} path must stay inside the manifest directory, got {rel_value!r}")
    if not full.is_file():
        _fail(f"prepared dataset {label} file does not exist: {full}")
    return full


def _optional_sha(raw: Mapping[str, Any], label: str) -> str | None:
    value = raw.get("sha256")
    if value is not None and (not isinstance(value, str) or not value):
        _fail(f"{label}.sha256 must be non-empty")
    return value


def _read_json(path: Path) -> Mapping[str, Any]:
    if not path.is_file():
        _fail(f"prepared dataset manifest does not exist: {path}")
    try:
        raw = json.loads(path.read_text(encoding="utf-8"))
    except OSError as exc:
        raise ContractError(f"failed to read prepared dataset manifest {path}: {exc}") from exc
    except json.JSONDecodeError as exc:
        raise ContractError(f"failed to parse prepared dataset manifest {path}: {exc}") from exc
    if not isinstance(raw, Mapping):
        _fail(f"prepared dataset manifest must be a JSON object: {path}")
    return raw


def _shards(data_dir: Path, raw_shards: list[Any], verify: bool) -> tuple[TokenShard, ...]:
    out = []
    cursor = 0
    for idx, item in enumerate(raw_shards):
        label = f"shards[{idx}]"
        shard = _obj(item, label)
        rel = _req_str(shard, "path", label)
        full = _inside(data_dir, rel, label)
        start, end = _req_int(shard, "start", label), _req_int(shard, "end", label)
        tokens, nbytes = _req_int(shard, "tokens", label), _req_int(shard, "bytes", label)
        if start != cursor or end < start or tokens != end - start:
            _fail(f"prepared dataset shards must be contiguous and correctly bounded; bad shard={idx}")
        size = full.stat().st_size
        if size % UINT32_BYTES:
            _fail(f"prepared dataset shard size is not divisible by uint32 size: {full}")
        if size // UINT32_BYTES != tokens:
            _fail(f"prepared dataset shard {rel} tokens={tokens} does not match file length={size // UINT32_BYTES}")
        if nbytes != size:
            _fail(f"prepared dataset shard {rel} bytes={nbytes} does not match file bytes={size}")
        sha = _optional_sha(shard, label)
        if verify and sha and file_sha256(full) != sha:
            _fail(f"prepared dataset checksum mismatch for {full}")
        out.append(TokenShard(Path(rel), start, end, tokens, nbytes, sha))
        cursor = end
    return tuple(out)


def _split(splits: Mapping[str, Any], name: str, num_tokens: int) -> TokenSplit:
    label = f"splits.{name}"
    raw = _obj(splits.get(name), label)
    start, end, tokens = _req_int(raw, "start", label), _req_int(raw, "end", label), _req_int(raw, "tokens", label)
    if not 0 <= start <= end <= num_tokens:
        _fail(f"prepared dataset split {name} has invalid bounds start={start}, end={end}, num_tokens={num_tokens}")
    if tokens != end - start:
        _fail(f"prepared dataset split {name} tokens={tokens} does not equal end-start={end - start}")
    return TokenSplit(start, end, tokens)


def _documents(data_dir: Path, raw: Mapping[str, Any], files: Mapping[str, Any], num_tokens: int,
               verify: bool) -> DocumentTable | None:
    has_docs = raw.get("documents") is not None
    has_offsets = files.get("document_offsets") is not None
    if not has_docs and not has_offsets:
        return None
    if has_docs != has_offsets:
        _fail("prepared dataset documents metadata requires files.document_offsets")
    count = _req_int(_obj(raw.get("documents"), "documents"), "count", "documents")
    if count <= 0:
        _fail(f"prepared dataset documents.count must be positive, got {count}")
    info = _obj(files.get("document_offsets"), "files.document_offsets")
    dtype = _req_str(info, "dtype", "files.document_offsets")
    if dtype != "uint64":
        _fail(f"prepared dataset document_offsets dtype must be uint64, got {dtype!r}")
    rel = _req_str(info, "path", "files.document_offsets")
    full = _inside(data_dir, rel, "document_offsets")
    declared = _req_int(info, "bytes", "files.document_offsets")
    actual = full.stat().st_size
    if declared != actual:
        _fail(f"prepared dataset document_offsets bytes={declared} does not match file bytes={actual}")
    if actual != (count + 1) * UINT64_BYTES:
        _fail(f"prepared dataset document_offsets file bytes={actual} does not match documents.count={count}")
    offsets = np.memmap(full, dtype="<u8", mode="r")
    if int(offsets[0]) != 0:
        _fail("prepared dataset document_offsets first offset must be 0")
    if int(offsets[-1]) != num_tokens:
        _fail(f"prepared dataset document_offsets final offset={int(offsets[-1])} must equal num_tokens={num_tokens}")
    if not bool(np.all(offsets[1:] > offsets[:-1])):
        _fail("prepared dataset document_offsets must be strictly increasing")
    sha = _optional_sha(info, "files.document_offsets")
    if verify and sha and file_sha256(full) != sha:
        _fail(f"prepared dataset document_offsets checksum mismatch for {full}")
    return DocumentTable(Path(rel), "uint64", count, declared, sha)


def validate_dataset_manifest(path: str | Path, *, tokenizer_id: str | None = None,
                              verify_checksums: bool = False) -> PreparedDatasetManifest:
    """Validate a prepared-token manifest and the files it names; returns the parsed manifest."""

    manifest_path = Path(path)
    raw = _read_json(manifest_path)
    data_dir = manifest_path.parent
    schema_version = _req_int(raw, "schema_version", "manifest")
    if schema_version <= 0:
        _fail(f"prepared dataset manifest schema_version must be positive, got {schema_version}")
    if raw.get("kind") != "training_tokens":
        _fail(f"prepared dataset manifest kind must be training_tokens, got {raw.get('kind')!r}")
    if raw.get("dtype") != "uint32":
        _fail(f"prepared dataset manifest dtype must be uint32, got {raw.get('dtype')!r}")
    tok = _obj(raw.get("tokenizer"), "tokenizer").get("name")
    if not isinstance(tok, str) or not tok:
        _fail("prepared dataset manifest tokenizer.name is required")
    if tokenizer_id is not None and tok != tokenizer_id:
        _fail(f"prepared dataset tokenizer {tok!r} does not match config tokenizer {tokenizer_id!r}")
    raw_shards = raw.get("shards")
    if not isinstance(raw_shards, list) or not raw_shards:
        _fail("prepared dataset manifest must contain non-empty shards")
    shards = _shards(data_dir, raw_shards, verify_checksums)
    num_tokens = _req_int(raw, "num_tokens", "manifest")
    shard_total = sum(s.tokens for s in shards)
    if num_tokens != shard_total:
        _fail(f"prepared dataset num_tokens={num_tokens} does not match shard total={shard_total}")
    splits = _obj(raw.get("splits"), "splits")
    train, val = _split(splits, "train", num_tokens), _split(splits, "val", num_tokens)
    if train.start < val.end and val.start < train.end:
        _fail(f"prepared dataset train/val splits overlap: train={train}, val={val}")
    files = _obj(raw.get("files"), "files")
    tb = _obj(files.get("token_bytes"), "files.token_bytes")
    tb_rel = _req_str(tb, "path", "files.token_bytes")
    tb_full = _inside(data_dir, tb_rel, "token_bytes")
    tb_sha = _optional_sha(tb, "files.token_bytes")
    if verify_checksums and tb_sha and file_sha256(tb_full) != tb_sha:
        _fail(f"prepared dataset token_bytes checksum mismatch for {tb_full}")
    documents = _documents(data_dir, raw, files, num_tokens, verify_checksums)
    return PreparedDatasetManifest(
        manifest_path=manifest_path, schema_version=schema_version, kind="training_tokens", dtype="uint32",
        tokenizer_id=tok, num_tokens=num_tokens, train=train, val=val, shards=shards,
        token_bytes_path=Path(tb_rel), token_bytes_sha256=tb_sha, documents=documents,
        manifest_sha256=dataset_manifest_sha256(manifest_path),
    )


load_dataset_manifest = validate_dataset_manifest


def dataset_manifest_summary(manifest: PreparedDatasetManifest) -> dict[str, Any]:
    """The ``data`` section of a run's ``manifest.json``."""

    docs = manifest.documents
    return {
        "manifest_path": manifest.manifest_path.as_posix(),
        "manifest_sha256": manifest.manifest_sha256,
        "tokenizer_id": manifest.tokenizer_id,
        "total_tokens": manifest.num_tokens,
        "train_tokens": manifest.train_tokens,
        "val_tokens": manifest.val_tokens,
        "shard_count": manifest.shard_count,
        "token_bytes_path": manifest.token_bytes_path.as_posix(),
        "document_aware": docs is not None,
        "document_count": None if docs is None else docs.count,
        "document_offsets_path": None if docs is None else docs.path.as_posix(),
        "document_offsets_sha256": None if docs is None else docs.sha256,
    }


def prepared_dataset_manifest_to_dict(manifest: PreparedDatasetManifest) -> dict[str, Any]:
    return normalize(manifest)


def prepared_dataset_manifest_to_json(manifest: PreparedDatasetManifest) -> str:
    return canonical_json(manifest)
