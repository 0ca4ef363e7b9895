"""Offline tokenisation: raw text -> uint32 shards + ``token_bytes.bin`` + ``document_offsets.u64`` + manifest.

Same prepare-TOML contract as the reference (src/jaxtitan/data/prepare.py:31-127, 724-759): sections ``[source]``
(type hf | parquet | jsonl | text), ``[tokenizer]`` (name, append_eot), ``[output]`` (path, max_tokens,
val_fraction, shard_tokens) and ``[tokenization]`` (workers, batch_docs, queue_batches); texts are tokenised in a
process pool in batches of documents, EOT is appended, the stream is cut at ``max_tokens`` and written through a
shard writer that keeps a running sha256 (prepare.py:163-275, 490-609).

Tokenizers: ``tiktoken`` encodings by name when the package (and its vocabulary files) are available offline, the
built-in ``byte-level`` tokenizer (256 byte ids + EOT) otherwise - enough to prepare real text without a network.
"""

from __future__ import annotations

import json
import shutil
import tomllib
from concurrent.futures import ProcessPoolExecutor
from dataclasses import dataclass, field
from hashlib import sha256
from pathlib import Path
from typing import Any, Iterable, Iterator, Mapping

import numpy as np

from research_b200.errors import ConfigError, ContractError

SOURCE_TYPES = ("hf", "jsonl", "parquet", "text")


@dataclass(frozen=True)
class PrepareSourceConfig:
    type: str
    dataset: str | None = None
    split: str | None = None
    paths: tuple[str, ...] = ()
    name: str | None = None
    data_dir: str | None = None
    text_column: str = "text"
    streaming: bool = True

    def __post_init__(self) -> None:
        if self.type not in SOURCE_TYPES:
            supported = "', '".join(sorted(SOURCE_TYPES))
            raise ConfigError(f"source.type must be one of '{supported}', got {self.type!r}")
        object.__setattr__(self, "paths", tuple(self.paths))
        if self.type == "hf" and not self.dataset:
            raise ConfigError("source.dataset must be a non-empty string")
        if self.type == "hf" and not self.split:
            raise ConfigError("source.split must be a non-empty string")
        if self.type != "hf" and not self.paths:
            raise ConfigError("source.paths must be a non-empty list of paths")
        if any(not isinstance(p, str) or not p for p in self.paths):
            raise ConfigError("source.paths must contain non-empty strings")
        if not self.text_column:
            raise ConfigError("source.text_column must be a non-empty string")
        if not isinstance(self.streaming, bool):
            raise ConfigError("source.streaming must be a boolean")


@dataclass(frozen=True)
class PrepareTokenizerConfig:
    name: str
    append_eot: bool = True

    def __post_init__(self) -> None:
        if not self.name:
            raise ConfigError("tokenizer.name must be a non-empty string")
        if not isinstance(self.append_eot, bool):
            raise ConfigError("tokenizer.append_eot must be a boolean")


@dataclass(frozen=True)
class PrepareOutputConfig:
    path: Path
    max_tokens: int
    val_fraction: float = 0.001
    shard_tokens: int = 128_000_000
    dtype: str = "uint32"

    def __post_init__(self) -> None:
        object.__setattr__(self, "path", Path(self.path))
        if self.dtype != "uint32":
            raise ConfigError(f"output.dtype must be 'uint32', got {self.dtype!r}")
        for name in ("max_tokens", "shard_tokens"):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"output.{name} must be a positive integer")
        if not isinstance(self.val_fraction, (int, float)) or isinstance(self.val_fraction, bool):
            raise ConfigError("output.val_fraction must be numeric")
        if not 0.0 < float(self.val_fraction) < 1.0:
            raise ConfigError(f"output.val_fraction must be between 0 and 1, got {self.val_fraction}")


@dataclass(frozen=True)
class PrepareTokenizationConfig:
    workers: int | str = "auto"
    batch_docs: int = 256
    queue_batches: int = 8

    def __post_init__(self) -> None:
        if self.workers != "auto" and (not isinstance(self.workers, int) or isinstance(self.workers, bool)
                                       or self.workers <= 0):
            raise ConfigError("tokenization.workers must be 'auto' or a positive integer")
        for name in ("batch_docs", "queue_batches"):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"tokenization.{name} must be a positive integer")


@dataclass(frozen=True)
class PrepareConfig:
    source: PrepareSourceConfig
    tokenizer: PrepareTokenizerConfig
    output: PrepareOutputConfig
    tokenization: PrepareTokenizationConfig = field(default_factory=PrepareTokenizationConfig)


def _table(raw: Mapping[str, Any], key: str, required: bool) -> Mapping[str, Any]:
    if key not in raw:
        if required:
            raise ConfigError(f"missing required [{key}] section")
        return {}
    if not isinstance(raw[key], Mapping):
        raise ConfigError(f"[{key}] must be a TOML table")
    return raw[key]


TOKEN_BYTES_FILENAME = "token_bytes.bin"
DOCUMENT_OFFSETS_FILENAME = "document_offsets.u64"


def load_prepare_config(path: str | Path) -> PrepareConfig:
    p = Path(path)
    try:
        raw = tomllib.loads(p.read_text())
    except OSError as exc:
        raise ConfigError(f"failed to read config {p}: {exc}") from exc
    except tomllib.TOMLDecodeError as exc:
        raise ConfigError(f"failed to parse config {p}: {exc}") from exc
    return prepare_config_from_mapping(raw)


def prepare_config_from_mapping(raw: Mapping[str, Any]) -> PrepareConfig:
    """The ``[source] / [tokenizer] / [output] / [tokenization]`` tables of a prepare config as a :class:`PrepareConfig`."""

    src, tok, out = _table(raw, "source", True), _table(raw, "tokenizer", True), _table(raw, "output", True)
    tz = _table(raw, "tokenization", False)
    for section, key, table in (("source", "type", src), ("tokenizer", "name", tok), ("output", "path", out)):
        if not isinstance(table.get(key), str) or not table.get(key):
            raise ConfigError(f"{section}.{key} must be a non-empty string")
    if not isinstance(out.get("max_tokens"), int) or isinstance(out.get("max_tokens"), bool):
        raise ConfigError("output.max_tokens must be an integer")
    paths = src.get("paths", ())
    if not isinstance(paths, (list, tuple)):
        raise ConfigError("source.paths must be a list of strings")
    return PrepareConfig(
        source=PrepareSourceConfig(type=src["type"], dataset=src.get("dataset"), split=src.get("split"),
                                   paths=tuple(paths), name=src.get("name"), data_dir=src.get("data_dir"),
                                   text_column=src.get("text_column") or "text", streaming=src.get("streaming", True)),
        tokenizer=PrepareTokenizerConfig(name=tok["name"], append_eot=tok.get("append_eot", True)),
        output=PrepareOutputConfig(path=Path(out["path"]), max_tokens=out["max_tokens"],
                                   val_fraction=float(out.get("val_fraction", 0.001)),
                                   shard_tokens=out.get("shard_tokens", 128_000_000), dtype=out.get("dtype") or "uint32"),
        tokenization=PrepareTokenizationConfig(workers=tz.get("workers", "auto"), batch_docs=tz.get("batch_docs", 256),
                                               queue_batches=tz.get("queue_batches", 8)),
    )


# ---- tokenizers ----------------------------------------------------------------------------------------
class ByteLevelTokenizer:
    """UTF-8 bytes as ids 0..255, EOT = 256."""

    name = "byte-level"
    vocab_size = 257
    eot_id = 256

    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))

    def token_byte_lengths(self) -> np.ndarray:
        out = np.ones(self.vocab_size, dtype=np.uint16)
        out[self.eot_id] = 0
        return out


class TiktokenTokenizer:
    def __init__(self, name: str):
        import tiktoken

        self.name = name
        self.enc = tiktoken.get_encoding(name)
        self.vocab_size = self.enc.n_vocab
        self.eot_id = self.enc.eot_token

    def encode(self, text: str) -> list[int]:
        return self.enc.encode_ordinary(text)

    def token_byte_lengths(self) -> np.ndarray:
        out = np.zeros(self.vocab_size, dtype=np.uint16)
        for i in range(self.vocab_size):
            try:
                out[i] = len(self.enc.decode_single_token_bytes(i))
            except Exception:
                out[i] = 0
        out[self.eot_id] = 0
        return out


def load_tokenizer(name: str):
    if name == "byte-level":
        return ByteLevelTokenizer()
    try:
        return TiktokenTokenizer(name)
    except Exception as exc:
        raise ContractError(f"tokenizer {name!r} is not available offline ({type(exc).__name__}: {exc}); "
                            "use tokenizer.name = \"byte-level\"") from exc


# ---- sources ---------------------------------------------------------------------------------------------
def resolve_source_files(paths: Iterable[str], base: Path) -> tuple[Path, ...]:
    """``source.paths`` entries as files: ``~`` expanded, relative to the config's folder, shell patterns expanded in
    sorted order (reference: src/jaxtitan/data/prepare.py:679-697)."""

    import glob
    import os

    files: list[Path] = []
    for raw_path in paths:
        expanded = os.path.expanduser(raw_path)
        if not os.path.isabs(expanded):
            expanded = os.path.join(str(base), expanded)
        matches = sorted(glob.glob(expanded)) if glob.has_magic(expanded) else [expanded]
        if not matches:
            raise ContractError(f"source.paths entry did not match any files: {raw_path!r}")
        for match in matches:
            path = Path(match)
            if not path.exists():
                raise ContractError(f"source path does not exist: {raw_path!r}")
            if path.is_dir():
                raise ContractError(f"source path must be a file, got directory: {path}")
            files.append(path)
    return tuple(files)


def source_manifest(source: PrepareSourceConfig, base: Path) -> dict[str, Any]:
    """The ``source`` section of a prepared manifest: what was read, and for local files how many and how large."""

    if source.type == "hf":
        return {"type": source.type, "dataset": source.dataset, "name": source.name, "data_dir": source.data_dir,
                "split": source.split, "text_column": source.text_column, "streaming": source.streaming}
    files = resolve_source_files(source.paths, base)
    return {"type": source.type, "paths": list(source.paths),
            "text_column": None if source.type == "text" else source.text_column,
            "resolved_file_count": len(files), "resolved_total_bytes": sum(f.stat().st_size for f in files)}


def iter_texts(source: PrepareSourceConfig, base: Path) -> Iterator[str]:
    if source.type == "hf":
        try:
            import datasets
        except ImportError as exc:
            raise ContractError("source.type='hf' needs the datasets package") from exc
        ds = datasets.load_dataset(source.dataset, name=source.name, data_dir=source.data_dir, split=source.split,
                                   streaming=source.streaming)
        for row in ds:
            text = row.get(source.text_column)
            if isinstance(text, str) and text:
                yield text
        return
    for path in resolve_source_files(source.paths, base):
        if source.type == "text":
            with path.open("r", encoding="utf-8") as handle:
                for line in handle:
                    line = line.rstrip("\n")
                    if line:
                        yield line
        elif source.type == "jsonl":
            with path.open("r", encoding="utf-8") as handle:
                for n, line in enumerate(handle, 1):
                    if not line.strip():
                        continue
                    try:
                        row = json.loads(line)
                    except json.JSONDecodeError as exc:
                        raise ContractError(f"failed to parse {path} line {n}: {exc}") from exc
                    text = row.get(source.text_column) if isinstance(row, dict) else None
                    if isinstance(text, str) and text:
                        yield text
        elif source.type == "parquet":
            import pyarrow.parquet as pq

            pf = pq.ParquetFile(path)
            for batch in pf.iter_batches(columns=[source.text_column]):
                for text in batch.column(0).to_pylist():
                    if isinstance(text, str) and text:
                        yield text


_WORKER_TOKENIZER = None


def _worker_init(name: str) -> None:
    global _WORKER_TOKENIZER
    _WORKER_TOKENIZER = load_tokenizer(name)


def _worker_encode(texts: list[str]) -> list[list[int]]:
    return [_WORKER_TOKENIZER.encode(t) for t in texts]


def _batches(items: Iterable[str], size: int) -> Iterator[list[str]]:
    batch: list[str] = []
    for item in items:
        batch.append(item)
        if len(batch) == size:
            yield batch
            batch = []
    if batch:
        yield batch


def tokenized_documents(cfg: PrepareConfig, base: Path) -> Iterator[list[int]]:
    workers = resolve_workers(cfg.tokenization.workers)
    texts = iter_texts(cfg.source, base)
    if workers == 1:
        tok = load_tokenizer(cfg.tokenizer.name)
        for text in texts:
            yield tok.encode(text)
        return
    with ProcessPoolExecutor(max_workers=workers, initializer=_worker_init, initargs=(cfg.tokenizer.name,)) as pool:
        pending = []
        for batch in _batches(texts, cfg.tokenization.batch_docs):
            pending.append(pool.submit(_worker_encode, batch))
            if len(pending) >= cfg.tokenization.queue_batches:
                for doc in pending.pop(0).result():
                    yield doc
        for fut in pending:
            for doc in fut.result():
                yield doc


class ShardWriter:
    """Appends uint32 tokens into ``tokens-%05d.bin`` files of ``shard_tokens`` each with running sha256."""

    def __init__(self, out_dir: Path, shard_tokens: int):
        self.out_dir, self.shard_tokens = out_dir, shard_tokens
        self.shards: list[dict[str, Any]] = []
        self.total = 0
        self._handle = None
        self._digest = None
        self._count = 0
        self._start = 0

    def _open(self) -> None:
        name = f"tokens-{len(self.shards):05d}.bin"
        self._handle = (self.out_dir / name).open("wb")
        self._digest = sha256()
        self._count = 0
        self._start = self.total
        self._name = name

    def _close(self) -> None:
        if self._handle is None:
            return
        self._handle.close()
        self.shards.append({"path": self._name, "start": self._start, "end": self._start + self._count,
                            "tokens": self._count, "bytes": self._count * 4, "sha256": self._digest.hexdigest()})
        self._handle = None

    def write(self, tokens: np.ndarray) -> None:
        pos = 0
        while pos < len(tokens):
            if self._handle is None:
                self._open()
            take = min(len(tokens) - pos, self.shard_tokens - self._count)
            chunk = np.ascontiguousarray(tokens[pos:pos + take], dtype="<u4").tobytes()
            self._handle.write(chunk)
            self._digest.update(chunk)
            self._count += take
            self.total += take
            pos += take
            if self._count == self.shard_tokens:
                self._close()

    def finish(self) -> list[dict[str, Any]]:
        self._close()
        return self.shards


def resolve_workers(workers) -> int:
    if workers == "auto":
        import os

        return max(1, min(8, (os.cpu_count() or 2) - 1))
    return int(workers)


def prepare_dataset(config_path: str | Path, *, overwrite: bool = False) -> dict[str, Any]:
    import time

    started = time.perf_counter()
    config_path = Path(config_path)
    cfg = load_prepare_config(config_path)
    out_dir = cfg.output.path if cfg.output.path.is_absolute() else Path.cwd() / cfg.output.path
    if out_dir.exists():
        if not overwrite:
            raise ContractError(f"output directory already exists: {out_dir}; rerun with --overwrite to replace it")
        shutil.rmtree(out_dir)
    out_dir.mkdir(parents=True)
    tok = load_tokenizer(cfg.tokenizer.name)
    writer = ShardWriter(out_dir, cfg.output.shard_tokens)
    offsets = [0]
    budget = cfg.output.max_tokens
    docs_seen = 0
    for doc in tokenized_documents(cfg, config_path.parent):
        docs_seen += 1
        ids = list(doc) + ([tok.eot_id] if cfg.tokenizer.append_eot else [])
        if not ids:
            continue
        if writer.total + len(ids) > budget:
            ids = ids[: budget - writer.total]
        if not ids:
            break
        writer.write(np.asarray(ids, dtype=np.uint32))
        offsets.append(writer.total)
        if writer.total >= budget:
            break
    shards = writer.finish()
    total = writer.total
    if total < 2 or len(offsets) < 2:
        raise ContractError("the source produced too few tokens to prepare a dataset")
    off = np.asarray(offsets, dtype="<u8")
    val_start = total - max(1, int(round(total * cfg.output.val_fraction)))
    pos = int(np.searchsorted(off, val_start, side="left"))
    val_start = int(off[min(pos, len(off) - 1)])
    val_start = min(max(val_start, 1), total - 1)
    (out_dir / DOCUMENT_OFFSETS_FILENAME).write_bytes(off.tobytes())
    tb = tok.token_byte_lengths().astype("<u2")
    (out_dir / TOKEN_BYTES_FILENAME).write_bytes(tb.tobytes())
    elapsed = time.perf_counter() - started
    from research_b200.services.artifacts import utc_now

    manifest = {
        "schema_version": 1, "created_at": utc_now(), "kind": "training_tokens", "dtype": "uint32",
        "tokenizer": {"name": cfg.tokenizer.name, "vocab_size": int(tok.vocab_size), "eot_id": int(tok.eot_id),
                      "eot_token": int(tok.eot_id), "append_eot": cfg.tokenizer.append_eot},
        "source": source_manifest(cfg.source, config_path.parent),
        "val_fraction": float(cfg.output.val_fraction), "max_tokens": cfg.output.max_tokens,
        "shard_tokens": cfg.output.shard_tokens,
        "num_tokens": total, "num_docs": len(offsets) - 1, "source_docs_seen": docs_seen,
        "elapsed_sec": elapsed, "tokens_per_sec": total / elapsed if elapsed > 0 else None,
        "tokenization": {"workers": resolve_workers(cfg.tokenization.workers),
                         "batch_docs": cfg.tokenization.batch_docs, "queue_batches": cfg.tokenization.queue_batches},
        "shards": shards,
        "splits": {"train": {"start": 0, "end": val_start, "tokens": val_start},
                   "val": {"start": val_start, "end": total, "tokens": total - val_start}},
        "train_tokens": val_start, "val_tokens": total - val_start,
        "documents": {"count": len(offsets) - 1},
        "files": {"token_bytes": {"path": "token_bytes.bin", "dtype": "uint16", "bytes": int(tb.nbytes),
                                  "sha256": sha256(tb.tobytes()).hexdigest()},
                  "document_offsets": {"path": "document_offsets.u64", "dtype": "uint64", "bytes": int(off.nbytes),
                                       "sha256": sha256(off.tobytes()).hexdigest()}},
    }
    manifest_path = out_dir / "manifest.json"
    manifest_path.write_text(json.dumps(manifest, sort_keys=True, indent=1))
    from research_b200.data.manifest import dataset_manifest_summary, validate_dataset_manifest

    validated = validate_dataset_manifest(manifest_path, tokenizer_id=cfg.tokenizer.name, verify_checksums=True)
    summary = dataset_manifest_summary(validated)
    summary["num_tokens"] = total
    return summary


def build_token_bytes(tokenizer) -> np.ndarray:
    """UTF-8 byte length of every token id as ``uint16`` (EOT counts zero): the table behind bits per byte."""

    return tokenizer.token_byte_lengths().astype("<u2")


def load_hf_texts(source: PrepareSourceConfig) -> Iterator[str]:
    """The documents of a Hugging Face source (``source.type = "hf"``) as strings."""

    if source.type != "hf":
        raise ContractError(f"load_hf_texts needs source.type='hf', got {source.type!r}")
    return iter_texts(source, Path.cwd())


def prepare_result_to_dict(summary: Mapping[str, Any]) -> dict[str, Any]:
    return dict(summary)


def prepare_result_to_json(summary: Mapping[str, Any]) -> str:
    return json.dumps(dict(summary), sort_keys=True, separators=(",", ":"))


def format_prepare_result(summary: Mapping[str, Any]) -> str:
    return (f"prepared {summary['num_tokens']:,} tokens at {summary['manifest_path']} "
            f"(train {summary['train_tokens']:,}, val {summary['val_tokens']:,}, shards {summary['shard_count']}, "
            f"documents {summary['document_count']})")
