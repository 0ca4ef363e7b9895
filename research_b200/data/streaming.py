"""Hugging Face streaming text -> token batches with exact resume
(reference: src/jaxtitan/data/streaming.py:28-370).

Rows of a streaming ``datasets`` dataset are tokenised on the fly (EOT appended) and laid end to end into one token
stream.  A record is ``seq_len + 1`` consecutive tokens and the next record starts ``seq_len`` further on, so every
token of the stream is a target exactly once.  Only what the next record needs is taken from the current document:
the pipeline never holds more than ``seq_len + 1`` pending tokens plus one tokenised document.

The checkpointable state is the dataset's own ``state_dict()`` taken *before* the current document was read, whether
a document is half consumed and at which token, the pending tokens, and the row / document / token counters - so a
resumed run re-reads that one document, skips to the saved offset and continues with the very next token.  The
``stream_state`` keys are the reference's (``hf_state``, ``current_doc_active``, ``current_doc_token_offset``,
``pending_tokens``, ``rows_seen``, ``docs_seen``, ``tokens_emitted``).  Needs the ``datasets`` package and a
reachable (or cached) dataset; tests inject a fake iterable dataset and tokenizer.
"""

from __future__ import annotations

import json
import os
from collections.abc import Mapping
from dataclasses import asdict
from typing import Any, Callable

import numpy as np

from research_b200.config.specs import DataSpec, HFStreamingSpec
from research_b200.contracts import Batch
from research_b200.data.pipeline import (BatchProvenance, DataPipelineState, PipelineBatch,
                                         data_pipeline_state_from_mapping, data_pipeline_state_to_dict)
from research_b200.errors import ContractError

STREAM_BACKEND = "hf_streaming"
STREAM_STATE_SCHEMA_VERSION = 2
STREAM_ORDER = "sequential"
STREAM_NUM_RECORDS_UNKNOWN = -1
SAMPLER_SUMMARY = "hf_streaming_sequential"


def datasets_version() -> str | None:
    from importlib import metadata

    try:
        return metadata.version("datasets")
    except metadata.PackageNotFoundError:
        return None


def _jsonable(value: Any) -> Any:
    return json.loads(json.dumps(value, sort_keys=True))


def source_summary(source: HFStreamingSpec) -> dict[str, Any]:
    return _jsonable(asdict(source))


def load_hf_dataset(source: HFStreamingSpec) -> Any:
    """``datasets.load_dataset(..., streaming=True)`` at the pinned revision; the access token comes from
    ``HF_TOKEN`` / ``HUGGING_FACE_HUB_TOKEN`` (reference: streaming.py:380-401)."""

    try:
        from datasets import load_dataset
    except ImportError as exc:
        raise ContractError("HF streaming requires the 'datasets' package") from exc
    kwargs: dict[str, Any] = {"split": source.split, "streaming": True, "revision": source.revision}
    if source.data_dir is not None:
        kwargs["data_dir"] = source.data_dir
    token = os.environ.get("HF_TOKEN") or os.environ.get("HUGGING_FACE_HUB_TOKEN")
    if token:
        kwargs["token"] = token
    try:
        if source.name is None:
            return load_dataset(source.dataset, **kwargs)
        return load_dataset(source.dataset, source.name, **kwargs)
    except Exception as exc:
        raise ContractError(f"failed to load HF streaming dataset {source.dataset!r}: {exc}") from exc


def _eot(tokenizer: Any) -> int:
    for name in ("eot_id", "eot_token"):
        if hasattr(tokenizer, name):
            return int(getattr(tokenizer, name))
    raise ContractError("the tokenizer has no end-of-text id")


class _DocumentCursor:
    """The token stream of a row iterator: which dataset state the current document was read from, the document's
    tokens and how many of them were handed out."""

    def __init__(self, pipeline: "HFStreamingTextPipeline", dataset: Any) -> None:
        self.pipeline = pipeline
        self.dataset = dataset
        self.iterator = iter(dataset)
        self.hf_state: Any = _jsonable(dataset.state_dict())
        self.tokens: list[int] | None = None
        self.offset = 0
        self.rows_seen = 0
        self.docs_seen = 0

    def _read_document(self) -> None:
        while True:
            self.hf_state = _jsonable(self.dataset.state_dict())
            try:
                row = next(self.iterator)
            except StopIteration as exc:
                raise StopIteration("HF streaming source ended before one full batch could be produced") from exc
            self.rows_seen += 1
            tokens = self.pipeline.tokens_from_row(row)
            if tokens:
                self.docs_seen += 1
                self.tokens, self.offset = tokens, 0
                return

    def take(self, count: int) -> list[int]:
        """Up to ``count`` tokens of the current document (a new one is read when the last is used up)."""

        if self.tokens is None:
            self._read_document()
        piece = self.tokens[self.offset:self.offset + count]
        self.offset += len(piece)
        if self.offset >= len(self.tokens):
            self.tokens, self.offset = None, 0
            self.hf_state = _jsonable(self.dataset.state_dict())
        return piece


class HFStreamingTextPipeline:
    def __init__(self, data: DataSpec | None = None, *, seq_len: int, batch_size: int,
                 source: HFStreamingSpec | None = None, tokenizer_id: str | None = None,
                 dataset_loader: Callable[[HFStreamingSpec], Any] | None = None, tokenizer: Any | None = None):
        if data is not None:
            source = source or data.hf_streaming
            tokenizer_id = tokenizer_id or data.tokenizer_id
        if source is None:
            raise ContractError("hf_streaming pipeline needs [data.hf_streaming]")
        if not tokenizer_id:
            raise ContractError("tokenizer_id is required for HF streaming data")
        if seq_len <= 0:
            raise ContractError(f"seq_len must be positive, got {seq_len}")
        if batch_size <= 0:
            raise ContractError(f"batch_size must be positive, got {batch_size}")
        self.source = self.spec = source
        self.tokenizer_id = tokenizer_id
        self.seq_len, self.batch_size = int(seq_len), int(batch_size)
        self.split, self.order, self.shuffle_seed = source.split, STREAM_ORDER, None
        self.worker_count, self.worker_buffer_size, self.prefetch = 0, 1, False
        self.backend_version = datasets_version()
        self.split_start = self.split_end = self.split_tokens = 0
        self._loader = dataset_loader or load_hf_dataset
        if tokenizer is None:
            from research_b200.data.prepare import load_tokenizer

            tokenizer = load_tokenizer(tokenizer_id)
        self.tokenizer = tokenizer
        self._eot = _eot(tokenizer) if source.append_eot else None
        self.source_summary = json.dumps(source_summary(source), sort_keys=True, separators=(",", ":"))
        self.sampler_summary = SAMPLER_SUMMARY
        self._cursor: _DocumentCursor | None = None
        self._pending: list[int] = []
        self._next_record = 0
        self._current: DataPipelineState | None = None

    # -- rows -> tokens ---------------------------------------------------------------------------------
    def tokens_from_row(self, row: Any) -> list[int]:
        column = self.source.text_column
        if not isinstance(row, Mapping):
            raise ContractError(f"HF streaming rows must be mappings, got {type(row).__name__}")
        if column not in row:
            raise ContractError(f"HF streaming row is missing text column {column!r}")
        text = row[column]
        if not isinstance(text, str):
            raise ContractError(f"HF streaming text column {column!r} must contain strings")
        tokens = [int(t) for t in self.tokenizer.encode(text)]
        if self._eot is not None:
            tokens.append(self._eot)
        return tokens

    # -- state ------------------------------------------------------------------------------------------
    def _snapshot(self) -> DataPipelineState:
        c = self._cursor
        emitted = self._next_record * self.seq_len
        return DataPipelineState(
            schema_version=STREAM_STATE_SCHEMA_VERSION, backend=STREAM_BACKEND, backend_version=self.backend_version,
            split=self.split, order=self.order, shuffle_seed=None, worker_count=0, worker_buffer_size=1,
            prefetch=False, manifest_path=None, manifest_sha256=None, tokenizer_id=self.tokenizer_id,
            seq_len=self.seq_len, batch_size=self.batch_size, num_records=STREAM_NUM_RECORDS_UNKNOWN,
            next_record_index=self._next_record, token_offset=emitted, epoch=0,
            sampler_summary=self.sampler_summary, source_summary=self.source_summary, grain_state={},
            stream_state={"hf_state": _jsonable(c.hf_state), "current_doc_active": c.tokens is not None,
                          "current_doc_token_offset": c.offset, "pending_tokens": list(self._pending),
                          "rows_seen": c.rows_seen, "docs_seen": c.docs_seen, "tokens_emitted": emitted})

    def initial_state(self) -> DataPipelineState:
        self._cursor = _DocumentCursor(self, self._loader(self.source))
        self._pending, self._next_record = [], 0
        self._current = self._snapshot()
        return self._current

    def _restore(self, state: DataPipelineState) -> None:
        stream = state.stream_state
        hf_state = _mapping(stream.get("hf_state"), "stream_state.hf_state")
        dataset = self._loader(self.source)
        if not hasattr(dataset, "load_state_dict"):
            raise ContractError("the streaming dataset cannot restore its state (no load_state_dict)")
        dataset.load_state_dict(dict(hf_state))
        cursor = _DocumentCursor(self, dataset)
        cursor.hf_state = _jsonable(hf_state)
        cursor.rows_seen = _int(stream, "rows_seen", "stream_state")
        cursor.docs_seen = _int(stream, "docs_seen", "stream_state")
        pending = stream.get("pending_tokens", [])
        if not isinstance(pending, list) or any(not isinstance(t, int) or isinstance(t, bool) for t in pending):
            raise ContractError("stream_state.pending_tokens must be a list of integers")
        if bool(stream.get("current_doc_active", False)):
            # the saved dataset state is the one from before the half-consumed document: read it again, skip ahead
            try:
                row = next(cursor.iterator)
            except StopIteration as exc:
                raise ContractError("HF streaming state points at a missing current document") from exc
            tokens = self.tokens_from_row(row)
            offset = _int(stream, "current_doc_token_offset", "stream_state")
            if offset < 0 or offset > len(tokens):
                raise ContractError(f"stream_state.current_doc_token_offset={offset} is outside current document tokens")
            cursor.tokens, cursor.offset = tokens, offset
        self._cursor, self._pending, self._next_record = cursor, list(pending), state.next_record_index
        self._current = state

    def _validate(self, state: DataPipelineState) -> None:
        checks = (
            ("schema_version", state.schema_version, STREAM_STATE_SCHEMA_VERSION),
            ("backend", state.backend, STREAM_BACKEND), ("backend_version", state.backend_version, self.backend_version),
            ("split", state.split, self.split), ("order", state.order, self.order),
            ("shuffle_seed", state.shuffle_seed, None), ("worker_count", state.worker_count, 0),
            ("worker_buffer_size", state.worker_buffer_size, 1), ("prefetch", state.prefetch, False),
            ("manifest_path", state.manifest_path, None), ("manifest_sha256", state.manifest_sha256, None),
            ("tokenizer_id", state.tokenizer_id, self.tokenizer_id), ("seq_len", state.seq_len, self.seq_len),
            ("batch_size", state.batch_size, self.batch_size),
            ("num_records", state.num_records, STREAM_NUM_RECORDS_UNKNOWN),
            ("sampler_summary", state.sampler_summary, self.sampler_summary),
            ("source_summary", state.source_summary, self.source_summary))
        for name, actual, wanted in checks:
            if actual != wanted:
                raise ContractError(f"HF streaming state {name} mismatch: state={actual!r} pipeline={wanted!r}")
        if state.next_record_index < 0:
            raise ContractError(f"HF streaming next_record_index must be non-negative, got {state.next_record_index}")
        if state.token_offset != state.next_record_index * self.seq_len:
            raise ContractError("HF streaming token_offset must match next_record_index * seq_len")
        if state.epoch != 0:
            raise ContractError("HF streaming supports only epoch=0")
        _mapping(state.stream_state.get("hf_state"), "stream_state.hf_state")

    # -- batches ----------------------------------------------------------------------------------------
    def _record(self) -> list[int]:
        need = self.seq_len + 1
        while len(self._pending) < need:
            self._pending.extend(self._cursor.take(need - len(self._pending)))
        record = self._pending[:need]
        self._pending = self._pending[self.seq_len:]          # the last token is the first input of the next record
        return record

    def next_batch(self, state: DataPipelineState) -> PipelineBatch:
        self._validate(state)
        if self._cursor is None or self._current != state:
            self._restore(state)
        start = self._next_record * self.seq_len
        rows = np.empty((self.batch_size, self.seq_len + 1), dtype=np.int32)
        for i in range(self.batch_size):
            rows[i] = self._record()
            self._next_record += 1
        self._current = self._snapshot()
        batch = Batch(input_ids=rows[:, :-1].copy(), target_ids=rows[:, 1:].copy(),
                      loss_mask=np.ones((self.batch_size, self.seq_len), dtype=np.bool_))
        offsets = tuple(start + i * self.seq_len for i in range(self.batch_size))
        return PipelineBatch(batch, self._current, BatchProvenance(
            split=self.split, epoch=0, token_start=offsets[0], token_end=offsets[-1] + self.seq_len,
            examples=self.batch_size, target_tokens=self.batch_size * self.seq_len, row_start_offsets=offsets))

    def state_to_json(self, state: DataPipelineState) -> dict[str, Any]:
        self._validate(state)
        return data_pipeline_state_to_dict(state)

    def state_from_json(self, raw: Mapping[str, Any]) -> DataPipelineState:
        state = data_pipeline_state_from_mapping({**raw, "num_records": raw.get("num_records",
                                                                                STREAM_NUM_RECORDS_UNKNOWN)})
        self._validate(state)
        return state

    def describe(self) -> dict[str, Any]:
        c = self._cursor
        return _jsonable({
            "schema_version": 1, "backend": STREAM_BACKEND, "backend_version": self.backend_version,
            "state_schema_version": STREAM_STATE_SCHEMA_VERSION, "split": self.split, "order": self.order,
            "shuffle": False, "shuffle_seed": None, "num_epochs": 1, "worker_count": 0, "worker_buffer_size": 1,
            "prefetch": False, "drop_remainder": True, "batch_size": self.batch_size, "seq_len": self.seq_len,
            "num_records": None, "manifest_path": None, "manifest_sha256": None, "tokenizer_id": self.tokenizer_id,
            "split_start": None, "split_end": None, "split_tokens": None, "document_aware": False,
            "document_count": None, "document_offsets_path": None, "document_offsets_sha256": None,
            "source": source_summary(self.source), "dataset": self.source.dataset, "revision": self.source.revision,
            "text_column": self.source.text_column, "append_eot": self.source.append_eot,
            "source_summary": self.source_summary, "sampler_summary": self.sampler_summary, "exact_resume": True,
            "rows_seen": 0 if c is None else c.rows_seen, "documents_seen": 0 if c is None else c.docs_seen,
            "tokens_emitted": self._next_record * self.seq_len})

    def close(self) -> None:
        self._cursor = None
        self._current = None


def _mapping(value: Any, name: str) -> Mapping[str, Any]:
    if not isinstance(value, Mapping):
        raise ContractError(f"{name} must be a JSON object")
    return value


def _int(raw: Mapping[str, Any], key: str, name: str) -> int:
    value = raw.get(key)
    if not isinstance(value, int) or isinstance(value, bool):
        raise ContractError(f"{name}.{key} must be an integer")
    return value


def build_hf_streaming_pipeline(data: DataSpec, *, seq_len: int, batch_size: int, **kwargs) -> HFStreamingTextPipeline:
    """The train pipeline of ``data.mode = "hf_streaming"``: sequential, unshuffled, no workers
    (reference: streaming.py:328-348)."""

    if data.tokenizer_id is None:
        raise ContractError("data.tokenizer_id is required when data.mode='hf_streaming'")
    if data.order != STREAM_ORDER:
        raise ContractError("HF streaming supports only data.order='sequential'")
    if data.shuffle_seed is not None:
        raise ContractError("HF streaming does not support data.shuffle_seed")
    if data.worker_count != 0 or data.worker_buffer_size != 1 or data.prefetch:
        raise ContractError("HF streaming requires worker_count=0, worker_buffer_size=1, and prefetch=false")
    return HFStreamingTextPipeline(data, seq_len=seq_len, batch_size=batch_size, **kwargs)


def hf_streaming_compat_payload(source: HFStreamingSpec, *, tokenizer_id: str, seq_len: int,
                                batch_size: int) -> dict[str, Any]:
    """What a resumed run must agree on with the run that wrote the checkpoint (reference: streaming.py:351-370)."""

    return _jsonable({"backend": STREAM_BACKEND, "backend_version": datasets_version(),
                      "state_schema_version": STREAM_STATE_SCHEMA_VERSION, "source": source_summary(source),
                      "tokenizer_id": tokenizer_id, "seq_len": seq_len, "batch_size": batch_size,
                      "order": STREAM_ORDER, "exact_resume": True})
