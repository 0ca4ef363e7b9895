"""Deterministic prepared-token batch pipelines with JSON-checkpointable state.

Three orders, as in the reference (src/jaxtitan/data/pipeline.py:71-832):

* ``sequential``      record ``k`` = tokens ``[start + k*S, start + k*S + S + 1)`` of the split;
* ``shuffle``         the same records visited through a seeded permutation (own permutation: the
                      reference uses Grain's index sampler, which is not available here, so the state
                      records ``backend="blackwell_native"`` and a resume across frameworks fails loudly);
* ``document_buffer`` the reference's document-buffer packer, reproduced draw for draw with the same NumPy
                      ``default_rng`` calls (pipeline.py:528-704), so batches and the saved state match.

Batches are NumPy arrays on the host; the training loop stages them through pinned memory.
"""

from __future__ import annotations

import bisect
from collections.abc import Mapping
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Protocol

import numpy as np

from research_b200 import __version__
from research_b200.config.canonical import normalize
from research_b200.contracts import Batch
from research_b200.data.manifest import PreparedDatasetManifest, validate_dataset_manifest
from research_b200.errors import ContractError

STATE_SCHEMA_VERSION = 2
BACKEND = "blackwell_native"
NUM_EPOCHS = 1
DROP_REMAINDER = True
DEFAULT_ORDER = "sequential"
DEFAULT_WORKER_COUNT = 0
DEFAULT_WORKER_BUFFER_SIZE = 1
DEFAULT_PREFETCH = False


def backend_version() -> str:
    return f"research_b200-{__version__}+numpy-{np.__version__}"


@dataclass(frozen=True, slots=True)
class DataPipelineState:
    """Host state of a data pipeline; field set matches the reference's ``DataPipelineState`` (state.py:36-66)."""

    schema_version: int
    backend: str
    backend_version: str | None
    split: str
    order: str
    shuffle_seed: int | None
    worker_count: int
    worker_buffer_size: int
    prefetch: bool
    manifest_path: Path | None
    manifest_sha256: str | None
    tokenizer_id: str
    seq_len: int
    batch_size: int
    num_records: int
    next_record_index: int
    token_offset: int
    epoch: int
    sampler_summary: str
    source_summary: str
    grain_state: dict[str, Any]
    stream_state: dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if self.manifest_path is not None:
            object.__setattr__(self, "manifest_path", Path(self.manifest_path))
        object.__setattr__(self, "grain_state", dict(self.grain_state))
        object.__setattr__(self, "stream_state", dict(self.stream_state))


def data_pipeline_state_to_dict(state: DataPipelineState) -> dict[str, Any]:
    return normalize(asdict(state))


_STATE_INT_FIELDS = ("schema_version", "worker_count", "worker_buffer_size", "seq_len", "batch_size", "num_records",
                     "next_record_index", "token_offset", "epoch")


def data_pipeline_state_from_mapping(raw: Mapping[str, Any]) -> DataPipelineState:
    if not isinstance(raw, Mapping):
        raise ContractError("data pipeline state must be a JSON object")
    for name in _STATE_INT_FIELDS:
        v = raw.get(name)
        if not isinstance(v, int) or isinstance(v, bool):
            raise ContractError(f"data pipeline state.{name} must be an integer")
    for name in ("backend", "split", "order", "tokenizer_id", "sampler_summary", "source_summary"):
        if not isinstance(raw.get(name), str):
            raise ContractError(f"data pipeline state.{name} must be a string")
    if not isinstance(raw.get("grain_state"), Mapping):
        raise ContractError("data pipeline state.grain_state must be an object")
    return DataPipelineState(
        schema_version=raw["schema_version"], backend=raw["backend"], backend_version=raw.get("backend_version"),
        split=raw["split"], order=raw["order"], shuffle_seed=raw.get("shuffle_seed"),
        worker_count=raw["worker_count"], worker_buffer_size=raw["worker_buffer_size"],
        prefetch=bool(raw.get("prefetch", False)), manifest_path=raw.get("manifest_path"),
        manifest_sha256=raw.get("manifest_sha256"), tokenizer_id=raw["tokenizer_id"], seq_len=raw["seq_len"],
        batch_size=raw["batch_size"], num_records=raw["num_records"], next_record_index=raw["next_record_index"],
        token_offset=raw["token_offset"], epoch=raw["epoch"], sampler_summary=raw["sampler_summary"],
        source_summary=raw["source_summary"], grain_state=dict(raw["grain_state"]),
        stream_state=dict(raw.get("stream_state") or {}),
    )


@dataclass(frozen=True, slots=True)
class BatchProvenance:
    split: str
    epoch: int
    token_start: int
    token_end: int
    examples: int
    target_tokens: int
    row_start_offsets: tuple[int, ...]
    row_doc_ids: tuple[int, ...] | None = None


@dataclass(frozen=True, slots=True)
class PipelineBatch:
    batch: Batch
    state: DataPipelineState
    provenance: BatchProvenance


class TrainingDataPipeline(Protocol):
    def initial_state(self) -> DataPipelineState: ...

    def next_batch(self, state: DataPipelineState) -> PipelineBatch: ...

    def state_from_json(self, raw: Mapping[str, Any]) -> DataPipelineState: ...

    def state_to_json(self, state: DataPipelineState) -> dict[str, Any]: ...

    def describe(self) -> dict[str, Any]: ...


# --------------------------------------------------------------------------------------------------
# token access
# --------------------------------------------------------------------------------------------------
class TokenReader:
    """Memory-mapped random access to the concatenated shards of a prepared dataset
    (reference: src/jaxtitan/data/tokens.py:17-65)."""

    def __init__(self, manifest: PreparedDatasetManifest) -> None:
        self.manifest = manifest
        self._starts = [s.start for s in manifest.shards]
        self._maps = [np.memmap(manifest.data_dir / s.path, dtype="<u4", mode="r") for s in manifest.shards]

    def read(self, start: int, end: int) -> np.ndarray:
        total = self.manifest.num_tokens
        if start < 0 or end < start or end > total:
            raise IndexError(f"token range is outside dataset bounds: start={start}, end={end}, total={total}")
        if end == start:
            return np.empty((0,), dtype=np.uint32)
        pieces = []
        cursor = start
        while cursor < end:
            idx = bisect.bisect_right(self._starts, cursor) - 1
            shard = self.manifest.shards[idx]
            if cursor >= shard.end:
                raise IndexError(f"token range crosses a gap before token {cursor}")
            stop = min(end, shard.end)
            pieces.append(np.asarray(self._maps[idx][cursor - shard.start:stop - shard.start], dtype=np.uint32))
            cursor = stop
        return pieces[0] if len(pieces) == 1 else np.concatenate(pieces)


def read_token_range(manifest: PreparedDatasetManifest, start: int, end: int) -> np.ndarray:
    return TokenReader(manifest).read(start, end)


def open_document_offsets(manifest: PreparedDatasetManifest) -> np.ndarray | None:
    if manifest.documents is None:
        return None
    return np.memmap(manifest.data_dir / manifest.documents.path, dtype="<u8", mode="r")


def document_spans(offsets: np.ndarray, split_start: int, split_end: int) -> dict[int, tuple[int, int]]:
    """Documents clipped to a split: ``{doc_id: (start, end)}`` for every document that overlaps it."""

    first = int(np.searchsorted(offsets, split_start, side="right")) - 1
    spans: dict[int, tuple[int, int]] = {}
    doc = max(first, 0)
    n_docs = len(offsets) - 1
    while doc < n_docs and int(offsets[doc]) < split_end:
        start = max(int(offsets[doc]), split_start)
        end = min(int(offsets[doc + 1]), split_end)
        if end > start:
            spans[doc] = (start, end)
        doc += 1
    return spans


def _split_of(manifest: PreparedDatasetManifest, split: str):
    if split not in ("train", "val"):
        raise ContractError(f"split must be 'train' or 'val', got {split!r}")
    return manifest.train if split == "train" else manifest.val


# --------------------------------------------------------------------------------------------------
# shared base
# --------------------------------------------------------------------------------------------------
class _PreparedPipelineBase:
    order = "sequential"

    def __init__(self, *, manifest: PreparedDatasetManifest, split: str, seq_len: int, batch_size: int,
                 shuffle_seed: int | None) -> None:
        if seq_len <= 0:
            raise ContractError(f"seq_len must be positive, got {seq_len}")
        if batch_size <= 0:
            raise ContractError(f"batch_size must be positive, got {batch_size}")
        token_split = _split_of(manifest, split)
        self.manifest = manifest
        self.split = split
        self.seq_len = int(seq_len)
        self.batch_size = int(batch_size)
        self.shuffle_seed = shuffle_seed
        self.split_start, self.split_end, self.split_tokens = token_split.start, token_split.end, token_split.tokens
        self.reader = TokenReader(manifest)
        self.document_offsets = open_document_offsets(manifest)
        self.document_aware = self.document_offsets is not None
        self.document_count = None if manifest.documents is None else manifest.documents.count
        self.backend_version = backend_version()
        self.num_records = 0
        self.source_summary = ""
        self.sampler_summary = ""
        # rows of every batch whose tokens this process needs (None: all).  The sampling state always advances
        # over the whole batch, so the order stays the same on every rank; only the token reads are skipped.
        self.local_rows: range | None = None

    def set_local_rows(self, rows: range | None) -> None:
        """Materialise only ``rows`` of each batch (a rank of a data-parallel job needs only its own rows); the
        other rows come back zero-filled and ``Batch.mask_count`` carries the whole batch's unmasked-token count."""

        if rows is not None and (rows.start < 0 or rows.stop > self.batch_size or rows.step != 1):
            raise ContractError(f"local rows {rows} are not inside a batch of {self.batch_size}")
        self.local_rows = rows

    def _is_local(self, row: int) -> bool:
        return self.local_rows is None or row in self.local_rows

    # -- state plumbing ----------------------------------------------------------------------------
    def _make_state(self, backend_state: Mapping[str, Any], next_record_index: int, epoch: int) -> DataPipelineState:
        return DataPipelineState(
            schema_version=STATE_SCHEMA_VERSION, backend=BACKEND, backend_version=self.backend_version,
            split=self.split, order=self.order, shuffle_seed=self.shuffle_seed, worker_count=0, worker_buffer_size=1,
            prefetch=False, manifest_path=self.manifest.manifest_path, manifest_sha256=self.manifest.manifest_sha256,
            tokenizer_id=self.manifest.tokenizer_id, seq_len=self.seq_len, batch_size=self.batch_size,
            num_records=self.num_records, next_record_index=next_record_index,
            token_offset=self.split_start + next_record_index * self.seq_len, epoch=epoch,
            sampler_summary=self.sampler_summary, source_summary=self.source_summary,
            grain_state=normalize(backend_state),
        )

    def _validate_state(self, state: DataPipelineState) -> None:
        expected = self._make_state(state.grain_state, state.next_record_index, state.epoch)
        for name in ("schema_version", "backend", "backend_version", "split", "order", "shuffle_seed", "worker_count",
                     "worker_buffer_size", "prefetch", "manifest_path", "manifest_sha256", "tokenizer_id", "seq_len",
                     "batch_size", "num_records", "sampler_summary", "source_summary"):
            actual, wanted = getattr(state, name), getattr(expected, name)
            if actual != wanted:
                raise ContractError(f"data pipeline state {name} mismatch: state={actual!r} pipeline={wanted!r}")
        if not 0 <= state.next_record_index <= self.num_records:
            raise ContractError(
                f"data pipeline next_record_index={state.next_record_index} is outside [0, {self.num_records}]"
            )
        if state.token_offset != expected.token_offset:
            raise ContractError(
                f"data pipeline token_offset={state.token_offset} does not match next_record_index "
                f"{state.next_record_index} expected_offset={expected.token_offset}"
            )
        if state.epoch != 0:
            raise ContractError("prepared-token pipelines support only epoch=0")

    def state_to_json(self, state: DataPipelineState) -> dict[str, Any]:
        self._validate_state(state)
        return data_pipeline_state_to_dict(state)

    def state_from_json(self, raw: Mapping[str, Any]) -> DataPipelineState:
        state = data_pipeline_state_from_mapping(raw)
        self._validate_state(state)
        return state

    def close(self) -> None:
        return None

    def _describe_common(self) -> dict[str, Any]:
        docs = self.manifest.documents
        return {
            "schema_version": 1,
            "backend": BACKEND,
            "backend_version": self.backend_version,
            "state_schema_version": STATE_SCHEMA_VERSION,
            "split": self.split,
            "order": self.order,
            "shuffle": self.order != "sequential",
            "shuffle_seed": self.shuffle_seed,
            "num_epochs": NUM_EPOCHS,
            "worker_count": 0,
            "worker_buffer_size": 1,
            "prefetch": False,
            "drop_remainder": DROP_REMAINDER,
            "batch_size": self.batch_size,
            "seq_len": self.seq_len,
            "num_records": self.num_records,
            "manifest_path": self.manifest.manifest_path.as_posix(),
            "manifest_sha256": self.manifest.manifest_sha256,
            "tokenizer_id": self.manifest.tokenizer_id,
            "split_start": self.split_start,
            "split_end": self.split_end,
            "split_tokens": self.split_tokens,
            "document_aware": self.document_aware,
            "document_count": self.document_count,
            "document_offsets_path": None if docs is None else docs.path.as_posix(),
            "document_offsets_sha256": None if docs is None else docs.sha256,
            "source_summary": self.source_summary,
            "sampler_summary": self.sampler_summary,
        }

    def describe(self) -> dict[str, Any]:
        return normalize(self._describe_common())


# --------------------------------------------------------------------------------------------------
# sequential / shuffle over fixed windows
# --------------------------------------------------------------------------------------------------
class PreparedTokenWindowPipeline(_PreparedPipelineBase):
    """Records are fixed windows of ``seq_len + 1`` tokens ``seq_len`` apart; visited in order or permuted."""

    def __init__(self, *, manifest: PreparedDatasetManifest, split: str, seq_len: int, batch_size: int,
                 order: str = "sequential", shuffle_seed: int | None = None) -> None:
        super().__init__(manifest=manifest, split=split, seq_len=seq_len, batch_size=batch_size,
                         shuffle_seed=shuffle_seed)
        if order not in ("sequential", "shuffle"):
            raise ContractError(f"window pipeline order must be 'sequential' or 'shuffle', got {order!r}")
        if order == "shuffle" and shuffle_seed is None:
            raise ContractError("data.shuffle_seed is required when data.order='shuffle'")
        self.order = order
        self.num_records = max(0, (self.split_tokens - 1) // self.seq_len)
        if self.num_records < self.batch_size:
            raise ContractError(
                f"{split} split has {self.num_records} records of seq_len={self.seq_len}, "
                f"but one batch requires {self.batch_size}"
            )
        self.source_summary = (
            f"PreparedTokenDataSource(manifest_sha256='{manifest.manifest_sha256}', split='{split}', "
            f"seq_len={self.seq_len}, tokenizer_id='{manifest.tokenizer_id}', document_aware={self.document_aware}, "
            f"document_count={self.document_count}, records={self.num_records})"
        )
        self.sampler_summary = (
            f"WindowSampler(order={order}, seed={shuffle_seed}, records={self.num_records}, num_epochs={NUM_EPOCHS})"
        )
        self._perm: np.ndarray | None = None
        if order == "shuffle":
            self._perm = np.random.default_rng(int(shuffle_seed)).permutation(self.num_records)

    def initial_state(self) -> DataPipelineState:
        return self._make_state({"next_index": 0}, 0, 0)

    def _record(self, key: int, materialise: bool = True) -> tuple[np.ndarray, int, int | None]:
        start = self.split_start + key * self.seq_len
        tokens = self.reader.read(start, start + self.seq_len + 1) if materialise else \
            np.zeros(self.seq_len + 1, dtype=np.int32)
        doc_id = None
        if self.document_offsets is not None:
            doc_id = int(np.searchsorted(self.document_offsets, start, side="right")) - 1
        return tokens, start, doc_id

    def next_batch(self, state: DataPipelineState) -> PipelineBatch:
        self._validate_state(state)
        first = state.next_record_index
        if first + self.batch_size > self.num_records:
            raise StopIteration(f"not enough records left in {self.split} split for one full batch")
        keys = range(first, first + self.batch_size)
        if self._perm is not None:
            keys = [int(self._perm[k]) for k in keys]
        rows = [self._record(int(k), self._is_local(i)) for i, k in enumerate(keys)]
        tokens = np.stack([r[0] for r in rows]).astype(np.int32)
        starts = tuple(r[1] for r in rows)
        doc_ids = None
        if self.document_offsets is not None:
            doc_ids = np.asarray([r[2] for r in rows], dtype=np.int32)
        batch = Batch(input_ids=tokens[:, :-1].copy(), target_ids=tokens[:, 1:].copy(),
                      loss_mask=np.ones((self.batch_size, self.seq_len), dtype=np.bool_), doc_ids=doc_ids,
                      mask_count=None if self.local_rows is None else float(self.batch_size * self.seq_len))
        nxt = first + self.batch_size
        return PipelineBatch(
            batch=batch,
            state=self._make_state({"next_index": nxt}, nxt, state.epoch),
            provenance=BatchProvenance(
                split=self.split, epoch=state.epoch, token_start=min(starts),
                token_end=max(starts) + self.seq_len, examples=self.batch_size,
                target_tokens=self.batch_size * self.seq_len, row_start_offsets=starts,
                row_doc_ids=None if doc_ids is None else tuple(int(v) for v in doc_ids.tolist()),
            ),
        )


# --------------------------------------------------------------------------------------------------
# document buffer
# --------------------------------------------------------------------------------------------------
class PreparedTokenDocumentBufferPipeline(_PreparedPipelineBase):
    """Packs each record from a small set of "active" documents picked at random.

    Algorithm (bit-compatible with the reference): ``rng = default_rng(seed)``; the document order is one
    ``rng.permutation`` of the split's document ids; the active set is kept filled to
    ``min(buffer_size, n_docs)`` from a refill queue that takes ``refill_size`` ids at a time; every piece
    of a record draws ``rng.integers(0, len(active))``, takes ``min(needed, remaining)`` tokens at that
    document's cursor and drops exhausted documents, until ``seq_len + 1`` tokens are gathered.
    ``loss_mask[i]`` is true when token ``i`` and token ``i + 1`` come from the same document.
    """

    order = "document_buffer"

    def __init__(self, *, manifest: PreparedDatasetManifest, split: str, seq_len: int, batch_size: int,
                 shuffle_seed: int, document_buffer_size: int, document_refill_size: int) -> None:
        if manifest.documents is None:
            raise ContractError("data.order='document_buffer' requires prepared manifest document offsets")
        super().__init__(manifest=manifest, split=split, seq_len=seq_len, batch_size=batch_size,
                         shuffle_seed=int(shuffle_seed))
        if document_buffer_size <= 0:
            raise ContractError(f"document_buffer_size must be positive, got {document_buffer_size}")
        if document_refill_size <= 0:
            raise ContractError(f"document_refill_size must be positive, got {document_refill_size}")
        self.document_buffer_size = int(document_buffer_size)
        self.document_refill_size = int(document_refill_size)
        self.document_spans = document_spans(self.document_offsets, self.split_start, self.split_end)
        self.document_ids = tuple(self.document_spans)
        self.num_records = max(0, self.split_tokens // (self.seq_len + 1))
        if not self.document_ids:
            raise ContractError(f"{split} split has no document spans")
        if self.num_records < self.batch_size:
            required = self.batch_size * (self.seq_len + 1)
            raise ContractError(
                f"{split} split has {self.split_tokens} tokens, but one document-buffer batch requires at least {required}"
            )
        self.source_summary = (
            f"PreparedTokenDocumentBufferPipeline(manifest_sha256='{manifest.manifest_sha256}', split='{split}', "
            f"seq_len={self.seq_len}, tokenizer_id='{manifest.tokenizer_id}', seed={self.shuffle_seed}, "
            f"buffer_size={self.document_buffer_size}, refill_size={self.document_refill_size}, "
            f"documents={len(self.document_ids)})"
        )
        self.sampler_summary = (
            f"DocumentBufferSampler(seed={self.shuffle_seed}, buffer_size={self.document_buffer_size}, "
            f"refill_size={self.document_refill_size}, documents={len(self.document_ids)})"
        )

    def initial_state(self) -> DataPipelineState:
        rng = np.random.default_rng(self.shuffle_seed)
        order = [int(v) for v in rng.permutation(np.asarray(self.document_ids, dtype=np.int64)).tolist()]
        backend = {"rng_state": normalize(rng.bit_generator.state), "document_order": order, "replacement_cursor": 0,
                   "refill_queue": [], "active": []}
        self._fill_active(backend)
        return self._make_state(backend, 0, 0)

    def _pop_replacement(self, backend: dict[str, Any]) -> int | None:
        if not backend["refill_queue"]:
            cursor = int(backend["replacement_cursor"])
            order = backend["document_order"]
            if cursor >= len(order):
                return None
            stop = min(cursor + self.document_refill_size, len(order))
            backend["refill_queue"] = [int(v) for v in order[cursor:stop]]
            backend["replacement_cursor"] = stop
        return int(backend["refill_queue"].pop(0))

    def _fill_active(self, backend: dict[str, Any]) -> None:
        target = min(self.document_buffer_size, len(self.document_ids))
        while len(backend["active"]) < target:
            doc = self._pop_replacement(backend)
            if doc is None:
                break
            start, end = self.document_spans[doc]
            backend["active"].append({"doc_id": int(doc), "cursor": int(start), "end": int(end)})

    def _next_record(self, backend: dict[str, Any], rng: np.random.Generator, materialise: bool = True):
        """One packed row.  ``materialise=False`` advances the sampler exactly as usual but reads no tokens: the row
        comes back zero-filled, with the number of unmasked targets it would have had."""

        need = self.seq_len + 1
        pieces: list[np.ndarray] = []
        piece_docs: list[tuple[int, int]] = []  # (doc_id, count)
        first_offset = None
        max_offset = 0
        got = 0
        while got < need:
            self._fill_active(backend)
            active = backend["active"]
            if not active:
                raise StopIteration
            idx = int(rng.integers(0, len(active)))
            entry = active[idx]
            cursor, end, doc_id = int(entry["cursor"]), int(entry["end"]), int(entry["doc_id"])
            take = min(need - got, end - cursor)
            if materialise:
                pieces.append(self.reader.read(cursor, cursor + take))
            piece_docs.append((doc_id, take))
            if first_offset is None:
                first_offset = cursor
            max_offset = max(max_offset, cursor + take)
            got += take
            cursor += take
            if cursor >= end:
                del active[idx]
            else:
                active[idx] = {"doc_id": doc_id, "cursor": cursor, "end": end}
        docs = np.asarray([d for d, _ in piece_docs], dtype=np.int64)
        # a target is masked where the document changes: once per pair of neighbouring pieces of different documents
        unmasked = self.seq_len - int(np.count_nonzero(docs[1:] != docs[:-1]))
        if not materialise:
            return (np.zeros(need, dtype=np.int32), np.zeros(self.seq_len, dtype=np.bool_),
                    np.zeros(need, dtype=np.int64), int(piece_docs[0][0]), int(first_offset), int(max_offset), unmasked)
        tokens = np.concatenate(pieces).astype(np.int32)
        token_docs = np.repeat(docs, np.asarray([c for _, c in piece_docs], dtype=np.int64))
        loss_mask = token_docs[:-1] == token_docs[1:]
        return tokens, loss_mask, token_docs, int(piece_docs[0][0]), int(first_offset), int(max_offset), unmasked

    def next_batch(self, state: DataPipelineState) -> PipelineBatch:
        self._validate_state(state)
        backend = _copy_backend(state.grain_state)
        rng = np.random.default_rng()
        rng.bit_generator.state = backend["rng_state"]
        rows = []
        for row in range(self.batch_size):
            try:
                rows.append(self._next_record(backend, rng, self._is_local(row)))
            except StopIteration as exc:
                raise StopIteration(
                    f"not enough document-buffer tokens left in {self.split} split for one full batch"
                ) from exc
        backend["rng_state"] = normalize(rng.bit_generator.state)
        tokens = np.stack([r[0] for r in rows])
        doc_ids = np.asarray([r[3] for r in rows], dtype=np.int32)
        batch = Batch(input_ids=tokens[:, :-1].copy(), target_ids=tokens[:, 1:].copy(),
                      loss_mask=np.stack([r[1] for r in rows]).astype(np.bool_), doc_ids=doc_ids,
                      token_doc_ids=np.stack([r[2][:-1] for r in rows]).astype(np.int32),
                      mask_count=None if self.local_rows is None else float(sum(r[6] for r in rows)))
        nxt = state.next_record_index + self.batch_size
        starts = tuple(r[4] for r in rows)
        return PipelineBatch(
            batch=batch,
            state=self._make_state(backend, nxt, state.epoch),
            provenance=BatchProvenance(
                split=self.split, epoch=state.epoch, token_start=min(starts), token_end=max(r[5] for r in rows),
                examples=self.batch_size, target_tokens=self.batch_size * self.seq_len, row_start_offsets=starts,
                row_doc_ids=tuple(int(v) for v in doc_ids.tolist()),
            ),
        )

    def _validate_state(self, state: DataPipelineState) -> None:
        super()._validate_state(state)
        gs = state.grain_state
        if not isinstance(gs.get("rng_state"), Mapping):
            raise ContractError("data pipeline state.rng_state must be an object")
        for name in ("document_order", "refill_queue"):
            v = gs.get(name)
            if not isinstance(v, list) or any(not isinstance(x, int) or isinstance(x, bool) for x in v):
                raise ContractError(f"data pipeline state.{name} must be a list of integers")
        if not isinstance(gs.get("replacement_cursor"), int):
            raise ContractError("data pipeline state.replacement_cursor must be an integer")
        active = gs.get("active")
        if not isinstance(active, list):
            raise ContractError("data pipeline state.active must be a list")
        for idx, item in enumerate(active):
            if not isinstance(item, Mapping):
                raise ContractError(f"data pipeline state.active[{idx}] must be an object")
            for key in ("doc_id", "cursor", "end"):
                if not isinstance(item.get(key), int) or isinstance(item.get(key), bool):
                    raise ContractError(f"data pipeline state.active[{idx}].{key} must be an integer")
            doc_id = item["doc_id"]
            if doc_id not in self.document_spans:
                raise ContractError(f"data pipeline active doc_id={doc_id} is not in split documents")
            start, end = self.document_spans[doc_id]
            if item["end"] != end or not start <= item["cursor"] <= end:
                raise ContractError(f"data pipeline active document cursor is invalid for doc_id={doc_id}")

    def describe(self) -> dict[str, Any]:
        out = self._describe_common()
        out["document_buffer_size"] = self.document_buffer_size
        out["document_refill_size"] = self.document_refill_size
        return normalize(out)


def _copy_backend(raw: Mapping[str, Any]) -> dict[str, Any]:
    out = dict(raw)
    out["rng_state"] = _rng_state_from_json(raw["rng_state"])
    out["document_order"] = list(raw["document_order"])
    out["refill_queue"] = list(raw["refill_queue"])
    out["active"] = [dict(item) for item in raw["active"]]
    return out


def _rng_state_from_json(raw: Mapping[str, Any]) -> dict[str, Any]:
    state = {k: (dict(v) if isinstance(v, Mapping) else v) for k, v in raw.items()}
    return state


# --------------------------------------------------------------------------------------------------
# factories
# --------------------------------------------------------------------------------------------------
def build_prepared_token_pipeline(path: str | Path, *, tokenizer_id: str | None, split: str, seq_len: int,
                                  batch_size: int, order: str = "sequential", shuffle_seed: int | None = None,
                                  worker_count: int = 0, worker_buffer_size: int = 1, prefetch: bool = False,
                                  document_buffer_size: int | None = None,
                                  document_refill_size: int | None = None) -> TrainingDataPipeline:
    manifest = validate_dataset_manifest(path, tokenizer_id=tokenizer_id)
    if order == "document_buffer":
        if document_buffer_size is None or document_refill_size is None:
            raise ContractError("document_buffer order requires document_buffer_size and document_refill_size")
        return PreparedTokenDocumentBufferPipeline(
            manifest=manifest, split=split, seq_len=seq_len, batch_size=batch_size, shuffle_seed=int(shuffle_seed or 0),
            document_buffer_size=document_buffer_size, document_refill_size=document_refill_size)
    return PreparedTokenWindowPipeline(manifest=manifest, split=split, seq_len=seq_len, batch_size=batch_size,
                                       order=order, shuffle_seed=shuffle_seed)


def data_pipeline_compat_payload(path: str | Path, **kwargs: Any) -> dict[str, Any]:
    """What the resume fingerprint records about the data pipeline (reference: pipeline.py:798-832)."""

    pipeline = build_prepared_token_pipeline(path, **kwargs)
    try:
        return pipeline.describe()
    finally:
        pipeline.close()
