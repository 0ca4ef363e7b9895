"""Hugging Face streaming text -> token batches with exact resume
(reference: src/jaxtitan/data/streaming.py:28-325).

Documents are tokenised on the fly (EOT appended), concatenated into a pending token buffer and cut into rows of
``seq_len + 1`` tokens.  The checkpointable state is the dataset iterator's own ``state_dict()`` plus the pending
tokens and the number of documents consumed, so a resumed run continues with the very next token.  Needs the
``datasets`` package and a reachable (or cached) dataset; tests inject a fake iterable dataset.
"""

from __future__ import annotations

from collections.abc import Mapping
from typing import Any, Callable

import numpy as np

from research_b200.config.canonical import normalize
from research_b200.config.specs import DataSpec
from research_b200.contracts import Batch
from research_b200.data.pipeline import (STATE_SCHEMA_VERSION, BatchProvenance, DataPipelineState, PipelineBatch,
                                         backend_version, data_pipeline_state_from_mapping,
                                         data_pipeline_state_to_dict)
from research_b200.errors import ContractError

STREAM_BACKEND = "hf_streaming"


def _default_loader(spec) -> Any:
    try:
        import datasets
    except ImportError as exc:
        raise ContractError("data.mode='hf_streaming' needs the datasets package") from exc
    return datasets.load_dataset(spec.dataset, name=spec.name, data_dir=spec.data_dir, split=spec.split,
                                 revision=spec.revision, streaming=True)


class HFStreamingTextPipeline:
    def __init__(self, data: DataSpec, *, seq_len: int, batch_size: int,
                 dataset_loader: Callable[[Any], Any] | None = None, tokenizer: Any | None = None):
        if data.hf_streaming is None or data.tokenizer_id is None:
            raise ContractError("hf_streaming pipeline needs [data.hf_streaming] and data.tokenizer_id")
        self.spec = data.hf_streaming
        self.tokenizer_id = data.tokenizer_id
        self.seq_len, self.batch_size = int(seq_len), int(batch_size)
        self._loader = dataset_loader or _default_loader
        if tokenizer is None:
            from research_b200.data.prepare import load_tokenizer

            tokenizer = load_tokenizer(self.tokenizer_id)
        self.tokenizer = tokenizer
        self._dataset = None
        self._iterator = None
        self._iterator_state: Mapping[str, Any] | None = None
        self.source_summary = (f"HFStreamingTextSource(dataset='{self.spec.dataset}', split='{self.spec.split}', "
                               f"revision='{self.spec.revision}', text_column='{self.spec.text_column}')")
        self.sampler_summary = "StreamingSequential()"

    # -- state -------------------------------------------------------------------------------------
    def _state(self, next_record: int, stream_state: Mapping[str, Any]) -> DataPipelineState:
        return DataPipelineState(
            schema_version=STATE_SCHEMA_VERSION, backend=STREAM_BACKEND, backend_version=backend_version(),
            split=self.spec.split, order="sequential", shuffle_seed=None, worker_count=0, worker_buffer_size=1,
            prefetch=False, manifest_path=None, manifest_sha256=None, tokenizer_id=self.tokenizer_id,
            seq_len=self.seq_len, batch_size=self.batch_size, num_records=-1, next_record_index=next_record,
            token_offset=next_record * self.seq_len, epoch=0, sampler_summary=self.sampler_summary,
            source_summary=self.source_summary, grain_state={}, stream_state=normalize(stream_state))

    def initial_state(self) -> DataPipelineState:
        return self._state(0, {"dataset_state": None, "pending_tokens": [], "documents_consumed": 0})

    def _open(self, dataset_state: Mapping[str, Any] | None) -> None:
        self._dataset = self._loader(self.spec)
        if dataset_state is not None:
            if not hasattr(self._dataset, "load_state_dict"):
                raise ContractError("the streaming dataset cannot restore its state (no load_state_dict)")
            self._dataset.load_state_dict(dict(dataset_state))
        self._iterator = iter(self._dataset)
        self._iterator_state = dataset_state

    def next_batch(self, state: DataPipelineState) -> PipelineBatch:
        if state.backend != STREAM_BACKEND:
            raise ContractError(f"data pipeline state backend mismatch: state={state.backend!r} pipeline={STREAM_BACKEND!r}")
        stream = dict(state.stream_state)
        if self._iterator is None or self._iterator_state != stream.get("dataset_state"):
            self._open(stream.get("dataset_state"))
        pending = list(stream.get("pending_tokens", []))
        docs = int(stream.get("documents_consumed", 0))
        need = self.batch_size * (self.seq_len + 1)
        while len(pending) < need:
            try:
                row = next(self._iterator)
            except StopIteration as exc:
                raise StopIteration("the streaming dataset ended before one full batch was available") from exc
            text = row.get(self.spec.text_column) if isinstance(row, Mapping) else None
            docs += 1
            if not isinstance(text, str) or not text:
                continue
            ids = list(self.tokenizer.encode(text))
            if self.spec.append_eot:
                ids.append(int(self.tokenizer.eot_id))
            pending.extend(ids)
        tokens = np.asarray(pending[:need], dtype=np.int32).reshape(self.batch_size, self.seq_len + 1)
        rest = pending[need:]
        dataset_state = self._dataset.state_dict() if hasattr(self._dataset, "state_dict") else None
        self._iterator_state = dataset_state
        nxt = state.next_record_index + self.batch_size
        new_state = self._state(nxt, {"dataset_state": dataset_state, "pending_tokens": rest,
                                      "documents_consumed": docs})
        batch = Batch(input_ids=tokens[:, :-1].copy(), target_ids=tokens[:, 1:].copy(),
                      loss_mask=np.ones((self.batch_size, self.seq_len), dtype=np.bool_))
        start = state.next_record_index * self.seq_len
        return PipelineBatch(batch, new_state, BatchProvenance(
            split=self.spec.split, epoch=0, token_start=start, token_end=start + self.batch_size * self.seq_len,
            examples=self.batch_size, target_tokens=self.batch_size * self.seq_len,
            row_start_offsets=tuple(start + i * self.seq_len for i in range(self.batch_size))))

    def state_to_json(self, state: DataPipelineState) -> dict[str, Any]:
        return data_pipeline_state_to_dict(state)

    def state_from_json(self, raw: Mapping[str, Any]) -> DataPipelineState:
        state = data_pipeline_state_from_mapping({**raw, "num_records": raw.get("num_records", -1)})
        if state.backend != STREAM_BACKEND or state.seq_len != self.seq_len or state.batch_size != self.batch_size:
            raise ContractError("streaming data pipeline state does not match this pipeline")
        return state

    def describe(self) -> dict[str, Any]:
        return normalize({"schema_version": 1, "backend": STREAM_BACKEND, "backend_version": backend_version(),
                          "state_schema_version": STATE_SCHEMA_VERSION, "split": self.spec.split,
                          "order": "sequential", "shuffle": False, "shuffle_seed": None, "batch_size": self.batch_size,
                          "seq_len": self.seq_len, "num_records": None, "manifest_path": None,
                          "tokenizer_id": self.tokenizer_id, "dataset": self.spec.dataset,
                          "revision": self.spec.revision, "text_column": self.spec.text_column,
                          "append_eot": self.spec.append_eot, "document_aware": False,
                          "source_summary": self.source_summary, "sampler_summary": self.sampler_summary})

    def close(self) -> None:
        self._iterator = None
        self._dataset = None


def build_hf_streaming_pipeline(data: DataSpec, *, seq_len: int, batch_size: int, **kwargs) -> HFStreamingTextPipeline:
    return HFStreamingTextPipeline(data, seq_len=seq_len, batch_size=batch_size, **kwargs)
