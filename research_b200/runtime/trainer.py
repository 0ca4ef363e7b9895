"""``Trainer``: everything one rank needs to train from a :class:`RunSpec` - mesh, model, parameter store,
optimizer, data pipelines, train / eval steps - behind the small API the host loop, preflight, the benchmark
and the tests all use.

Build order mirrors the reference's ``_run_training_initialized`` (src/jaxtitan/runtime/training.py:271-346):
schedule steps resolved from ``target_tokens``, data pipeline, mesh, model (seeded), sharding plan, optimizer,
train state, step functions.
"""

from __future__ import annotations

import atexit
import math
import os
import queue
import threading
from dataclasses import replace
from typing import Any

import torch

from research_b200.config.specs import RunSpec
from research_b200.contracts import Batch, RngState, StepMetrics
from research_b200.data.pipeline import DataPipelineState, PipelineBatch, build_prepared_token_pipeline
from research_b200.errors import ContractError
from research_b200.models.build import ModelBuildResult, build_model
from research_b200.optim.build import OptimizerBuildResult, build_optimizer
from research_b200.optim.optimizer import Optimizer
from research_b200.parallel.mesh import MeshContext, build_mesh_context, execution_context_for
from research_b200.config.specs import resolve_expert_parallel_axis
from research_b200.parallel.sharding import ParamStore
from research_b200.steps.eval import EvalStep
from research_b200.steps.moe_balance import init_moe_balance
from research_b200.steps.train import TrainStep


def with_runtime_schedule_steps(spec: RunSpec) -> RunSpec:
    """cosine / wsd schedules without ``total_steps`` get ``ceil(target_tokens / tokens_per_step)``
    (reference: runtime/training.py:653-665)."""

    tokens_per_step = (spec.training.global_batch_size * spec.training.seq_len *
                       spec.training.gradient_accumulation_steps)
    total = math.ceil(spec.training.target_tokens / tokens_per_step)

    def fix(schedule):
        if schedule is None or schedule.name == "constant" or schedule.total_steps is not None:
            return schedule
        return replace(schedule, total_steps=total)

    optimizer = replace(spec.optimizer, schedule=fix(spec.optimizer.schedule),
                        adamw_fallback_schedule=fix(spec.optimizer.adamw_fallback_schedule))
    return replace(spec, optimizer=optimizer)


def compute_dtype_for(spec: RunSpec, device: torch.device) -> torch.dtype:
    """``training.precision`` decides the compute dtype: ``fp32`` -> float32; ``bf16`` / ``mixed_bf16`` ->
    the model's ``compute_dtype`` (bfloat16 by default) with fp32 master weights."""

    if spec.training.precision == "fp32" or spec.model.compute_dtype == "float32":
        return torch.float32
    return torch.bfloat16


class BatchPrefetcher:
    """One worker thread that assembles the microbatches of the coming optimizer steps while the GPU runs the
    current one.  Batch assembly is host work (document packing, token-window gathers in the C++ library) that
    releases the interpreter lock for most of its time; without the thread it sits between two steps.

    Items are ``(microbatches, provenance, pipeline state after them)``; the trainer adopts the state only when
    it consumes an item, so a checkpoint never records batches that were assembled but not trained on.
    """

    def __init__(self, pipeline, state: DataPipelineState, accumulation: int, depth: int = 2):
        self.pipeline, self.accumulation = pipeline, accumulation
        self.queue: queue.Queue = queue.Queue(maxsize=depth)
        self.stop = threading.Event()
        self.thread = threading.Thread(target=self._work, args=(state,), name="batch-prefetch", daemon=True)
        self.thread.start()
        atexit.register(self.close)      # never leave the worker inside native code while the interpreter exits

    def _work(self, state: DataPipelineState) -> None:
        while not self.stop.is_set():
            try:
                batches, prov = [], []
                for _ in range(self.accumulation):
                    pb: PipelineBatch = self.pipeline.next_batch(state)
                    state = pb.state
                    batches.append(pb.batch)
                    prov.append(pb.provenance)
                item = (batches, prov, state)
            except BaseException as exc:  # handed to the consumer, which re-raises it
                item = exc
            while not self.stop.is_set():
                try:
                    self.queue.put(item, timeout=0.1)
                    break
                except queue.Full:
                    continue
            if isinstance(item, BaseException):
                return

    def get(self):
        item = self.queue.get()
        if isinstance(item, BaseException):
            raise item
        return item

    def close(self) -> None:
        self.stop.set()
        self.thread.join(timeout=5.0)
        atexit.unregister(self.close)


class Trainer:
    def __init__(self, spec: RunSpec, *, mesh: MeshContext | None = None, device: torch.device | str | None = None,
                 build_data: bool = True):
        self.spec = spec = with_runtime_schedule_steps(spec)
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        self.mesh = mesh or build_mesh_context(spec.mesh, device=self.device)
        self.execution = execution_context_for(self.mesh, spec.parallelism)
        self.compute_dtype = compute_dtype_for(spec, self.device)
        self.result: ModelBuildResult = build_model(spec.model, seed=spec.seed, execution=self.execution,
                                                    device=self.device)
        self.optimizer_build: OptimizerBuildResult = build_optimizer(spec.optimizer, self.result.metadata,
                                                                     tp_size=self.execution.tp_size)
        ep = resolve_expert_parallel_axis(spec.parallelism, self.mesh.sizes)
        self.store = ParamStore(self.result, self.mesh, mode=spec.parallelism.mode, compute_dtype=self.compute_dtype,
                                backend_of=self.optimizer_build.backend_by_name(), ep_axis=ep.axis,
                                decay_of=self.optimizer_build.weight_decay_by_name(),
                                resident=spec.parallelism.fsdp_resident)
        if not self.store.resident:
            self.result.model.layer_prepare = self.store.acquire_layer
        self.optimizer = Optimizer(self.optimizer_build, self.store)
        self.check_layout_agreement()
        moe = spec.model.trinity.moe if spec.model.trinity is not None else None
        self.moe_balance = init_moe_balance(self.result.model, None if moe is None else moe.balance, store=self.store)
        self.train_step_fn = TrainStep(spec, self.result, self.store, self.optimizer, self.mesh, self.moe_balance)
        self.eval_step_fn = EvalStep(self.result, self.store, self.mesh)
        self.rng = RngState.from_seed(spec.seed)
        self.step = 0
        self.tokens_seen = 0
        self.data = None
        self._data_state: DataPipelineState | None = None
        self._prefetcher: BatchPrefetcher | None = None
        self.prefetch = True
        self.debug_checks = self.device.type == "cuda" and os.environ.get("RESEARCH_B200_DEBUG", "0") == "1"
        self.last_provenance: list[Any] = []
        if build_data:
            self.data = self.build_pipeline("train")
            self.data_state = self.data.initial_state()

    def layout_fingerprint(self) -> int:
        """62 bits of the sha256 over what every rank must agree on before the first collective of a step: the mesh,
        the parameter store's sections (sizes, axes, backends) and, per section, the order in which the optimizer
        reduces over the mesh axes."""

        import hashlib

        from research_b200.config.canonical import canonical_json

        payload = {"mesh": [list(self.mesh.axis_names), list(self.mesh.axis_sizes)], "store": self.store.describe(),
                   "sum_axes": [self.optimizer._sum_axes(sec) for sec in self.store.sections],
                   "routes": [[a.name, a.backend] for a in self.optimizer_build.route_assignments]}
        return int.from_bytes(hashlib.sha256(canonical_json(payload).encode()).digest()[:8], "big") >> 2

    def check_layout_agreement(self) -> None:
        """Every rank must have laid the run out in the same way; a rank that did not would not fail, it would wait
        in a collective that its peers never start.  One small reduction at start-up turns that into an error."""

        if self.mesh.world_size == 1 or not torch.distributed.is_initialized():
            return
        mine = self.layout_fingerprint()
        both = torch.tensor([mine, -mine], dtype=torch.int64, device=self.device)
        torch.distributed.all_reduce(both, op=torch.distributed.ReduceOp.MAX)
        highest, lowest = int(both[0]), -int(both[1])
        if highest != lowest:
            raise ContractError(
                f"rank {self.mesh.rank} laid the run out differently from another rank (layout fingerprint "
                f"{mine:#x}, job-wide {lowest:#x} .. {highest:#x}): the ranks would deadlock in their first step")

    # ---- data --------------------------------------------------------------------------------------
    @property
    def data_state(self) -> DataPipelineState | None:
        """Pipeline state after the last batch handed out (what a checkpoint records)."""

        return self._data_state

    @data_state.setter
    def data_state(self, state: DataPipelineState | None) -> None:
        self.close_prefetcher()          # batches assembled ahead belong to the old position
        self._data_state = state

    def close_prefetcher(self) -> None:
        if self._prefetcher is not None:
            self._prefetcher.close()
            self._prefetcher = None

    def build_pipeline(self, split: str):
        d, t = self.spec.data, self.spec.training
        if d.mode != "prepared":
            from research_b200.data.streaming import build_hf_streaming_pipeline

            if split == "train":
                return build_hf_streaming_pipeline(d, seq_len=t.seq_len, batch_size=t.global_batch_size)
        manifest = d.train_manifest if (split == "train" or d.validation_manifest is None) else d.validation_manifest
        if manifest is None:
            raise ContractError("a prepared manifest is required for this split")
        order = d.order if split == "train" else "sequential"
        pipeline = build_prepared_token_pipeline(
            manifest, tokenizer_id=d.tokenizer_id, split=split, seq_len=t.seq_len, batch_size=t.global_batch_size,
            order=order, shuffle_seed=d.shuffle_seed if split == "train" else None,
            document_buffer_size=d.document_buffer_size if split == "train" else None,
            document_refill_size=d.document_refill_size if split == "train" else None)
        if split == "train" and self.mesh.world_size > 1 and hasattr(pipeline, "set_local_rows"):
            # every rank walks the same sampling sequence but reads only the tokens of its own rows
            from research_b200.steps.train import local_batch_slices

            rows, _ = local_batch_slices(self.mesh, t.global_batch_size, t.seq_len)
            pipeline.set_local_rows(range(rows.start, rows.stop))
        return pipeline

    def next_accumulated_batch(self) -> list[Batch]:
        """The microbatches of one optimizer step (reference: runtime/training.py:744-757)."""

        if self.data is None or self.data_state is None:
            raise ContractError("this trainer was built without a data pipeline")
        accumulation = self.spec.training.gradient_accumulation_steps
        if self.prefetch:
            if self._prefetcher is None:
                self._prefetcher = BatchPrefetcher(self.data, self._data_state, accumulation)
            try:
                batches, prov, state = self._prefetcher.get()
            except StopIteration as exc:
                self.close_prefetcher()
                raise ContractError(f"training data exhausted before target_tokens was reached: {exc}") from exc
            except BaseException:
                self.close_prefetcher()
                raise
            self._data_state = state
            self.last_provenance = prov
            return batches
        batches, prov = [], []
        for _ in range(accumulation):
            try:
                pb: PipelineBatch = self.data.next_batch(self.data_state)
            except StopIteration as exc:
                raise ContractError(f"training data exhausted before target_tokens was reached: {exc}") from exc
            self._data_state = pb.state
            batches.append(pb.batch)
            prov.append(pb.provenance)
        self.last_provenance = prov
        return batches

    # ---- steps -------------------------------------------------------------------------------------
    def train_on(self, batches: list[Batch], *, diagnostics: bool = False) -> StepMetrics:
        metrics = self.train_step_fn.run(batches, diagnostics=diagnostics)
        if self.debug_checks:
            # guard words behind every peer-memory buffer, and the kernels' status word (bounded waits that gave up)
            from research_b200.ops import native
            from research_b200.parallel.symmetric import check_all_canaries

            check_all_canaries()
            native.check_status()
        self.step += 1
        self.tokens_seen += sum(int(b.input_ids.shape[0] * b.input_ids.shape[1]) for b in batches)
        return metrics

    def train_step(self, *, diagnostics: bool = False) -> StepMetrics:
        """Public one-call step: pull the next microbatches from the data pipeline and train on them."""

        return self.train_on(self.next_accumulated_batch(), diagnostics=diagnostics)

    def evaluate(self, num_batches: int) -> dict[str, float]:
        """Validation loss over ``num_batches`` batches; with a prepared dataset also bits per byte
        (``loss_sum / (ln 2 * bytes of the scored target tokens)``, tokenizer-independent; reference:
        src/research/evals.py)."""

        import numpy as np

        pipeline = self.build_pipeline("val")
        state = pipeline.initial_state()
        loss_sum = token_count = 0.0
        byte_count = 0
        token_bytes = None
        manifest = getattr(pipeline, "manifest", None)
        if manifest is not None and getattr(manifest, "token_bytes_path", None) is not None:
            path = manifest.manifest_path.parent / manifest.token_bytes_path
            if path.is_file():
                token_bytes = np.fromfile(path, dtype="<u2")
        done = 0
        token_start = token_end = None
        examples = target_tokens = 0
        doc_ids: list[int] = []
        document_aware = True
        self.result.model.eval()
        try:
            for _ in range(num_batches):
                try:
                    pb = pipeline.next_batch(state)
                except StopIteration:
                    break
                state = pb.state
                prov = getattr(pb, "provenance", None)
                if prov is not None:
                    token_start = prov.token_start if token_start is None else token_start
                    token_end = prov.token_end
                    examples += prov.examples
                    target_tokens += prov.target_tokens
                    if prov.row_doc_ids is None:
                        document_aware = False
                    else:
                        doc_ids.extend(prov.row_doc_ids)
                else:
                    document_aware = False
                    examples += int(pb.batch.input_ids.shape[0])
                    target_tokens += int(pb.batch.input_ids.shape[0] * pb.batch.input_ids.shape[1])
                m = self.eval_step_fn.run(pb.batch)
                loss_sum += m.loss_sum
                token_count += m.token_count
                if token_bytes is not None:
                    targets = np.asarray(pb.batch.target_ids)
                    mask = np.asarray(pb.batch.loss_mask) > 0
                    byte_count += int(token_bytes[np.minimum(targets, len(token_bytes) - 1)][mask].sum())
                done += 1
        finally:
            self.result.model.train()
            pipeline.close()
        if done == 0:
            raise ContractError("validation split has no full batch")
        out = {"loss_sum": loss_sum, "token_count": token_count, "loss": loss_sum / max(token_count, 1.0),
               "num_batches": done, "token_start": token_start, "token_end": token_end, "examples": examples,
               "target_tokens": target_tokens, "document_aware": document_aware,
               "documents_touched": len(set(doc_ids)) if document_aware else None,
               "document_min": min(doc_ids) if document_aware and doc_ids else None,
               "document_max": max(doc_ids) if document_aware and doc_ids else None}
        if byte_count > 0:
            out["byte_count"] = byte_count
            out["bpb"] = loss_sum / (math.log(2.0) * byte_count)
        return out

    def close(self) -> None:
        """Stop the prefetch thread and give back the symmetric device memory of this trainer (collective when the
        parameter store uses peer memory: every rank calls it)."""

        self.close_prefetcher()
        from research_b200.parallel import symmetric

        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
            symmetric.close_all_arenas()

    @property
    def is_writer(self) -> bool:
        return self.mesh.rank == 0

    def parameter_count(self) -> int:
        return self.result.parameter_count()
