"""Frozen, validated run-contract dataclasses.

Same fields, defaults and error messages as the reference's spec layer (src/jaxtitan/specs/model.py,
optimizer.py, data.py, mesh.py, parallelism.py, run.py, eval.py, generation.py), restated over a small
set of shared checkers, plus the keys the B200 build adds (all optional with reference-compatible
defaults): ``model.tied_embeddings`` is honoured, ``model.init``, ``model.qk_norm``,
``model.attention_doc_mask``; ``model.trinity.moe.router`` / ``capacity_factor`` / ``aux_loss_coef``;
``optimizer.name = "dion"``; ``generation.page_size``.
"""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass, field, replace
from pathlib import Path
from typing import Any

from research_b200.errors import ContractError

DTYPE_NAMES = ("bfloat16", "float32")
REMAT_POLICIES = ("block", "none")
INIT_POLICIES = ("nnx_default", "normal_0.02")
TRINITY_NORM_POLICIES = ("afmoe_dual", "depth_scaled_sandwich")
TRINITY_EMBEDDING_SCALES = ("sqrt_hidden",)
MOE_BALANCE_POLICIES = ("none", "smebu")
MOE_ROUTERS = ("sigmoid", "softmax")
SCHEDULE_NAMES = ("constant", "cosine", "wsd")
OPTIMIZER_NAMES = ("adamw", "aurora", "dion", "muon", "riemannian_aurora", "soap")
REFERENCE_OPTIMIZER_NAMES = ("adamw", "aurora", "muon", "riemannian_aurora", "soap")
MUON_TP_MODES = ("distributed", "duplicated")
PARALLELISM_MODES = ("ddp", "fsdp", "zero2")
EXPERT_PARALLEL_AXES = ("auto", "data", "ep", "fsdp")
PRECISION_NAMES = ("bf16", "fp32", "mixed_bf16")

# Long axis spellings (tensor, context, expert) accepted in [mesh].axis_names and mapped to the reference spelling
AXIS_ALIASES = {"tensor": "tp", "context": "cp", "expert": "ep"}
SUPPORTED_AXES = ("data", "fsdp", "tp", "cp", "ep", "expert_fsdp")


def _is_int(v: Any) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _is_num(v: Any) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


def _one_of(label: str, value: Any, allowed: tuple[str, ...]) -> None:
    if value not in allowed:
        raise ContractError(f"{label} must be one of {sorted(allowed)}, got {value!r}")


def _bool(label: str, value: Any) -> None:
    if not isinstance(value, bool):
        raise ContractError(f"{label} must be a boolean")


@dataclass(frozen=True, slots=True)
class MoeBalanceSpec:
    name: str = "none"
    load_lr: float = 5e-4
    momentum: float = 0.5
    clamp: float = 2.0
    sequence_aux_loss_weight: float = 1e-4

    def __post_init__(self) -> None:
        _one_of("model.trinity.moe.balance.name", self.name, MOE_BALANCE_POLICIES)
        for name in ("load_lr", "momentum", "clamp"):
            v = getattr(self, name)
            if not _is_num(v) or v <= 0.0:
                raise ContractError(f"model.trinity.moe.balance.{name} must be positive, got {v!r}")
        v = self.sequence_aux_loss_weight
        if not _is_num(v) or v < 0.0:
            raise ContractError(f"model.trinity.moe.balance.sequence_aux_loss_weight must be non-negative, got {v!r}")


@dataclass(frozen=True, slots=True)
class TrinityMoeSpec:
    num_experts: int
    top_k: int
    expert_intermediate_size: int | None = None
    num_shared_experts: int = 0
    route_scale: float = 1.0
    balance: MoeBalanceSpec | Mapping[str, Any] = MoeBalanceSpec()
    router: str = "sigmoid"
    capacity_factor: float | None = None
    aux_loss_coef: float = 0.0

    def __post_init__(self) -> None:
        if isinstance(self.balance, Mapping):
            object.__setattr__(self, "balance", MoeBalanceSpec(**dict(self.balance)))
        elif not isinstance(self.balance, MoeBalanceSpec):
            raise ContractError("model.trinity.moe.balance must be a MoeBalanceSpec or mapping")
        for name in ("num_experts", "top_k"):
            v = getattr(self, name)
            if not _is_int(v) or v <= 0:
                raise ContractError(f"model.trinity.moe.{name} must be a positive integer, got {v!r}")
        if self.top_k > self.num_experts:
            raise ContractError("model.trinity.moe.top_k must be <= model.trinity.moe.num_experts")
        v = self.expert_intermediate_size
        if v is not None and (not _is_int(v) or v <= 0):
            raise ContractError(f"model.trinity.moe.expert_intermediate_size must be a positive integer, got {v!r}")
        v = self.num_shared_experts
        if not _is_int(v) or v < 0:
            raise ContractError(f"model.trinity.moe.num_shared_experts must be a non-negative integer, got {v!r}")
        if not _is_num(self.route_scale) or self.route_scale <= 0.0:
            raise ContractError(f"model.trinity.moe.route_scale must be positive, got {self.route_scale!r}")
        _one_of("model.trinity.moe.router", self.router, MOE_ROUTERS)
        if self.capacity_factor is not None and (not _is_num(self.capacity_factor) or self.capacity_factor <= 0.0):
            raise ContractError(f"model.trinity.moe.capacity_factor must be positive, got {self.capacity_factor!r}")
        if not _is_num(self.aux_loss_coef) or self.aux_loss_coef < 0.0:
            raise ContractError(f"model.trinity.moe.aux_loss_coef must be non-negative, got {self.aux_loss_coef!r}")


@dataclass(frozen=True, slots=True)
class TrinitySpec:
    initial_dense_layers: int
    local_window: int
    local_layers_per_global: int
    attention_gate: bool = True
    qk_norm: bool = True
    norm_policy: str = "depth_scaled_sandwich"
    embedding_scale: str = "sqrt_hidden"
    init_std: float | None = None
    moe: TrinityMoeSpec | Mapping[str, Any] | None = None

    def __post_init__(self) -> None:
        if isinstance(self.moe, Mapping):
            object.__setattr__(self, "moe", TrinityMoeSpec(**dict(self.moe)))
        elif self.moe is not None and not isinstance(self.moe, TrinityMoeSpec):
            raise ContractError("model.trinity.moe must be a TrinityMoeSpec or mapping")
        for name in ("initial_dense_layers", "local_window", "local_layers_per_global"):
            v = getattr(self, name)
            if not _is_int(v):
                raise ContractError(f"model.trinity.{name} must be an integer, got {v!r}")
            if (v < 0) if name == "initial_dense_layers" else (v <= 0):
                raise ContractError(f"model.trinity.{name} is invalid: {v}")
        _bool("model.trinity.attention_gate", self.attention_gate)
        _bool("model.trinity.qk_norm", self.qk_norm)
        _one_of("model.trinity.norm_policy", self.norm_policy, TRINITY_NORM_POLICIES)
        _one_of("model.trinity.embedding_scale", self.embedding_scale, TRINITY_EMBEDDING_SCALES)
        if self.init_std is not None and self.init_std <= 0.0:
            raise ContractError(f"model.trinity.init_std must be positive, got {self.init_std}")


@dataclass(frozen=True, slots=True)
class ModelSpec:
    name: str
    variant: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_layers: int
    num_heads: int
    max_seq_len: int
    n_kv_heads: int | None = None
    rope_theta: float = 1_000_000.0
    norm_epsilon: float = 1e-6
    tied_embeddings: bool = False
    param_dtype: str = "float32"
    compute_dtype: str = "bfloat16"
    remat: str = "none"
    trinity: TrinitySpec | Mapping[str, Any] | None = None
    init: str = "nnx_default"
    qk_norm: bool = True
    attention_doc_mask: bool = False

    def __post_init__(self) -> None:
        trinity = self.trinity
        if isinstance(trinity, Mapping):
            trinity = TrinitySpec(**dict(trinity))
            object.__setattr__(self, "trinity", trinity)
        elif trinity is not None and not isinstance(trinity, TrinitySpec):
            raise ContractError("model.trinity must be a TrinitySpec or mapping")
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_layers", "num_heads", "max_seq_len"):
            v = getattr(self, name)
            if v <= 0:
                raise ContractError(f"model.{name} must be positive, got {v}")
        for name in ("rope_theta", "norm_epsilon"):
            v = getattr(self, name)
            if v <= 0.0:
                raise ContractError(f"model.{name} must be positive, got {v}")
        _one_of("model.param_dtype", self.param_dtype, DTYPE_NAMES)
        _one_of("model.compute_dtype", self.compute_dtype, DTYPE_NAMES)
        _one_of("model.remat", self.remat, REMAT_POLICIES)
        _one_of("model.init", self.init, INIT_POLICIES)
        _bool("model.tied_embeddings", self.tied_embeddings)
        _bool("model.qk_norm", self.qk_norm)
        _bool("model.attention_doc_mask", self.attention_doc_mask)
        if self.name == "trinity":
            if trinity is None:
                raise ContractError("model.name='trinity' requires [model.trinity]")
            if trinity.moe is not None and trinity.moe.expert_intermediate_size is None:
                trinity = replace(trinity, moe=replace(trinity.moe, expert_intermediate_size=self.intermediate_size))
                object.__setattr__(self, "trinity", trinity)
            if trinity.initial_dense_layers > self.num_layers:
                raise ContractError("model.trinity.initial_dense_layers must be <= model.num_layers")
            if trinity.moe is not None and trinity.initial_dense_layers >= self.num_layers:
                raise ContractError("model.trinity.initial_dense_layers must leave at least one MoE layer")
            if trinity.local_window > self.max_seq_len:
                raise ContractError("model.trinity.local_window must be <= model.max_seq_len")
        elif trinity is not None:
            raise ContractError("[model.trinity] is only valid when model.name='trinity'")
        n_kv = self.num_heads if self.n_kv_heads is None else self.n_kv_heads
        if n_kv <= 0:
            raise ContractError(f"model.n_kv_heads must be positive, got {n_kv}")
        if self.hidden_size % self.num_heads != 0:
            raise ContractError(
                f"model.hidden_size must be divisible by model.num_heads, got {self.hidden_size} and {self.num_heads}"
            )
        if self.num_heads % n_kv != 0:
            raise ContractError(
                f"model.num_heads must be divisible by model.n_kv_heads, got {self.num_heads} and {n_kv}"
            )
        object.__setattr__(self, "n_kv_heads", n_kv)

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads


@dataclass(frozen=True, slots=True)
class ScheduleSpec:
    peak_lr: float
    name: str = "constant"
    warmup_steps: int = 0
    total_steps: int | None = None
    min_lr_ratio: float = 0.0
    stable_steps: int | None = None

    def __post_init__(self) -> None:
        _one_of("optimizer.schedule.name", self.name, SCHEDULE_NAMES)
        if self.peak_lr <= 0:
            raise ContractError(f"optimizer.schedule.peak_lr must be positive, got {self.peak_lr}")
        if self.warmup_steps < 0:
            raise ContractError(f"optimizer.schedule.warmup_steps must be non-negative, got {self.warmup_steps}")
        if self.total_steps is not None and self.total_steps <= 0:
            raise ContractError(f"optimizer.schedule.total_steps must be positive, got {self.total_steps}")
        if not 0.0 <= self.min_lr_ratio <= 1.0:
            raise ContractError(f"optimizer.schedule.min_lr_ratio must be in [0, 1], got {self.min_lr_ratio}")
        if self.stable_steps is not None and self.stable_steps < 0:
            raise ContractError(f"optimizer.schedule.stable_steps must be non-negative, got {self.stable_steps}")


@dataclass(frozen=True, slots=True)
class ParamRouteRule:
    tag: str
    transform: str
    weight_decay: bool = True

    def __post_init__(self) -> None:
        if not self.tag:
            raise ContractError("optimizer route tag must be non-empty")
        if not self.transform:
            raise ContractError("optimizer route transform must be non-empty")


@dataclass(frozen=True, slots=True)
class OptimizerSpec:
    name: str
    schedule: ScheduleSpec
    weight_decay: float = 0.0
    grad_clip_norm: float | None = None
    adamw_fallback_schedule: ScheduleSpec | None = None
    muon_tp_mode: str = "duplicated"
    route_rules: tuple[ParamRouteRule, ...] = ()

    def __post_init__(self) -> None:
        if self.name not in OPTIMIZER_NAMES:
            raise ContractError(
                f"optimizer.name must be one of {sorted(REFERENCE_OPTIMIZER_NAMES)}, got {self.name!r}"
            )
        matrix_optimizer = self.name in ("muon", "dion")
        if not matrix_optimizer and self.adamw_fallback_schedule is not None:
            raise ContractError("optimizer.adamw_fallback_schedule is only supported when optimizer.name is 'muon'")
        _one_of("optimizer.muon_tp_mode", self.muon_tp_mode, MUON_TP_MODES)
        if not matrix_optimizer and self.muon_tp_mode != "duplicated":
            raise ContractError("optimizer.muon_tp_mode is only supported when optimizer.name is 'muon'")
        if self.weight_decay < 0:
            raise ContractError(f"optimizer.weight_decay must be non-negative, got {self.weight_decay}")
        if self.grad_clip_norm is not None and self.grad_clip_norm <= 0:
            raise ContractError(f"optimizer.grad_clip_norm must be positive, got {self.grad_clip_norm}")
        object.__setattr__(self, "route_rules", tuple(self.route_rules))


@dataclass(frozen=True, slots=True)
class HFStreamingSpec:
    dataset: str
    split: str
    revision: str
    name: str | None = None
    data_dir: str | None = None
    text_column: str = "text"
    append_eot: bool = True

    def __post_init__(self) -> None:
        if not self.dataset:
            raise ContractError("data.hf_streaming.dataset must be a non-empty string")
        if not self.split:
            raise ContractError("data.hf_streaming.split must be a non-empty string")
        if not self.revision:
            raise ContractError("data.hf_streaming.revision must be a non-empty pinned revision")
        if self.name is not None and not self.name:
            raise ContractError("data.hf_streaming.name must be non-empty when provided")
        if self.data_dir is not None and not self.data_dir:
            raise ContractError("data.hf_streaming.data_dir must be non-empty when provided")
        if not self.text_column:
            raise ContractError("data.hf_streaming.text_column must be a non-empty string")
        _bool("data.hf_streaming.append_eot", self.append_eot)


@dataclass(frozen=True, slots=True)
class DataSpec:
    mode: str = "prepared"
    train_manifest: Path | None = None
    tokenizer_id: str | None = None
    validation_manifest: Path | None = None
    hf_streaming: HFStreamingSpec | None = None
    order: str = "sequential"
    shuffle_seed: int | None = None
    worker_count: int = 0
    worker_buffer_size: int = 1
    prefetch: bool = False
    document_buffer_size: int | None = None
    document_refill_size: int | None = None

    def __post_init__(self) -> None:
        if self.mode not in ("prepared", "hf_streaming"):
            raise ContractError(f"data.mode must be 'prepared' or 'hf_streaming', got {self.mode!r}")
        streaming = self.mode == "hf_streaming"
        if not streaming:
            if self.train_manifest is None:
                raise ContractError("data.train_manifest is required when data.mode='prepared'")
            object.__setattr__(self, "train_manifest", Path(self.train_manifest))
            if self.hf_streaming is not None:
                raise ContractError("data.hf_streaming is only valid when data.mode='hf_streaming'")
        else:
            if self.train_manifest is not None:
                raise ContractError("data.train_manifest must be omitted when data.mode='hf_streaming'")
            if self.hf_streaming is None:
                raise ContractError("data.hf_streaming is required when data.mode='hf_streaming'")
            if self.tokenizer_id is None:
                raise ContractError("data.tokenizer_id is required when data.mode='hf_streaming'")
        if self.validation_manifest is not None:
            object.__setattr__(self, "validation_manifest", Path(self.validation_manifest))
        if self.tokenizer_id is not None and not self.tokenizer_id:
            raise ContractError("data.tokenizer_id must be non-empty when provided")
        if self.order not in ("sequential", "shuffle", "document_buffer"):
            raise ContractError(
                f"data.order must be 'sequential', 'shuffle', or 'document_buffer', got {self.order!r}"
            )
        plain_workers = self.worker_count == 0 and self.worker_buffer_size == 1 and not self.prefetch
        has_buffer_keys = self.document_buffer_size is not None or self.document_refill_size is not None
        if streaming:
            if self.order != "sequential":
                raise ContractError("data.mode='hf_streaming' supports only data.order='sequential'")
            if self.shuffle_seed is not None:
                raise ContractError("data.shuffle_seed must be null or omitted when data.mode='hf_streaming'")
            if not plain_workers:
                raise ContractError(
                    "data.mode='hf_streaming' requires worker_count=0, worker_buffer_size=1, and prefetch=false"
                )
            if has_buffer_keys:
                raise ContractError("document buffer settings are not supported when data.mode='hf_streaming'")
        if self.order in ("shuffle", "document_buffer") and self.shuffle_seed is None:
            raise ContractError(f"data.shuffle_seed is required when data.order={self.order!r}")
        if self.order == "sequential" and self.shuffle_seed is not None:
            raise ContractError("data.shuffle_seed must be null or omitted when data.order='sequential'")
        if self.shuffle_seed is not None and not _is_int(self.shuffle_seed):
            raise ContractError("data.shuffle_seed must be an integer when provided")
        if not _is_int(self.worker_count):
            raise ContractError("data.worker_count must be an integer")
        if not _is_int(self.worker_buffer_size):
            raise ContractError("data.worker_buffer_size must be an integer")
        _bool("data.prefetch", self.prefetch)
        if self.shuffle_seed is not None and self.shuffle_seed < 0:
            raise ContractError(f"data.shuffle_seed must be non-negative, got {self.shuffle_seed}")
        if self.worker_count < 0:
            raise ContractError(f"data.worker_count must be non-negative, got {self.worker_count}")
        if self.worker_buffer_size <= 0:
            raise ContractError(f"data.worker_buffer_size must be positive, got {self.worker_buffer_size}")
        for name in ("document_buffer_size", "document_refill_size"):
            v = getattr(self, name)
            if v is not None and (not _is_int(v) or v <= 0):
                raise ContractError(f"data.{name} must be a positive integer when provided")
        if self.order == "document_buffer":
            if self.document_buffer_size is None:
                raise ContractError("data.document_buffer_size is required when data.order='document_buffer'")
            if self.document_refill_size is None:
                raise ContractError("data.document_refill_size is required when data.order='document_buffer'")
            if not plain_workers:
                raise ContractError(
                    "data.order='document_buffer' requires worker_count=0, worker_buffer_size=1, and prefetch=false"
                )
        elif has_buffer_keys:
            raise ContractError("document buffer settings require data.order='document_buffer'")


@dataclass(frozen=True, slots=True)
class MeshSpec:
    axis_names: tuple[str, ...] = ("data",)
    axis_sizes: tuple[int, ...] = (1,)

    def __post_init__(self) -> None:
        names = tuple(AXIS_ALIASES.get(n, n) for n in self.axis_names)
        object.__setattr__(self, "axis_names", names)
        object.__setattr__(self, "axis_sizes", tuple(self.axis_sizes))
        if len(self.axis_names) != len(self.axis_sizes):
            raise ContractError("mesh.axis_names and mesh.axis_sizes must have the same length")
        if not self.axis_names:
            raise ContractError("mesh must define at least one axis")
        if len(set(self.axis_names)) != len(self.axis_names):
            raise ContractError(f"mesh axis names must be unique, got {self.axis_names}")
        for n in self.axis_names:
            if not n:
                raise ContractError("mesh axis names must be non-empty")
        for s in self.axis_sizes:
            if s <= 0:
                raise ContractError(f"mesh axis sizes must be positive, got {self.axis_sizes}")

    @property
    def sizes(self) -> dict[str, int]:
        return dict(zip(self.axis_names, self.axis_sizes, strict=True))

    @property
    def device_count(self) -> int:
        n = 1
        for s in self.axis_sizes:
            n *= s
        return n


@dataclass(frozen=True, slots=True)
class ExpertParallelAxisPolicy:
    enabled: bool
    axis: str | None = None
    axis_size: int = 1
    axis_sharing: str | None = None


@dataclass(frozen=True, slots=True)
class ExpertFSDPPolicy:
    enabled: bool
    axis: str | None = None
    axis_size: int = 1
    axis_sharing: str | None = None


@dataclass(frozen=True, slots=True)
class ParallelismSpec:
    mode: str = "ddp"
    tensor_parallel: bool = False
    context_parallel: bool = False
    expert_parallel: bool = False
    expert_parallel_axis: str = "auto"
    context_attention: str = "gather"    # "gather": K/V all-gather; "ulysses": head <-> sequence all-to-all
    # false: with mode="fsdp" the compute copy of the weights is kept only where it is owned and every layer's
    # weights are fetched from their owners right before the layer runs (ZeRO-3); true keeps them on every rank
    fsdp_resident: bool = True
    # true: under tensor parallelism the lm_head is split over the vocabulary (each rank scores its slice of the
    # vocabulary for all tokens; max / sum-exp / target logit are reduced over the group) instead of being kept
    # whole on every rank with the tokens split
    vocab_parallel_head: bool = False

    def __post_init__(self) -> None:
        _one_of("parallelism.mode", self.mode, PARALLELISM_MODES)
        _bool("parallelism.fsdp_resident", self.fsdp_resident)
        _bool("parallelism.vocab_parallel_head", self.vocab_parallel_head)
        if self.vocab_parallel_head and not self.tensor_parallel:
            raise ContractError("parallelism.vocab_parallel_head=true requires parallelism.tensor_parallel=true")
        if not self.fsdp_resident and self.mode != "fsdp":
            raise ContractError("parallelism.fsdp_resident=false requires parallelism.mode='fsdp'")
        _one_of("parallelism.context_attention", self.context_attention, ("gather", "ulysses"))
        _bool("parallelism.tensor_parallel", self.tensor_parallel)
        _bool("parallelism.context_parallel", self.context_parallel)
        _bool("parallelism.expert_parallel", self.expert_parallel)
        _one_of("parallelism.expert_parallel_axis", self.expert_parallel_axis, EXPERT_PARALLEL_AXES)
        if not self.expert_parallel and self.expert_parallel_axis != "auto":
            raise ContractError("parallelism.expert_parallel_axis requires parallelism.expert_parallel=true")


def resolve_expert_parallel_axis(parallelism: ParallelismSpec, axis_sizes: Mapping[str, int]) -> ExpertParallelAxisPolicy:
    """Which mesh axis owns routed experts: dedicated ``ep``, folded onto ``fsdp``, or shared with ``data``
    (reference: specs/parallelism.py:62-112)."""

    if not parallelism.expert_parallel:
        return ExpertParallelAxisPolicy(enabled=False)
    axis = parallelism.expert_parallel_axis
    if axis == "auto":
        if "ep" in axis_sizes:
            axis = "ep"
        elif parallelism.mode == "fsdp" and "fsdp" in axis_sizes:
            axis = "fsdp"
        else:
            raise ContractError(
                "parallelism.expert_parallel=true requires a mesh ep axis or "
                "parallelism.mode='fsdp' with a mesh fsdp axis for folded expert parallelism"
            )
    sharing = {"ep": "dedicated_ep", "data": "shared_with_data", "fsdp": "shared_with_fsdp"}
    if axis == "fsdp" and parallelism.mode != "fsdp":
        raise ContractError("parallelism.expert_parallel_axis='fsdp' requires parallelism.mode='fsdp'")
    if axis not in sharing:
        raise ContractError(f"unsupported expert parallel axis {axis!r}")
    if axis not in axis_sizes:
        raise ContractError(f"parallelism.expert_parallel_axis='{axis}' requires a mesh {axis} axis")
    return ExpertParallelAxisPolicy(True, axis, axis_sizes[axis], sharing[axis])


def resolve_expert_fsdp_axis(parallelism: ParallelismSpec, axis_sizes: Mapping[str, int]) -> ExpertFSDPPolicy:
    """Optional sharding of routed expert matrices over ``expert_fsdp`` (reference: specs/parallelism.py:115-136)."""

    size = axis_sizes.get("expert_fsdp", 1)
    if size == 1:
        return ExpertFSDPPolicy(enabled=False)
    if parallelism.mode != "fsdp":
        raise ContractError("mesh expert_fsdp axis with size > 1 requires parallelism.mode='fsdp'")
    if not parallelism.expert_parallel:
        raise ContractError("mesh expert_fsdp axis with size > 1 requires parallelism.expert_parallel=true")
    if resolve_expert_parallel_axis(parallelism, axis_sizes).axis != "ep":
        raise ContractError("mesh expert_fsdp axis with size > 1 requires a dedicated expert_parallel_axis='ep'")
    return ExpertFSDPPolicy(True, "expert_fsdp", size, "expert_region_internal")


@dataclass(frozen=True, slots=True)
class RunDirs:
    root: Path
    run_id: str

    def __post_init__(self) -> None:
        object.__setattr__(self, "root", Path(self.root))
        if not self.run_id:
            raise ContractError("run_id must be non-empty")

    @property
    def run_dir(self) -> Path:
        return self.root / self.run_id

    @property
    def config_dir(self) -> Path:
        return self.run_dir / "config"

    @property
    def metrics_dir(self) -> Path:
        return self.run_dir / "metrics"

    @property
    def checkpoints_dir(self) -> Path:
        return self.run_dir / "checkpoints"


@dataclass(frozen=True, slots=True)
class ArtifactSpec:
    root: Path = Path("runs")
    wandb_enabled: bool = False
    wandb_project: str = "jaxtitan"
    wandb_entity: str | None = None
    wandb_group: str | None = None
    wandb_tags: tuple[str, ...] = ()
    wandb_mode: str = "online"

    def __post_init__(self) -> None:
        object.__setattr__(self, "root", Path(self.root))
        object.__setattr__(self, "wandb_tags", tuple(self.wandb_tags))
        _bool("artifacts.wandb_enabled", self.wandb_enabled)
        if not isinstance(self.wandb_project, str) or not self.wandb_project:
            raise ContractError("artifacts.wandb_project must be a non-empty string")
        for name in ("wandb_entity", "wandb_group"):
            v = getattr(self, name)
            if v is not None and (not isinstance(v, str) or not v):
                raise ContractError(f"artifacts.{name} must be non-empty when provided")
        if self.wandb_mode not in ("online", "offline"):
            raise ContractError("artifacts.wandb_mode must be 'online' or 'offline'")
        if any(not isinstance(t, str) or not t for t in self.wandb_tags):
            raise ContractError("artifacts.wandb_tags must contain only non-empty strings")


@dataclass(frozen=True, slots=True)
class ProfilingSpec:
    enabled: bool = False
    trace_start_step: int = 3
    trace_steps: int = 2
    create_perfetto_trace: bool = True
    create_perfetto_link: bool = False

    def __post_init__(self) -> None:
        _bool("profiling.enabled", self.enabled)
        for name in ("trace_start_step", "trace_steps"):
            v = getattr(self, name)
            if not _is_int(v):
                raise ContractError(f"profiling.{name} must be an integer")
            if v <= 0:
                raise ContractError(f"profiling.{name} must be positive, got {v}")
        _bool("profiling.create_perfetto_trace", self.create_perfetto_trace)
        _bool("profiling.create_perfetto_link", self.create_perfetto_link)

    @property
    def trace_end_step(self) -> int:
        return self.trace_start_step + self.trace_steps - 1


@dataclass(frozen=True, slots=True)
class KernelSpec:
    enabled: bool = False
    strict: bool = False
    compile: str = "lazy"

    def __post_init__(self) -> None:
        _bool("kernels.enabled", self.enabled)
        _bool("kernels.strict", self.strict)
        if self.compile not in ("lazy", "ahead_of_time"):
            raise ContractError("kernels.compile must be 'lazy' or 'ahead_of_time'")


@dataclass(frozen=True, slots=True)
class TrainingLossSpec:
    z_loss_weight: float = 0.0

    def __post_init__(self) -> None:
        if not _is_num(self.z_loss_weight) or self.z_loss_weight < 0.0:
            raise ContractError(f"training.loss.z_loss_weight must be non-negative, got {self.z_loss_weight!r}")


@dataclass(frozen=True, slots=True)
class TrainingSpec:
    seq_len: int
    global_batch_size: int
    target_tokens: int
    precision: str = "bf16"
    gradient_accumulation_steps: int = 1
    log_every_steps: int = 10
    checkpoint_every_steps: int = 1000
    eval_every_steps: int | None = None
    grad_clip_norm: float | None = None
    loss: TrainingLossSpec = field(default_factory=TrainingLossSpec)

    def __post_init__(self) -> None:
        if isinstance(self.loss, Mapping):
            object.__setattr__(self, "loss", TrainingLossSpec(**self.loss))
        elif not isinstance(self.loss, TrainingLossSpec):
            raise ContractError("training.loss must be a TrainingLossSpec or mapping")
        _one_of("training.precision", self.precision, PRECISION_NAMES)
        for name in ("seq_len", "global_batch_size", "target_tokens", "gradient_accumulation_steps",
                     "log_every_steps", "checkpoint_every_steps"):
            v = getattr(self, name)
            if v <= 0:
                raise ContractError(f"training.{name} must be positive, got {v}")
        if self.eval_every_steps is not None and self.eval_every_steps <= 0:
            raise ContractError(f"training.eval_every_steps must be positive, got {self.eval_every_steps}")
        if self.grad_clip_norm is not None and self.grad_clip_norm <= 0:
            raise ContractError(f"training.grad_clip_norm must be positive, got {self.grad_clip_norm}")


@dataclass(frozen=True, slots=True)
class EvalSpec:
    name: str
    every_steps: int
    num_batches: int

    def __post_init__(self) -> None:
        if not self.name:
            raise ContractError("eval.name must be non-empty")
        if self.every_steps <= 0:
            raise ContractError(f"eval.every_steps must be positive, got {self.every_steps}")
        if self.num_batches <= 0:
            raise ContractError(f"eval.num_batches must be positive, got {self.num_batches}")


@dataclass(frozen=True, slots=True)
class GenerationSpec:
    max_new_tokens: int
    temperature: float = 1.0
    top_k: int | None = None
    top_p: float | None = None
    page_size: int = 128

    def __post_init__(self) -> None:
        if self.max_new_tokens <= 0:
            raise ContractError(f"generation.max_new_tokens must be positive, got {self.max_new_tokens}")
        if self.temperature <= 0:
            raise ContractError(f"generation.temperature must be positive, got {self.temperature}")
        if self.top_k is not None and self.top_k <= 0:
            raise ContractError(f"generation.top_k must be positive, got {self.top_k}")
        if self.top_p is not None and not 0.0 < self.top_p <= 1.0:
            raise ContractError(f"generation.top_p must be in (0, 1], got {self.top_p}")
        if not _is_int(self.page_size) or self.page_size <= 0:
            raise ContractError(f"generation.page_size must be a positive integer, got {self.page_size!r}")


@dataclass(frozen=True, slots=True)
class RunSpec:
    run_id: str
    seed: int
    output_dir: Path
    model: ModelSpec
    optimizer: OptimizerSpec
    data: DataSpec
    mesh: MeshSpec
    training: TrainingSpec
    parallelism: ParallelismSpec = ParallelismSpec()
    artifacts: ArtifactSpec = ArtifactSpec()
    profiling: ProfilingSpec = ProfilingSpec()
    kernels: KernelSpec = KernelSpec()
    evals: tuple[EvalSpec, ...] = ()
    generation: GenerationSpec | None = None

    def __post_init__(self) -> None:
        object.__setattr__(self, "output_dir", Path(self.output_dir))
        object.__setattr__(self, "evals", tuple(self.evals))
        if not self.run_id:
            raise ContractError("run.id must be non-empty")
        if self.seed < 0:
            raise ContractError(f"run.seed must be non-negative, got {self.seed}")

    @property
    def dirs(self) -> RunDirs:
        return RunDirs(root=self.output_dir, run_id=self.run_id)


@dataclass(frozen=True, slots=True)
class RunManifest:
    schema_version: int
    artifact_layout_version: int
    run_id: str
    created_at: str
    source_config_path: Path
    source_config_sha256: str
    resolved_config_sha256: str
    package: dict[str, str]
    directories: dict[str, str]
    run_dir: Path
    data: dict[str, Any] | None = None

    def __post_init__(self) -> None:
        object.__setattr__(self, "source_config_path", Path(self.source_config_path))
        object.__setattr__(self, "run_dir", Path(self.run_dir))
        if self.schema_version <= 0:
            raise ContractError(f"manifest.schema_version must be positive, got {self.schema_version}")
        if self.artifact_layout_version <= 0:
            raise ContractError(
                f"manifest.artifact_layout_version must be positive, got {self.artifact_layout_version}"
            )
        for name in ("run_id", "created_at", "source_config_sha256", "resolved_config_sha256"):
            if not getattr(self, name):
                raise ContractError(f"manifest.{name} must be non-empty")
