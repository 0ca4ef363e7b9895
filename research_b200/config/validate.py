"""Cross-section validation of a resolved run spec.

The checks and their messages are the reference's contract (src/jaxtitan/config/validate.py:10-115): the first rule
that fails decides the error a user sees, so the table below is ordered.  A rule is ``(applies, message)``: both are
functions of :class:`Facts`, a flat view of the spec with the derived quantities (axis sizes, the resolved expert
axes, the effective batch) computed once and lazily.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from functools import cached_property
from typing import Callable

from research_b200.config.specs import RunSpec, resolve_expert_fsdp_axis, resolve_expert_parallel_axis
from research_b200.errors import ConfigError


@dataclass
class Facts:
    spec: RunSpec

    def size(self, axis: str) -> int:
        return self.spec.mesh.sizes.get(axis, 1)

    def has(self, axis: str) -> bool:
        return axis in self.spec.mesh.sizes

    @property
    def model(self):
        return self.spec.model

    @property
    def training(self):
        return self.spec.training

    @property
    def par(self):
        return self.spec.parallelism

    @cached_property
    def moe(self):
        return self.model.trinity.moe if self.model.trinity is not None else None

    @cached_property
    def is_moe_model(self) -> bool:
        return self.model.name == "trinity" and self.moe is not None

    @cached_property
    def step_tokens(self) -> int:
        t = self.training
        return t.global_batch_size * t.seq_len * t.gradient_accumulation_steps

    @cached_property
    def estimated_steps(self) -> int:
        return math.ceil(self.training.target_tokens / self.step_tokens)

    @cached_property
    def expert_width(self) -> int:
        return self.moe.expert_intermediate_size or self.model.intermediate_size

    @cached_property
    def expert_axis(self):
        return resolve_expert_parallel_axis(self.par, self.spec.mesh.sizes)

    @cached_property
    def expert_fsdp(self):
        return resolve_expert_fsdp_axis(self.par, self.spec.mesh.sizes)

    @cached_property
    def ulysses_head_split(self) -> int:
        return (self.size("tp") if self.par.tensor_parallel else 1) * self.size("cp")


Rule = tuple[Callable[[Facts], bool], Callable[[Facts], str]]


def _indivisible(label: str, value: Callable[[Facts], int], axis: str, *, when: Callable[[Facts], bool],
                 size: Callable[[Facts], int] | None = None) -> Rule:
    """``value`` must be a multiple of the size of ``axis`` whenever ``when`` holds."""

    size = size or (lambda f: f.size(axis))
    return (lambda f: when(f) and value(f) % size(f) != 0,
            lambda f: f"{label} ({value(f)}) must be divisible by {axis} axis size ({size(f)})")


def _ulysses_heads(label: str, value: Callable[[Facts], int]) -> Rule:
    # heads are exchanged for sequence: every cp rank attends with heads / cp heads over the whole sequence
    return (lambda f: f.par.context_parallel and f.par.context_attention == "ulysses"
            and value(f) % f.ulysses_head_split != 0,
            lambda f: f"{label} ({value(f)}) must be divisible by tp x cp ({f.ulysses_head_split}) for "
                      "parallelism.context_attention='ulysses'")


def _tp(f: Facts) -> bool:
    return f.par.tensor_parallel


def _efsdp(f: Facts) -> bool:
    return f.size("expert_fsdp") != 1


def _ep(f: Facts) -> bool:
    return f.par.expert_parallel


RULES: tuple[Rule, ...] = (
    # ---- shapes and batch arithmetic
    (lambda f: f.model.max_seq_len < f.training.seq_len,
     lambda f: f"model.max_seq_len ({f.model.max_seq_len}) must be >= training.seq_len ({f.training.seq_len})"),
    (lambda f: f.training.target_tokens < f.step_tokens,
     lambda f: "training.target_tokens must cover at least one effective optimizer batch"),
    (lambda f: f.spec.optimizer.grad_clip_norm is not None and f.training.grad_clip_norm is not None,
     lambda f: "set grad_clip_norm in either [optimizer] or [training], not both"),
    (lambda f: f.training.global_batch_size % f.size("data") != 0,
     lambda f: f"training.global_batch_size ({f.training.global_batch_size}) must be divisible by "
               f"the data axis size ({f.size('data')})"),
    # ---- context parallelism
    (lambda f: f.size("cp") != 1 and not f.par.context_parallel,
     lambda f: "mesh cp axis size greater than 1 requires parallelism.context_parallel=true"),
    (lambda f: f.par.context_parallel and not f.has("cp"),
     lambda f: "parallelism.context_parallel=true requires a mesh cp axis"),
    _indivisible("training.seq_len", lambda f: f.training.seq_len, "cp", when=lambda f: f.par.context_parallel),
    _ulysses_heads("model.num_heads", lambda f: f.model.num_heads),
    _ulysses_heads("model.n_kv_heads", lambda f: f.model.n_kv_heads or f.model.num_heads),
    # ---- tensor parallelism
    (lambda f: f.size("tp") != 1 and not f.par.tensor_parallel,
     lambda f: "mesh tp axis size greater than 1 requires parallelism.tensor_parallel=true"),
    (lambda f: _tp(f) and not f.has("tp"), lambda f: "parallelism.tensor_parallel=true requires a mesh tp axis"),
    _indivisible("model.hidden_size", lambda f: f.model.hidden_size, "tp", when=_tp),
    _indivisible("model.intermediate_size", lambda f: f.model.intermediate_size, "tp", when=_tp),
    _indivisible("model.vocab_size", lambda f: f.model.vocab_size, "tp", when=_tp),
    _indivisible("model.num_heads", lambda f: f.model.num_heads, "tp", when=_tp),
    _indivisible("model.n_kv_heads", lambda f: f.model.n_kv_heads, "tp", when=_tp),
    _indivisible("training.seq_len", lambda f: f.training.seq_len, "tp", when=_tp),
    _indivisible("model.trinity.moe.expert_intermediate_size", lambda f: f.expert_width, "tp",
                 when=lambda f: _tp(f) and f.moe is not None),
    # ---- state sharding mode against the mesh
    (lambda f: f.par.mode == "ddp" and f.size("fsdp") != 1,
     lambda f: "parallelism.mode='ddp' requires mesh fsdp axis size to be 1"),
    (lambda f: f.par.mode in ("zero2", "fsdp") and not f.has("fsdp"),
     lambda f: f"parallelism.mode='{f.par.mode}' requires a mesh fsdp axis"),
    # ---- experts
    (lambda f: f.has("ep") and f.size("ep") != 1 and not f.par.expert_parallel,
     lambda f: "mesh ep axis size greater than 1 requires parallelism.expert_parallel=true"),
    (lambda f: _efsdp(f) and not f.expert_fsdp.enabled,
     lambda f: "mesh expert_fsdp axis size greater than 1 did not resolve to expert FSDP"),
    (lambda f: _efsdp(f) and not f.is_moe_model,
     lambda f: "mesh expert_fsdp axis size greater than 1 requires a Trinity MoE model"),
    _indivisible("model.trinity.moe.expert_intermediate_size", lambda f: f.expert_width, "expert_fsdp", when=_efsdp,
                 size=lambda f: f.expert_fsdp.axis_size),
    (lambda f: _efsdp(f) and f.spec.optimizer.name == "muon",
     lambda f: "optimizer.name='muon' is not supported with expert_fsdp axis size greater than 1; "
               "routed expert matrices are internally sharded and require an exact distributed expert optimizer"),
    (lambda f: _ep(f) and f.expert_axis is not None and not f.is_moe_model,
     lambda f: "parallelism.expert_parallel=true requires a Trinity MoE model"),
    (lambda f: _ep(f) and f.expert_axis.axis == "data" and _efsdp(f),
     lambda f: "parallelism.expert_parallel_axis='data' does not support mesh expert_fsdp axis size greater than 1"),
    (lambda f: _ep(f) and f.moe.num_experts % f.expert_axis.axis_size != 0,
     lambda f: f"model.trinity.moe.num_experts ({f.moe.num_experts}) must be divisible by "
               f"{f.expert_axis.axis} axis size ({f.expert_axis.axis_size})"),
    # ---- data and profiling
    (lambda f: f.spec.data.mode == "hf_streaming" and bool(f.spec.evals) and f.spec.data.validation_manifest is None,
     lambda f: "data.validation_manifest is required for evals when data.mode='hf_streaming'"),
    (lambda f: f.spec.profiling.enabled and f.spec.profiling.trace_start_step > f.estimated_steps,
     lambda f: "profiling.trace_start_step must be reachable by training.target_tokens; "
               f"trace_start_step={f.spec.profiling.trace_start_step} estimated_steps={f.estimated_steps}"),
)


def validate_run_spec(spec: RunSpec) -> None:
    """Raise :class:`ConfigError` with the message of the first rule of :data:`RULES` that ``spec`` breaks.  Resolving
    the expert axes can itself raise (an axis the mesh does not have): that error passes through unchanged."""

    facts = Facts(spec)
    for broken, message in RULES:
        if broken(facts):
            raise ConfigError(message(facts))
