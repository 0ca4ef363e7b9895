"""Cross-section validation of a resolved run spec (reference: src/jaxtitan/config/validate.py:10-115)."""

from __future__ import annotations

import math

from research_b200.config.specs import RunSpec, resolve_expert_fsdp_axis, resolve_expert_parallel_axis
from research_b200.errors import ConfigError


def _divisible(label: str, value: int, axis: str, size: int) -> None:
    if value % size != 0:
        raise ConfigError(f"{label} ({value}) must be divisible by {axis} axis size ({size})")


def validate_run_spec(spec: RunSpec) -> None:
    model, training, par = spec.model, spec.training, spec.parallelism
    if model.max_seq_len < training.seq_len:
        raise ConfigError(
            f"model.max_seq_len ({model.max_seq_len}) must be >= training.seq_len ({training.seq_len})"
        )
    effective_batch_tokens = training.global_batch_size * training.seq_len * training.gradient_accumulation_steps
    if training.target_tokens < effective_batch_tokens:
        raise ConfigError("training.target_tokens must cover at least one effective optimizer batch")
    if spec.optimizer.grad_clip_norm is not None and training.grad_clip_norm is not None:
        raise ConfigError("set grad_clip_norm in either [optimizer] or [training], not both")
    sizes = spec.mesh.sizes
    data_size = sizes.get("data", 1)
    if training.global_batch_size % data_size != 0:
        raise ConfigError(
            f"training.global_batch_size ({training.global_batch_size}) must be divisible by "
            f"the data axis size ({data_size})"
        )
    fsdp, ep, tp, cp, efsdp = (sizes.get(k, 1) for k in ("fsdp", "ep", "tp", "cp", "expert_fsdp"))
    moe = model.trinity.moe if model.trinity is not None else None
    is_moe_model = model.name == "trinity" and moe is not None
    if cp != 1 and not par.context_parallel:
        raise ConfigError("mesh cp axis size greater than 1 requires parallelism.context_parallel=true")
    if par.context_parallel:
        if "cp" not in sizes:
            raise ConfigError("parallelism.context_parallel=true requires a mesh cp axis")
        _divisible("training.seq_len", training.seq_len, "cp", cp)
        if par.context_attention == "ulysses":
            # heads are exchanged for sequence: every cp rank attends with heads / cp heads over the whole sequence
            shard = tp if par.tensor_parallel else 1
            for label, value in (("model.num_heads", model.num_heads),
                                 ("model.n_kv_heads", model.n_kv_heads or model.num_heads)):
                if value % (shard * cp) != 0:
                    raise ConfigError(f"{label} ({value}) must be divisible by tp x cp ({shard * cp}) for "
                                      "parallelism.context_attention='ulysses'")
    if tp != 1 and not par.tensor_parallel:
        raise ConfigError("mesh tp axis size greater than 1 requires parallelism.tensor_parallel=true")
    if par.tensor_parallel:
        if "tp" not in sizes:
            raise ConfigError("parallelism.tensor_parallel=true requires a mesh tp axis")
        for label, value in (
            ("model.hidden_size", model.hidden_size),
            ("model.intermediate_size", model.intermediate_size),
            ("model.vocab_size", model.vocab_size),
            ("model.num_heads", model.num_heads),
            ("model.n_kv_heads", model.n_kv_heads),
            ("training.seq_len", training.seq_len),
        ):
            _divisible(label, value, "tp", tp)
        if moe is not None:
            _divisible("model.trinity.moe.expert_intermediate_size",
                       moe.expert_intermediate_size or model.intermediate_size, "tp", tp)
    if par.mode == "ddp" and fsdp != 1:
        raise ConfigError("parallelism.mode='ddp' requires mesh fsdp axis size to be 1")
    if par.mode in ("zero2", "fsdp") and "fsdp" not in sizes:
        raise ConfigError(f"parallelism.mode='{par.mode}' requires a mesh fsdp axis")
    if "ep" in sizes and ep != 1 and not par.expert_parallel:
        raise ConfigError("mesh ep axis size greater than 1 requires parallelism.expert_parallel=true")
    if efsdp != 1:
        policy = resolve_expert_fsdp_axis(par, sizes)
        if not policy.enabled:
            raise ConfigError("mesh expert_fsdp axis size greater than 1 did not resolve to expert FSDP")
        if not is_moe_model:
            raise ConfigError("mesh expert_fsdp axis size greater than 1 requires a Trinity MoE model")
        _divisible("model.trinity.moe.expert_intermediate_size",
                   moe.expert_intermediate_size or model.intermediate_size, "expert_fsdp", policy.axis_size)
        if spec.optimizer.name == "muon":
            raise ConfigError(
                "optimizer.name='muon' is not supported with expert_fsdp axis size greater than 1; "
                "routed expert matrices are internally sharded and require an exact distributed expert optimizer"
            )
    if par.expert_parallel:
        axis = resolve_expert_parallel_axis(par, sizes)
        if not is_moe_model:
            raise ConfigError("parallelism.expert_parallel=true requires a Trinity MoE model")
        if axis.axis == "data" and efsdp != 1:
            raise ConfigError(
                "parallelism.expert_parallel_axis='data' does not support mesh expert_fsdp axis size greater than 1"
            )
        if moe.num_experts % axis.axis_size != 0:
            raise ConfigError(
                f"model.trinity.moe.num_experts ({moe.num_experts}) must be divisible by "
                f"{axis.axis} axis size ({axis.axis_size})"
            )
    if spec.data.mode == "hf_streaming" and spec.evals and spec.data.validation_manifest is None:
        raise ConfigError("data.validation_manifest is required for evals when data.mode='hf_streaming'")
    if spec.profiling.enabled:
        estimated_steps = math.ceil(training.target_tokens / effective_batch_tokens)
        if spec.profiling.trace_start_step > estimated_steps:
            raise ConfigError(
                "profiling.trace_start_step must be reachable by training.target_tokens; "
                f"trace_start_step={spec.profiling.trace_start_step} estimated_steps={estimated_steps}"
            )
