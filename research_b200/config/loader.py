"""TOML run contract -> :class:`RunSpec`.

The section and key set, the defaults and the error strings follow the reference loader
(src/jaxtitan/config/load.py:42-448); the mechanism here is one declarative table per section that a
single typed reader walks.  Unknown keys are ignored, as in the reference.
"""

from __future__ import annotations

import tomllib
from collections.abc import Mapping
from pathlib import Path
from typing import Any, Callable

from research_b200.config import specs as S
from research_b200.config.validate import validate_run_spec
from research_b200.errors import ConfigError, ContractError

_MISSING = object()


# -- typed readers -------------------------------------------------------------------------------------
def _str(section: str, key: str, value: Any) -> str:
    if not isinstance(value, str) or not value:
        raise ConfigError(f"{section}.{key} must be a non-empty string")
    return value


def _int(section: str, key: str, value: Any) -> int:
    if not isinstance(value, int) or isinstance(value, bool):
        raise ConfigError(f"{section}.{key} must be an integer")
    return value


def _loose_int(section: str, key: str, value: Any) -> int:
    # reference quirk: required integers accept TOML booleans (isinstance(True, int))
    if not isinstance(value, int):
        raise ConfigError(f"{section}.{key} must be an integer")
    return value


def _num(section: str, key: str, value: Any) -> float:
    if not isinstance(value, (int, float)) or isinstance(value, bool):
        raise ConfigError(f"{section}.{key} must be numeric")
    return float(value)


def _loose_num(section: str, key: str, value: Any) -> float:
    if not isinstance(value, (int, float)):
        raise ConfigError(f"{section}.{key} must be numeric")
    return float(value)


def _bool(section: str, key: str, value: Any) -> bool:
    if not isinstance(value, bool):
        raise ConfigError(f"{section}.{key} must be a boolean")
    return value


def _path(section: str, key: str, value: Any) -> Path:
    return Path(_str(section, key, value))


def _coerce_int(section: str, key: str, value: Any) -> int:
    return int(value)


def _coerce_float(section: str, key: str, value: Any) -> float:
    return float(value)


def _str_list(section: str, key: str, value: Any) -> tuple[str, ...]:
    if not isinstance(value, list):
        raise ConfigError(f"{section}.{key} must be a list of strings")
    for idx, item in enumerate(value):
        if not isinstance(item, str) or not item:
            raise ConfigError(f"{section}.{key}[{idx}] must be a non-empty string")
    return tuple(value)


Reader = Callable[[str, str, Any], Any]
# (key, reader, default) ; default _MISSING = required ; default None = optional-without-default
Field = tuple[str, Reader, Any]


def _read(raw: Mapping[str, Any], section: str, fields: tuple[Field, ...]) -> dict[str, Any]:
    out: dict[str, Any] = {}
    for key, reader, default in fields:
        if default is _MISSING:
            out[key] = reader(section, key, raw.get(key))
            continue
        value = raw.get(key, default)
        out[key] = None if value is None else reader(section, key, value)
    return out


def _table(value: Any, name: str) -> Mapping[str, Any]:
    if not isinstance(value, Mapping):
        raise ConfigError(f"[{name}] must be a TOML table")
    return value


def _required_table(raw: Mapping[str, Any], key: str) -> Mapping[str, Any]:
    if key not in raw:
        raise ConfigError(f"missing required [{key}] section")
    return _table(raw[key], key)


# -- section tables -----------------------------------------------------------------------------------
RUN_FIELDS: tuple[Field, ...] = (
    ("id", _str, _MISSING),
    ("seed", _coerce_int, 0),
    ("output_dir", _path, "runs"),
)
MODEL_FIELDS: tuple[Field, ...] = (
    ("name", _str, _MISSING),
    ("variant", _str, _MISSING),
    ("vocab_size", _loose_int, _MISSING),
    ("hidden_size", _loose_int, _MISSING),
    ("intermediate_size", _loose_int, _MISSING),
    ("num_layers", _loose_int, _MISSING),
    ("num_heads", _loose_int, _MISSING),
    ("max_seq_len", _loose_int, _MISSING),
    ("n_kv_heads", _int, None),
    ("rope_theta", _num, 1_000_000.0),
    ("norm_epsilon", _num, 1e-6),
    ("tied_embeddings", _bool, False),
    ("param_dtype", _str, "float32"),
    ("compute_dtype", _str, "bfloat16"),
    ("remat", _str, "none"),
    ("init", _str, "nnx_default"),
    ("qk_norm", _bool, True),
    ("attention_doc_mask", _bool, False),
)
TRINITY_FIELDS: tuple[Field, ...] = (
    ("initial_dense_layers", _loose_int, _MISSING),
    ("local_window", _loose_int, _MISSING),
    ("local_layers_per_global", _loose_int, _MISSING),
    ("attention_gate", _bool, True),
    ("qk_norm", _bool, True),
    ("norm_policy", _str, "depth_scaled_sandwich"),
    ("embedding_scale", _str, "sqrt_hidden"),
    ("init_std", _num, None),
)
MOE_FIELDS: tuple[Field, ...] = (
    ("num_experts", _loose_int, _MISSING),
    ("top_k", _loose_int, _MISSING),
    ("expert_intermediate_size", _int, None),
    ("num_shared_experts", _int, 0),
    ("route_scale", _num, 1.0),
    ("router", _str, "sigmoid"),
    ("capacity_factor", _num, None),
    ("aux_loss_coef", _num, 0.0),
)
BALANCE_FIELDS: tuple[Field, ...] = (
    ("name", _str, "none"),
    ("load_lr", _num, 5e-4),
    ("momentum", _num, 0.5),
    ("clamp", _num, 2.0),
    ("sequence_aux_loss_weight", _num, 1e-4),
)
OPTIMIZER_FIELDS: tuple[Field, ...] = (
    ("name", _str, _MISSING),
    ("weight_decay", _coerce_float, 0.0),
    ("grad_clip_norm", _num, None),
    ("muon_tp_mode", _str, "duplicated"),
)
SCHEDULE_FIELDS: tuple[Field, ...] = (
    ("peak_lr", _loose_num, _MISSING),
    ("name", _str, "constant"),
    ("warmup_steps", _coerce_int, 0),
    ("total_steps", _int, None),
    ("min_lr_ratio", _coerce_float, 0.0),
    ("stable_steps", _int, None),
)
DATA_FIELDS: tuple[Field, ...] = (
    ("mode", _str, "prepared"),
    ("train_manifest", _path, None),
    ("tokenizer_id", _str, None),
    ("validation_manifest", _path, None),
    ("order", _str, "sequential"),
    ("shuffle_seed", _int, None),
    ("worker_count", _int, 0),
    ("worker_buffer_size", _int, 1),
    ("prefetch", _bool, False),
    ("document_buffer_size", _int, None),
    ("document_refill_size", _int, None),
)
HF_STREAMING_FIELDS: tuple[Field, ...] = (
    ("dataset", _str, _MISSING),
    ("split", _str, _MISSING),
    ("revision", _str, _MISSING),
    ("name", _str, None),
    ("data_dir", _str, None),
    ("text_column", _str, "text"),
    ("append_eot", _bool, True),
)
TRAINING_FIELDS: tuple[Field, ...] = (
    ("seq_len", _loose_int, _MISSING),
    ("global_batch_size", _loose_int, _MISSING),
    ("target_tokens", _loose_int, _MISSING),
    ("precision", _str, "bf16"),
    ("gradient_accumulation_steps", _coerce_int, 1),
    ("log_every_steps", _coerce_int, 10),
    ("checkpoint_every_steps", _coerce_int, 1000),
    ("eval_every_steps", _int, None),
    ("grad_clip_norm", _num, None),
)
LOSS_FIELDS: tuple[Field, ...] = (("z_loss_weight", _num, 0.0),)
PARALLELISM_FIELDS: tuple[Field, ...] = (
    ("mode", _str, "ddp"),
    ("tensor_parallel", _bool, False),
    ("context_parallel", _bool, False),
    ("expert_parallel", _bool, False),
    ("expert_parallel_axis", _str, "auto"),
    ("context_attention", _str, "gather"),
    ("fsdp_resident", _bool, True),
    ("vocab_parallel_head", _bool, False),
)
ARTIFACT_FIELDS: tuple[Field, ...] = (
    ("wandb_enabled", _bool, False),
    ("wandb_project", _str, "jaxtitan"),
    ("wandb_entity", _str, None),
    ("wandb_group", _str, None),
    ("wandb_tags", _str_list, []),
    ("wandb_mode", _str, "online"),
)
PROFILING_FIELDS: tuple[Field, ...] = (
    ("enabled", _bool, False),
    ("trace_start_step", _int, 3),
    ("trace_steps", _int, 2),
    ("create_perfetto_trace", _bool, True),
    ("create_perfetto_link", _bool, False),
)
KERNEL_FIELDS: tuple[Field, ...] = (
    ("enabled", _bool, False),
    ("strict", _bool, False),
    ("compile", _str, "lazy"),
)
EVAL_FIELDS: tuple[Field, ...] = (
    ("name", _str, _MISSING),
    ("every_steps", _loose_int, _MISSING),
    ("num_batches", _loose_int, _MISSING),
)
GENERATION_FIELDS: tuple[Field, ...] = (
    ("max_new_tokens", _loose_int, _MISSING),
    ("temperature", _coerce_float, 1.0),
    ("top_k", _int, None),
    ("top_p", _num, None),
    ("page_size", _int, 128),
)


def load_config(path: str | Path) -> S.RunSpec:
    """Read a TOML run config and resolve it into a validated :class:`RunSpec`."""

    config_path = Path(path)
    try:
        with config_path.open("rb") as handle:
            raw = tomllib.load(handle)
    except OSError as exc:
        raise ConfigError(f"failed to read config {config_path}: {exc}") from exc
    except tomllib.TOMLDecodeError as exc:
        raise ConfigError(f"failed to parse config {config_path}: {exc}") from exc
    return run_spec_from_mapping(raw)


def _model_spec(raw: Mapping[str, Any]) -> S.ModelSpec:
    model = _read(raw, "model", MODEL_FIELDS)
    trinity_raw = raw.get("trinity")
    if trinity_raw is not None:
        trinity_raw = _table(trinity_raw, "model.trinity")
        trinity = _read(trinity_raw, "model.trinity", TRINITY_FIELDS)
        moe_raw = trinity_raw.get("moe")
        if moe_raw is not None:
            moe_raw = _table(moe_raw, "model.trinity.moe")
            route_scale = moe_raw.get("route_scale", 1.0)
            if not isinstance(route_scale, (int, float)) or isinstance(route_scale, bool):
                raise ConfigError("model.trinity.moe.route_scale must be numeric")
            moe = _read(moe_raw, "model.trinity.moe", MOE_FIELDS)
            balance = _read(_table(moe_raw.get("balance", {}), "model.trinity.moe.balance"),
                            "model.trinity.moe.balance", BALANCE_FIELDS)
            moe["balance"] = S.MoeBalanceSpec(**balance)
            trinity["moe"] = S.TrinityMoeSpec(**moe)
        model["trinity"] = S.TrinitySpec(**trinity)
    return S.ModelSpec(**model)


def _optimizer_spec(raw: Mapping[str, Any]) -> S.OptimizerSpec:
    fields = _read(raw, "optimizer", OPTIMIZER_FIELDS)
    schedule = S.ScheduleSpec(**_read(_required_table(raw, "schedule"), "optimizer.schedule", SCHEDULE_FIELDS))
    fallback_raw = raw.get("adamw_fallback_schedule")
    fallback = None
    if fallback_raw is not None:
        fallback = S.ScheduleSpec(
            **_read(_table(fallback_raw, "optimizer.adamw_fallback_schedule"), "optimizer.schedule", SCHEDULE_FIELDS)
        )
    return S.OptimizerSpec(schedule=schedule, adamw_fallback_schedule=fallback, **fields)


def _data_spec(raw: Mapping[str, Any]) -> S.DataSpec:
    fields = _read(raw, "data", DATA_FIELDS)
    streaming_raw = raw.get("hf_streaming")
    streaming = None
    if streaming_raw is not None:
        streaming = S.HFStreamingSpec(
            **_read(_table(streaming_raw, "data.hf_streaming"), "data.hf_streaming", HF_STREAMING_FIELDS)
        )
    return S.DataSpec(hf_streaming=streaming, **fields)


def run_spec_from_mapping(raw: Mapping[str, Any]) -> S.RunSpec:
    """Resolve a TOML-like mapping into a validated :class:`RunSpec`."""

    try:
        run = _read(_required_table(raw, "run"), "run", RUN_FIELDS)
        model = _model_spec(_required_table(raw, "model"))
        optimizer = _optimizer_spec(_required_table(raw, "optimizer"))
        data = _data_spec(_required_table(raw, "data"))
        training_raw = _required_table(raw, "training")
        training = _read(training_raw, "training", TRAINING_FIELDS)
        training["loss"] = S.TrainingLossSpec(
            **_read(_table(training_raw.get("loss", {}), "training.loss"), "training.loss", LOSS_FIELDS)
        )
        mesh_raw = _table(raw.get("mesh", {}), "mesh")
        mesh = S.MeshSpec(
            axis_names=tuple(mesh_raw.get("axis_names", ("data",))),
            axis_sizes=tuple(int(size) for size in mesh_raw.get("axis_sizes", (1,))),
        )
        evals_raw = raw.get("evals", [])
        if not isinstance(evals_raw, list):
            raise ConfigError("evals must be an array of TOML tables")
        generation_raw = raw.get("generation")
        spec = S.RunSpec(
            run_id=run["id"],
            seed=run["seed"],
            output_dir=run["output_dir"],
            model=model,
            optimizer=optimizer,
            data=data,
            mesh=mesh,
            training=S.TrainingSpec(**training),
            parallelism=S.ParallelismSpec(**_read(_table(raw.get("parallelism", {}), "parallelism"), "parallelism",
                                                  PARALLELISM_FIELDS)),
            artifacts=S.ArtifactSpec(root=run["output_dir"], **_read(_table(raw.get("artifacts", {}), "artifacts"),
                                                                     "artifacts", ARTIFACT_FIELDS)),
            profiling=S.ProfilingSpec(**_read(_table(raw.get("profiling", {}), "profiling"), "profiling",
                                              PROFILING_FIELDS)),
            kernels=S.KernelSpec(**_read(_table(raw.get("kernels", {}), "kernels"), "kernels", KERNEL_FIELDS)),
            evals=tuple(S.EvalSpec(**_read(_table(item, "evals[]"), "evals[]", EVAL_FIELDS)) for item in evals_raw),
            generation=None if generation_raw is None else S.GenerationSpec(
                **_read(_table(generation_raw, "generation"), "generation", GENERATION_FIELDS)),
        )
        validate_run_spec(spec)
    except ContractError as exc:
        raise ConfigError(str(exc)) from exc
    return spec
