"""Canonical JSON of a run spec, its sha256, and reloading a spec from ``config/resolved.json``.

Canonical form = ``json.dumps(sort_keys=True, separators=(",", ":"))`` over the dataclass tree with paths
as POSIX strings (reference: src/jaxtitan/config/serialize.py:18-27, config/resolved.py:20-74).
"""

from __future__ import annotations

import json
from dataclasses import asdict, is_dataclass
from hashlib import sha256
from pathlib import Path
from typing import Any, Mapping

from research_b200.config import specs as S
from research_b200.config.validate import validate_run_spec
from research_b200.errors import ConfigError, ContractError


def normalize(value: Any) -> Any:
    if isinstance(value, Path):
        return value.as_posix()
    if is_dataclass(value) and not isinstance(value, type):
        return normalize(asdict(value))
    if isinstance(value, Mapping):
        return {str(k): normalize(v) for k, v in value.items()}
    if isinstance(value, (tuple, list)):
        return [normalize(v) for v in value]
    return value


def canonical_json(value: Any) -> str:
    return json.dumps(normalize(value), sort_keys=True, separators=(",", ":"))


def run_spec_to_dict(spec: S.RunSpec) -> dict[str, Any]:
    return normalize(asdict(spec))


def run_spec_to_json(spec: S.RunSpec) -> str:
    return canonical_json(run_spec_to_dict(spec))


def resolved_config_sha256(spec: S.RunSpec) -> str:
    return sha256(run_spec_to_json(spec).encode("utf-8")).hexdigest()


def source_config_sha256(path: str | Path) -> str:
    return sha256(Path(path).read_bytes()).hexdigest()


def run_spec_from_resolved(raw: Mapping[str, Any]) -> S.RunSpec:
    """Rebuild a RunSpec from the dictionary form written to ``config/resolved.json``."""

    try:
        model_raw = dict(raw["model"])
        trinity_raw = model_raw.pop("trinity", None)
        if trinity_raw is not None:
            trinity_raw = dict(trinity_raw)
            moe_raw = trinity_raw.pop("moe", None)
            if moe_raw is not None:
                moe_raw = dict(moe_raw)
                moe_raw["balance"] = S.MoeBalanceSpec(**moe_raw.get("balance", {}))
                trinity_raw["moe"] = S.TrinityMoeSpec(**moe_raw)
            model_raw["trinity"] = S.TrinitySpec(**trinity_raw)
        opt_raw = dict(raw["optimizer"])
        opt_raw["schedule"] = S.ScheduleSpec(**opt_raw["schedule"])
        if opt_raw.get("adamw_fallback_schedule") is not None:
            opt_raw["adamw_fallback_schedule"] = S.ScheduleSpec(**opt_raw["adamw_fallback_schedule"])
        opt_raw["route_rules"] = tuple(S.ParamRouteRule(**r) for r in opt_raw.get("route_rules", ()))
        data_raw = dict(raw["data"])
        if data_raw.get("hf_streaming") is not None:
            data_raw["hf_streaming"] = S.HFStreamingSpec(**data_raw["hf_streaming"])
        training_raw = dict(raw["training"])
        training_raw["loss"] = S.TrainingLossSpec(**training_raw.get("loss", {}))
        spec = S.RunSpec(
            run_id=raw["run_id"],
            seed=raw["seed"],
            output_dir=Path(raw["output_dir"]),
            model=S.ModelSpec(**model_raw),
            optimizer=S.OptimizerSpec(**opt_raw),
            data=S.DataSpec(**data_raw),
            mesh=S.MeshSpec(**raw["mesh"]),
            training=S.TrainingSpec(**training_raw),
            parallelism=S.ParallelismSpec(**raw.get("parallelism", {})),
            artifacts=S.ArtifactSpec(**raw.get("artifacts", {})),
            profiling=S.ProfilingSpec(**raw.get("profiling", {})),
            kernels=S.KernelSpec(**raw.get("kernels", {})),
            evals=tuple(S.EvalSpec(**e) for e in raw.get("evals", ())),
            generation=None if raw.get("generation") is None else S.GenerationSpec(**raw["generation"]),
        )
        validate_run_spec(spec)
    except (KeyError, TypeError) as exc:
        raise ConfigError(f"resolved config is malformed: {exc}") from exc
    except ContractError as exc:
        raise ConfigError(str(exc)) from exc
    return spec


def load_resolved_config(path: str | Path) -> S.RunSpec:
    p = Path(path)
    try:
        raw = json.loads(p.read_text(encoding="utf-8"))
    except OSError as exc:
        raise ConfigError(f"failed to read resolved config {p}: {exc}") from exc
    except json.JSONDecodeError as exc:
        raise ConfigError(f"failed to parse resolved config {p}: {exc}") from exc
    if not isinstance(raw, Mapping):
        raise ConfigError(f"resolved config must be a JSON object: {p}")
    return run_spec_from_resolved(raw)
