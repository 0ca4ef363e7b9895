"""TOML run contract: defaults, error strings, canonical JSON, every reference config loads."""

import glob
import json
import os
from pathlib import Path

import pytest

from research_b200.config import (load_config, resolved_config_sha256, run_spec_from_mapping, run_spec_from_resolved,
                                  run_spec_to_json)
from research_b200.errors import ConfigError
from tests.helpers import tiny_raw_config

# the reference checkout, when one sits beside this repository (or where JAXTITAN_REFERENCE points)
_REFERENCE = Path(os.environ.get("JAXTITAN_REFERENCE", Path(__file__).resolve().parents[2] / "reference"))
REFERENCE_CONFIGS = sorted(glob.glob(str(_REFERENCE / "configs" / "jaxtitan" / "*.toml")))


def _raw(**kw):
    return tiny_raw_config(Path("m.json"), **kw)


def test_defaults_and_canonical_json_roundtrip():
    spec = run_spec_from_mapping(_raw())
    assert spec.model.rope_theta == 10000.0 and spec.model.norm_epsilon == 1e-6
    assert spec.parallelism.mode == "ddp" and spec.mesh.axis_names == ("data",)
    assert spec.training.log_every_steps == 1 and spec.kernels.compile == "lazy"
    text = run_spec_to_json(spec)
    assert text == json.dumps(json.loads(text), sort_keys=True, separators=(",", ":"))
    assert run_spec_from_resolved(json.loads(text)) == spec
    assert len(resolved_config_sha256(spec)) == 64


@pytest.mark.skipif(not REFERENCE_CONFIGS, reason="reference configs not mounted")
def test_every_reference_config_loads_and_roundtrips():
    for path in REFERENCE_CONFIGS:
        spec = load_config(path)
        assert run_spec_from_resolved(json.loads(run_spec_to_json(spec))) == spec, path


def test_axis_aliases_are_canonicalised():
    raw = _raw(mesh={"tensor": 2, "context": 1, "expert": 1})
    raw["parallelism"] = {"tensor_parallel": True}
    spec = run_spec_from_mapping(raw)
    assert spec.mesh.axis_names == ("tp", "cp", "ep")


@pytest.mark.parametrize("mutate,message", [
    (lambda r: r.pop("model"), "missing required [model] section"),
    (lambda r: r["run"].update(id=""), "run.id must be a non-empty string"),
    (lambda r: r["model"].update(vocab_size="x"), "model.vocab_size must be an integer"),
    (lambda r: r["model"].update(hidden_size=65), "model.hidden_size must be divisible by model.num_heads, got 65 and 4"),
    (lambda r: r["model"].update(remat="all"), "model.remat must be one of ['block', 'none'], got 'all'"),
    (lambda r: r["optimizer"].update(name="sgd"),
     "optimizer.name must be one of ['adamw', 'aurora', 'muon', 'riemannian_aurora', 'soap'], got 'sgd'"),
    (lambda r: r["optimizer"]["schedule"].update(peak_lr=0), "optimizer.schedule.peak_lr must be positive, got 0.0"),
    (lambda r: r["data"].update(order="random"),
     "data.order must be 'sequential', 'shuffle', or 'document_buffer', got 'random'"),
    (lambda r: r["data"].pop("shuffle_seed"), "data.shuffle_seed is required when data.order='document_buffer'"),
    (lambda r: r["training"].update(target_tokens=1), "training.target_tokens must cover at least one effective optimizer batch"),
    (lambda r: r["training"].update(grad_clip_norm=1.0), "set grad_clip_norm in either [optimizer] or [training], not both"),
    (lambda r: r.update(mesh={"axis_names": ["data"], "axis_sizes": [3]}),
     "training.global_batch_size (4) must be divisible by the data axis size (3)"),
    (lambda r: r.update(mesh={"axis_names": ["tp"], "axis_sizes": [2]}),
     "mesh tp axis size greater than 1 requires parallelism.tensor_parallel=true"),
    (lambda r: r.update(parallelism={"mode": "fsdp"}), "parallelism.mode='fsdp' requires a mesh fsdp axis"),
    (lambda r: r.update(parallelism={"expert_parallel": True}),
     "parallelism.expert_parallel=true requires a mesh ep axis or parallelism.mode='fsdp' with a mesh fsdp axis "
     "for folded expert parallelism"),
    (lambda r: r.update(profiling={"enabled": True, "trace_start_step": 99}),
     "profiling.trace_start_step must be reachable by training.target_tokens; trace_start_step=99 estimated_steps=4"),
    (lambda r: r.update(generation={"max_new_tokens": 0}), "generation.max_new_tokens must be positive, got 0"),
])
def test_error_messages(mutate, message):
    raw = _raw()
    mutate(raw)
    with pytest.raises(ConfigError) as err:
        run_spec_from_mapping(raw)
    assert str(err.value) == message


def test_trinity_moe_section_and_new_keys():
    raw = _raw(kind="trinity")
    raw["model"]["trinity"]["moe"].update(router="softmax", capacity_factor=1.25, aux_loss_coef=0.01)
    raw["model"]["tied_embeddings"] = True
    spec = run_spec_from_mapping(raw)
    moe = spec.model.trinity.moe
    assert moe.expert_intermediate_size == 32 and moe.router == "softmax" and moe.capacity_factor == 1.25
    assert moe.balance.name == "smebu" and spec.model.tied_embeddings


def test_unknown_keys_are_ignored_and_bad_toml_is_reported(tmp_path):
    raw = _raw()
    raw["model"]["not_a_key"] = 1
    run_spec_from_mapping(raw)
    bad = tmp_path / "bad.toml"
    bad.write_text("[run\nid=")
    with pytest.raises(ConfigError, match="failed to parse config"):
        load_config(bad)
    with pytest.raises(ConfigError, match="failed to read config"):
        load_config(tmp_path / "missing.toml")
