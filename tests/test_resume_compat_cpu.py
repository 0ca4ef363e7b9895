"""Resume compatibility: what the fingerprint covers, what may change, and how a mismatch is reported."""

import copy
import types

import pytest

from research_b200.config import run_spec_from_mapping
from research_b200.errors import ContractError
from research_b200.runtime.resume import (RESUME_COMPAT_VERSION, RESUME_METADATA_SCHEMA_VERSION, build_resume_compat,
                                          checkpoint_metadata, validate_resume_compat, validate_resume_metadata)
from tests.helpers import tiny_dataset, tiny_raw_config


@pytest.fixture(scope="module")
def manifest(tmp_path_factory):
    return tiny_dataset(tmp_path_factory.mktemp("resume"))


def _spec(manifest, mutate=None, **kw):
    raw = tiny_raw_config(manifest, **kw)
    if mutate is not None:
        mutate(raw)
    return run_spec_from_mapping(raw)


def _set(section, key, value):
    def apply(raw):
        target = raw
        for part in section.split("."):
            target = target[part]
        target[key] = value
    return apply


ROW = {"step": 4, "tokens_seen": 512, "loss": 2.5}


def test_fingerprint_is_stable_and_a_function_of_the_payload(manifest):
    a, b = build_resume_compat(_spec(manifest)), build_resume_compat(_spec(manifest))
    assert a.runtime_fingerprint == b.runtime_fingerprint and len(a.runtime_fingerprint) == 64
    assert a.payload == b.payload and a.payload["compat_version"] == RESUME_COMPAT_VERSION
    for key in ("seed", "model", "optimizer", "mesh", "parallelism", "data", "training"):
        assert key in a.payload, key
    assert a.payload["data"]["pipeline"]["manifest_sha256"] and a.payload["training"]["seq_len"] == 32
    assert a.payload["parallelism"]["expert_parallel"]["enabled"] is False


@pytest.mark.parametrize("mutate, where", [
    (_set("run", "seed", 1), "compatibility.seed"),
    (_set("model", "hidden_size", 128), "compatibility.model.hidden_size"),
    (_set("model", "num_layers", 3), "compatibility.model.num_layers"),
    (_set("model", "rope_theta", 5000.0), "compatibility.model.rope_theta"),
    (_set("optimizer", "weight_decay", 0.1), "compatibility.optimizer.spec.weight_decay"),
    (_set("optimizer.schedule", "peak_lr", 1e-3), "compatibility.optimizer.spec.schedule.peak_lr"),
    (_set("optimizer", "grad_clip_norm", 0.5), "compatibility.optimizer.spec.grad_clip_norm"),
    (_set("training", "seq_len", 16), "compatibility.data.pipeline"),
    (_set("training", "global_batch_size", 8), "compatibility.data.pipeline"),
    (_set("training", "gradient_accumulation_steps", 2), "compatibility.training.gradient_accumulation_steps"),
    (_set("data", "shuffle_seed", 9), "compatibility.data.pipeline"),
    (_set("data", "document_buffer_size", 16), "compatibility.data.pipeline"),
])
def test_changes_that_break_a_resume_are_named(manifest, mutate, where):
    spec = _spec(manifest)
    metadata = checkpoint_metadata(spec, ROW, reason="cadence")
    validate_resume_metadata(metadata, spec)
    changed = _spec(manifest, mutate)
    assert build_resume_compat(changed).runtime_fingerprint != metadata["runtime_fingerprint"]
    with pytest.raises(ContractError, match="resume compatibility mismatch at " + where.replace(".", r"\.")):
        validate_resume_metadata(metadata, changed)


@pytest.mark.parametrize("mutate", [
    _set("training", "log_every_steps", 7),
    _set("training", "checkpoint_every_steps", 3),
    _set("training", "target_tokens", 32 * 4 * 40),          # the constant schedule has no total_steps to protect
])
def test_mutable_controls_do_not_change_the_fingerprint(manifest, mutate):
    spec = _spec(manifest)
    metadata = checkpoint_metadata(spec, ROW, reason="final")
    validate_resume_metadata(metadata, _spec(manifest, mutate))
    assert metadata["mutable_controls"] == {"target_tokens": 512, "log_every_steps": 1, "checkpoint_every_steps": 1000}


def test_target_tokens_is_protected_when_the_schedule_length_derives_from_it(manifest):
    def cosine(raw):
        raw["optimizer"]["schedule"] = {"peak_lr": 3e-3, "name": "cosine", "warmup_steps": 1}
    spec = _spec(manifest, cosine)
    metadata = checkpoint_metadata(spec, ROW, reason="cadence")

    def longer(raw):
        cosine(raw)
        raw["training"]["target_tokens"] = 32 * 4 * 40
    with pytest.raises(ContractError, match="total_steps"):
        validate_resume_metadata(metadata, _spec(manifest, longer))

    def pinned(raw):
        raw["optimizer"]["schedule"] = {"peak_lr": 3e-3, "name": "cosine", "warmup_steps": 1, "total_steps": 50}
    fixed = _spec(manifest, pinned)
    meta2 = checkpoint_metadata(fixed, ROW, reason="cadence")

    def pinned_longer(raw):
        pinned(raw)
        raw["training"]["target_tokens"] = 32 * 4 * 40
    validate_resume_metadata(meta2, _spec(manifest, pinned_longer))       # an explicit total_steps frees target_tokens


def test_optimizer_policy_and_pipeline_description_enter_the_fingerprint(manifest):
    spec = _spec(manifest)
    plain = build_resume_compat(spec)
    with_policy = build_resume_compat(spec, optimizer_policy={"name": "adamw", "backend_parameter_counts": {"adamw": 25}})
    other_policy = build_resume_compat(spec, optimizer_policy={"name": "adamw", "backend_parameter_counts": {"adamw": 26}})
    ignored = build_resume_compat(spec, optimizer_policy={"name": "adamw", "backend_parameter_counts": {"adamw": 25},
                                                          "description": "free text", "routes": [1, 2]})
    assert len({plain.runtime_fingerprint, with_policy.runtime_fingerprint, other_policy.runtime_fingerprint}) == 3
    assert ignored.runtime_fingerprint == with_policy.runtime_fingerprint       # only the identity keys count
    described = build_resume_compat(spec, data_pipeline={"backend": "x", "order": "sequential"})
    assert described.payload["data"]["pipeline"] == {"backend": "x", "order": "sequential"}
    assert described.runtime_fingerprint != plain.runtime_fingerprint


def test_checkpoint_metadata_shape_and_required_row_fields(manifest):
    spec = _spec(manifest)
    meta = checkpoint_metadata(spec, ROW, reason="cadence", eval_row={"loss": 2.75})
    assert meta["schema_version"] == RESUME_METADATA_SCHEMA_VERSION and meta["run_id"] == "tiny"
    assert meta["checkpoint"] == {"step": 4, "tokens_seen": 512, "reason": "cadence"}
    assert meta["metrics"] == {"train_loss": 2.5, "eval_loss": 2.75}
    assert checkpoint_metadata(spec, ROW, reason="final")["metrics"]["eval_loss"] is None
    for missing in ("step", "tokens_seen", "loss"):
        row = {k: v for k, v in ROW.items() if k != missing}
        with pytest.raises(ContractError, match=f"missing '{missing}'"):
            checkpoint_metadata(spec, row, reason="cadence")


def test_metadata_validation_errors(manifest):
    spec = _spec(manifest)
    good = checkpoint_metadata(spec, ROW, reason="cadence")

    def broken(**changes):
        meta = copy.deepcopy(good)
        meta.update(changes)
        return meta

    cases = [
        (broken(schema_version=2), "schema_version must be 1"),
        (broken(compat_version=0), "compat_version must be 1"),
        (broken(run_id="other"), "run_id mismatch: checkpoint='other' current='tiny'"),
        (broken(compatibility=None), "compatibility must be an object"),
        (broken(runtime_fingerprint=""), "runtime_fingerprint must be a non-empty string"),
        (broken(runtime_fingerprint="0" * 64), "does not match compatibility payload"),
        (broken(checkpoint=None), "checkpoint must be an object"),
        (broken(checkpoint={"step": "4", "tokens_seen": 512}), r"checkpoint\.step must be an integer"),
        (broken(checkpoint={"step": 4, "tokens_seen": True}), r"checkpoint\.tokens_seen must be an integer"),
    ]
    for meta, match in cases:
        with pytest.raises(ContractError, match=match):
            validate_resume_metadata(meta, spec)
    tampered = copy.deepcopy(good)
    tampered["compatibility"]["seed"] = 5                          # edited by hand: the stored hash no longer fits
    with pytest.raises(ContractError, match="does not match compatibility payload"):
        validate_resume_metadata(tampered, spec)


def test_restored_state_must_agree_with_its_metadata(manifest):
    spec = _spec(manifest)
    meta = checkpoint_metadata(spec, ROW, reason="cadence")
    dataset = {"next_record_index": 16}

    def restored(**kw):
        base = dict(metadata=meta, step=4, host_state={"dataset": dataset}, dataset_state=dataset)
        base.update(kw)
        return types.SimpleNamespace(**base)

    validate_resume_compat(restored(), spec, state_step=4, state_tokens=512)
    with pytest.raises(ContractError, match="step mismatch: manager=5 metadata=4"):
        validate_resume_compat(restored(step=5), spec, state_step=4, state_tokens=512)
    with pytest.raises(ContractError, match="step mismatch: train_state=3 metadata=4"):
        validate_resume_compat(restored(), spec, state_step=3, state_tokens=512)
    with pytest.raises(ContractError, match="tokens_seen mismatch: train_state=500 metadata=512"):
        validate_resume_compat(restored(), spec, state_step=4, state_tokens=500)
    with pytest.raises(ContractError, match="host_state.dataset does not match dataset_state"):
        validate_resume_compat(restored(host_state={"dataset": {"next_record_index": 0}}), spec, state_step=4,
                               state_tokens=512)


def test_parallel_layout_is_part_of_the_contract(manifest):
    base = build_resume_compat(_spec(manifest))
    tp = build_resume_compat(_spec(manifest, mesh={"data": 1, "tp": 2}, parallelism={"mode": "ddp", "tensor_parallel": True}))
    assert tp.runtime_fingerprint != base.runtime_fingerprint
    assert tp.payload["parallelism"]["tensor_parallel"] == {"enabled": True, "axis_size": 2, "sequence_parallel": True}
    moe = build_resume_compat(_spec(manifest, kind="trinity", mesh={"data": 1, "ep": 2},
                                    parallelism={"mode": "ddp", "expert_parallel": True}))
    ep = moe.payload["parallelism"]["expert_parallel"]
    assert ep["enabled"] is True and ep["axis"] == "ep" and ep["axis_size"] == 2
