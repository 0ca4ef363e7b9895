"""Per-group optimizer diagnostics, their health roll-up, the router layer summary and the non-finite guard."""

import json
import math

import numpy as np
import pytest
import torch

from research_b200.config import run_spec_from_mapping
from research_b200.errors import ContractError
from research_b200.optim.diagnostics import groups_payload, health_fields, router_layers_payload
from research_b200.runtime.inspect import inspect_run
from research_b200.runtime.trainer import Trainer
from research_b200.runtime.training import run_training
from tests.helpers import run_gloo, tiny_dataset, tiny_raw_config, write_toml


def _jsonl(path):
    return [json.loads(line) for line in path.read_text().splitlines() if line.strip()]


def test_groups_cover_every_parameter_and_match_whole_model_norms(tmp_path):
    manifest = tiny_dataset(tmp_path)
    trainer = Trainer(run_spec_from_mapping(tiny_raw_config(manifest, kind="trinity", optimizer="muon")), device="cpu")
    m = trainer.train_step(diagnostics=True)
    groups = m.optimizer_groups
    names = {g["group"] for g in groups}
    assert {"embedding:adamw", "attention_q:muon", "moe_gate:muon", "final_norm:adamw"} <= names
    assert sum(g["parameter_count"] for g in groups) == trainer.parameter_count()
    assert sum(g["leaf_count"] for g in groups) == len(trainer.result.metadata)
    # the groups partition the model: their squared norms add up to the whole-model norms of the same step
    for key, whole in (("grad_norm", m.grad_norm), ("update_norm", m.update_norm), ("param_norm", m.param_norm)):
        total = math.sqrt(sum(g[key] ** 2 for g in groups))
        assert total == pytest.approx(whole, rel=1e-4), key
    bias = next(g for g in groups if g["tag"] == "moe_expert_bias")
    assert bias["weight_decay_enabled_count"] == 0 and bias["grad_norm"] == 0.0
    health = health_fields(groups)
    assert health["optimizer_nonfinite_group_count"] == 0 and health["optimizer_nonfinite_groups"] == []
    assert health["optimizer_groups_with_zero_grad"] >= 1
    assert health["optimizer_route_backend_counts"]["muon"] > 0
    assert health["optimizer_update_param_ratio_max"] >= health["optimizer_update_param_ratio_mean"] > 0.0
    # without diagnostics the step does not pay for them
    assert trainer.train_step(diagnostics=False).optimizer_groups == []


def test_payload_and_health_flag_nonfinite_groups():
    templates = [{"group": "a:adamw", "tag": "a", "backend": "adamw", "leaf_count": 2, "parameter_count": 10,
                  "weight_decay_enabled_count": 2, "auto_resolved_count": 0},
                 {"group": "b:muon", "tag": "b", "backend": "muon", "leaf_count": 1, "parameter_count": 4,
                  "weight_decay_enabled_count": 1, "auto_resolved_count": 1}]
    rows = groups_payload(templates, [[4.0, 1.0, 16.0], [float("inf"), 0.0, 0.0]])
    assert rows[0]["grad_norm"] == 2.0 and rows[0]["update_param_ratio"] == 0.25 and rows[0]["grad_norm_finite"]
    assert not rows[1]["grad_norm_finite"] and rows[1]["update_param_ratio"] == 0.0
    health = health_fields(rows)
    assert health["optimizer_nonfinite_groups"] == ["b:muon"] and health["optimizer_grad_norm_max_group"] == "a:adamw"
    assert health["optimizer_groups_with_zero_update"] == 1
    assert health_fields(None)["optimizer_nonfinite_groups"] is None


def test_router_layer_rows_have_quantiles_and_entropy():
    rows = router_layers_payload([{"layer_index": 3, "counts": torch.tensor([10.0, 0.0, 30.0, 60.0]),
                                   "importance": torch.tensor([0.25, 0.25, 0.25, 0.25])}])
    r = rows[0]
    assert r["layer_index"] == 3 and r["total_assignments"] == 100.0 and r["experts_active"] == 3
    assert r["load_min"] == 0.0 and r["load_max"] == 60.0 and r["load_p50"] == pytest.approx(20.0)
    assert r["importance_cv"] == 0.0 and r["importance_entropy"] == pytest.approx(math.log(4))
    assert r["load_cv"] == pytest.approx(np.std([10, 0, 30, 60]) / 25 * 100)


def test_rows_summary_and_inspect_carry_the_roll_ups(tmp_path):
    manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, kind="trinity", optimizer="muon", steps=3, run_id="diag",
                          output_dir=(tmp_path / "runs").as_posix())
    summary = run_training(write_toml(raw, tmp_path / "diag.toml"))
    rows = _jsonl(tmp_path / "runs" / "diag" / "metrics" / "train.jsonl")
    last = rows[-1]
    assert last["optimizer_groups"] and last["optimizer_nonfinite_group_count"] == 0
    assert last["moe_router_layers"][0]["load_p90"] >= last["moe_router_layers"][0]["load_p10"]
    assert summary.final_optimizer_groups and summary.final_optimizer_nonfinite_groups == []
    assert summary.final_optimizer_update_param_ratio_max > 0
    final = json.loads((tmp_path / "runs" / "diag" / "summaries" / "final.json").read_text())
    assert final["final_optimizer_grad_norm_max_group"] == summary.final_optimizer_grad_norm_max_group
    report = inspect_run(tmp_path / "runs" / "diag")
    assert report["optimizer_health"]["group_count"] == len(last["optimizer_groups"])
    assert report["optimizer_health"]["worst_update_ratio_group"]["group"] == \
        report["optimizer_health"]["update_param_ratio_max_group"]
    assert report["router_health"]["layer_count"] == 1
    assert report["router_health"]["worst_layer"]["layer_index"] == last["moe_router_layers"][0]["layer_index"]


def test_nonfinite_group_stops_the_run_and_names_the_group(tmp_path):
    manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, steps=3, run_id="nf", output_dir=(tmp_path / "runs").as_posix())
    cfg = write_toml(raw, tmp_path / "nf.toml")

    def poison(trainer):
        original = trainer.train_step_fn.run

        def run(batches, diagnostics=False):
            metrics = original(batches, diagnostics=diagnostics)
            if metrics.optimizer_groups:
                metrics.optimizer_groups[0]["update_norm"] = float("nan")
            return metrics

        trainer.train_step_fn.run = run

    with pytest.raises(ContractError, match="optimizer state became non-finite at step 1: embedding:adamw"):
        run_training(cfg, trainer_hook=poison)
    events = _jsonl(tmp_path / "runs" / "nf" / "events.jsonl")
    event = next(e for e in events if e["type"] == "optimizer_nonfinite")
    assert event["optimizer_nonfinite_groups"] == ["embedding:adamw"] and events[-1]["type"] == "training_failed"


def _group_norms(rank, world, raw):
    trainer = Trainer(run_spec_from_mapping(raw), device="cpu")
    trainer.train_step()
    m = trainer.train_step(diagnostics=True)
    return {g["group"]: (g["grad_norm"], g["update_norm"], g["param_norm"]) for g in m.optimizer_groups}


@pytest.mark.parametrize("optimizer,mesh,parallelism", [
    ("muon", {"fsdp": 2}, {"mode": "fsdp"}),
    ("adamw", {"tp": 2}, {"mode": "ddp", "tensor_parallel": True}),
])
def test_group_norms_do_not_depend_on_the_layout(tmp_path, optimizer, mesh, parallelism):
    manifest = tiny_dataset(tmp_path)
    want = _group_norms(0, 1, tiny_raw_config(manifest, optimizer=optimizer, steps=4))
    raw = tiny_raw_config(manifest, optimizer=optimizer, mesh=mesh, parallelism=parallelism, steps=4)
    for got in run_gloo(2, _group_norms, raw):
        got = {k.replace(":dist_muon", ":muon"): v for k, v in got.items()}
        assert set(got) == set(want)
        for name, values in want.items():
            assert got[name] == pytest.approx(values, rel=2e-2 if optimizer == "muon" else 2e-3, abs=1e-6), name
