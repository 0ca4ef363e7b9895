"""Validation matrices: derived configs, the plan of a dry run, and the analyzers' gates on synthetic run directories
(reference pattern: tests/jaxtitan/test_moe_m1_analysis.py and test_dist_muon_*_analysis.py feed hand-made payloads to
the cloud analyzers)."""

import json
import tarfile
import tomllib
from pathlib import Path

import pytest

from research_b200.errors import ContractError
from research_b200.runtime import validation_matrix as vm


def _write_run(root: Path, run_id: str, *, step_sec: float, losses=None, events=None, rows: int = 12,
               groups=None) -> Path:
    run = root / run_id
    (run / "metrics").mkdir(parents=True)
    (run / "summaries").mkdir()
    (run / "diagnostics").mkdir()
    losses = losses or [10.0 - 0.2 * i for i in range(rows)]
    with (run / "metrics" / "train.jsonl").open("w") as f:
        for i, loss in enumerate(losses):
            row = {"step": i + 1, "loss": loss, "train_step_sec": step_sec, "step_sec": step_sec * 1.02,
                   "train_tokens_per_sec": 8192 / step_sec}
            if groups is not None and i == len(losses) - 1:
                row["optimizer_groups"] = groups
                row["optimizer_nonfinite_groups"] = sum(1 for g in groups if not g.get("finite", True))
            f.write(json.dumps(row) + "\n")
    events = events if events is not None else ["training_started", "training_completed"]
    (run / "events.jsonl").write_text("".join(json.dumps({"type": t, "step": 3}) + "\n" for t in events))
    (run / "summaries" / "final.json").write_text(json.dumps({"status": "completed"}))
    (run / "diagnostics" / "runtime.json").write_text(json.dumps(
        {"runtime": {"device_kind": "NVIDIA B200"}, "mesh": {"device_count": 4}, "optimizer": {"name": "muon"}}))
    return run


def test_every_case_derives_a_config_that_passes_the_run_contract(tmp_path):
    from research_b200.config import run_spec_from_mapping

    for name, cases in vm.MATRICES.items():
        assert len({c.run_id for c in cases}) == len(cases)
        for case in cases:
            raw = vm.derive_config(case, tmp_path / "manifest.json", tmp_path / "out")
            back = tomllib.loads(vm.write_toml(raw))
            assert back == json.loads(json.dumps(raw)), case.run_id          # the TOML writer loses nothing
            spec = run_spec_from_mapping(back)
            assert spec.mesh.device_count == case.gpus == 4
            assert spec.training.target_tokens == spec.training.global_batch_size * spec.training.seq_len * case.steps
            assert spec.profiling.enabled == (name == "profile64")


def test_toml_writer_handles_nesting_and_rejects_what_toml_cannot_hold():
    raw = {"a": 1, "t": {"x": True, "y": [1, 2.5, "s"], "deep": {"k": "v"}}, "empty": {}}
    assert tomllib.loads(vm.write_toml(raw)) == raw
    with pytest.raises(ContractError, match="cannot write"):
        vm.write_toml({"t": {"x": None}})


def test_dry_run_plans_one_launch_per_case_and_skips_what_does_not_fit(tmp_path):
    launched = []
    plan = vm.run_matrix("correctness17", tmp_path, gpus=4, manifest=tmp_path / "m.json", dry_run=True,
                         runner=lambda *a, **k: launched.append(a))
    assert not launched and all(c["status"] == "planned" for c in plan["cases"])
    first = plan["cases"][0]
    assert first["command"][1:4] == ["-m", "torch.distributed.run", "--nnodes=1"] and "--nproc-per-node=4" in first["command"]
    assert first["command"][-4:-1] == ["research_b200", "run", "train"] and Path(first["command"][-1]).is_file()
    nccl = next(c for c in plan["cases"] if c["case"]["run_id"].endswith("dense_fsdp4_muon_nccl"))
    assert nccl["env"] == {"RESEARCH_B200_PEER_COLLECTIVES": "0"}
    assert json.loads((tmp_path / "correctness17" / "matrix.json").read_text())["matrix"] == "correctness17"
    subset = vm.run_matrix("correctness17", tmp_path / "sub", gpus=4, manifest=tmp_path / "m.json", dry_run=True,
                           only=("moe_ep4", "cp4_muon_fused"))
    assert sorted(c["case"]["run_id"].split("17_")[1] for c in subset["cases"]) == [
        "dense_cp4_muon_fused", "moe_ep4_adamw_fused", "moe_ep4_adamw_nccl", "moe_ep4_dion_fused"]
    small = vm.run_matrix("correctness17", tmp_path / "two", gpus=2, manifest=tmp_path / "m.json", dry_run=True)
    assert all(c["status"] == "skipped" for c in small["cases"])
    with pytest.raises(ContractError, match="unknown validation matrix"):
        vm.run_matrix("nope", tmp_path, gpus=4, manifest="m.json", dry_run=True)


def test_run_matrix_records_exit_codes_and_bundles_the_runs(tmp_path):
    class Proc:
        def __init__(self, rc):
            self.returncode, self.stderr = rc, "boom" if rc else ""

    calls = []

    def runner(cmd, **kwargs):
        calls.append((cmd, kwargs["env"].get("RESEARCH_B200_PEER_COLLECTIVES")))
        if len(calls) == 1:                                        # what a run leaves behind: metrics and a checkpoint
            run = tmp_path / "correctness17" / "some_run"
            (run / "checkpoints" / "000017" / "train").mkdir(parents=True)
            (run / "checkpoints" / "000017" / "train" / "leaf").write_bytes(b"x" * 4096)
            (run / "metrics").mkdir()
            (run / "metrics" / "train.jsonl").write_text("{}\n")
        return Proc(1 if len(calls) == 2 else 0)

    out = vm.run_matrix("correctness17", tmp_path, gpus=4, manifest=tmp_path / "m.json", runner=runner)
    assert len(calls) == len(vm.MATRICES["correctness17"])
    assert [c["status"] for c in out["cases"]].count("failed") == 1 and out["cases"][1]["stderr_tail"] == "boom"
    assert calls[1][1] == "0"                                     # the NCCL case ran with the switch in its environment
    with tarfile.open(tmp_path / "correctness17.tgz") as archive:
        names = archive.getnames()
    assert "correctness17/matrix.json" in names and "correctness17/some_run/metrics/train.jsonl" in names
    assert not any("000017" in n for n in names)                  # checkpoints stay out of the bundle


def test_analyzer_gates_runs_pairs_and_baseline(tmp_path):
    cand = tmp_path / "cand"
    _write_run(cand, "m_dense_fsdp4_muon_fused", step_sec=0.100)
    _write_run(cand, "m_dense_fsdp4_muon_nccl", step_sec=0.105)
    _write_run(cand, "m_moe_ep4_adamw_fused", step_sec=0.200)
    payload = vm.analyze_matrix(cand, work_dir=tmp_path / "w")
    assert payload["overall_gate"] and len(payload["runs"]) == 3
    pair = payload["pairs"][0]
    assert pair["kind"] == "transport" and pair["gate"] and abs(pair["step_time_ratio"] - 0.100 / 0.105) < 1e-9
    text = vm.format_matrix_analysis(payload)
    assert "overall_gate=True" in text and "m_moe_ep4_adamw_fused" in text
    # a baseline bundle (as .tgz): one run got slower than the allowed fraction
    base = tmp_path / "base"
    _write_run(base, "m_dense_fsdp4_muon_fused", step_sec=0.080)
    _write_run(base, "m_moe_ep4_adamw_fused", step_sec=0.205)
    with tarfile.open(tmp_path / "base.tgz", "w:gz") as archive:
        archive.add(base, arcname="base")
    against = vm.analyze_matrix(cand, baseline=tmp_path / "base.tgz", min_speedup=0.95, work_dir=tmp_path / "w")
    gates = {a["run_id"]: a["gate"] for a in against["baseline"]}
    assert gates == {"m_dense_fsdp4_muon_fused": False, "m_moe_ep4_adamw_fused": True} and not against["overall_gate"]
    assert vm.main(["analyze", str(cand), "--work-dir", str(tmp_path / "w")]) == 0
    assert vm.main(["analyze", str(cand), "--baseline", str(tmp_path / "base.tgz"), "--work-dir", str(tmp_path / "w"),
                    "--json-out", str(tmp_path / "cmp.json")]) == 1
    assert json.loads((tmp_path / "cmp.json").read_text())["overall_gate"] is False


@pytest.mark.parametrize("kwargs,needle", [
    ({"events": ["training_started"]}, "no training_completed event"),
    ({"events": ["training_started", "optimizer_nonfinite", "training_failed"]}, "failure events"),
    ({"losses": [5.0, 5.1, 5.2, 5.3, 5.4, 5.5]}, "loss did not fall"),
    ({"losses": [5.0, 4.0, float("nan"), 3.0]}, "non-finite loss"),
    ({"groups": [{"group": "matrix:muon", "finite": False, "update_param_ratio": 1.0}]}, "nonfinite_groups"),
])
def test_a_run_that_breaks_a_gate_is_named_with_its_problem(tmp_path, kwargs, needle):
    _write_run(tmp_path / "c", "bad_run_fused", step_sec=0.1, **kwargs)
    _write_run(tmp_path / "c", "good_run_fused", step_sec=0.1)
    payload = vm.analyze_matrix(tmp_path / "c", work_dir=tmp_path / "w")
    by_id = {r["run_id"]: r for r in payload["runs"]}
    assert by_id["good_run_fused"]["gate"] and not by_id["bad_run_fused"]["gate"] and not payload["overall_gate"]
    assert any(needle in p for p in by_id["bad_run_fused"]["problems"]), by_id["bad_run_fused"]["problems"]
    assert "FAIL" in vm.format_matrix_analysis(payload)


def test_groups_without_gradient_are_noted_not_failed(tmp_path):
    groups = [{"group": "router_bias:adamw", "finite": True, "update_param_ratio": 0.0}]
    run = _write_run(tmp_path / "c", "moe_fused", step_sec=0.1, groups=groups)
    rows = [json.loads(line) for line in (run / "metrics" / "train.jsonl").read_text().splitlines()]
    rows[-1].update(optimizer_groups_with_zero_grad=1, optimizer_groups_with_zero_update=1)
    (run / "metrics" / "train.jsonl").write_text("".join(json.dumps(r) + "\n" for r in rows))
    payload = vm.analyze_matrix(tmp_path / "c", work_dir=tmp_path / "w")
    only = payload["runs"][0]
    assert only["gate"] and payload["overall_gate"]
    assert only["notes"] == ["groups_with_zero_grad = 1", "groups_with_zero_update = 1"]
    assert "(groups_with_zero_grad = 1; groups_with_zero_update = 1)" in vm.format_matrix_analysis(payload)


def test_slow_fused_path_breaks_the_pair_envelope(tmp_path):
    _write_run(tmp_path / "c", "x_fused", step_sec=0.130)
    _write_run(tmp_path / "c", "x_nccl", step_sec=0.100)
    payload = vm.analyze_matrix(tmp_path / "c", work_dir=tmp_path / "w")
    assert all(r["gate"] for r in payload["runs"]) and not payload["pairs"][0]["gate"] and not payload["overall_gate"]


def test_materialize_rejects_missing_and_unknown_artifacts(tmp_path):
    with pytest.raises(ContractError, match="missing artifact"):
        vm.materialize(tmp_path / "nothing.tgz", tmp_path / "w")
    (tmp_path / "x.zip").write_text("no")
    with pytest.raises(ContractError, match="unsupported artifact type"):
        vm.materialize(tmp_path / "x.zip", tmp_path / "w")
    assert vm.main(["analyze", str(tmp_path / "nothing.tgz")]) == 2


def test_muon_selector_artifact_gate(tmp_path):
    def cand(execution, ms, ok=True, det=True, rep=0.0):
        return {"execution": execution, "correctness_gate": ok, "deterministic": det, "replica_max_abs_error": rep,
                "max_update_abs_error": 1e-5, "max_parameter_abs_error": 1e-6, "timing_ms": {"median": ms}}

    good = {"transport": "arena", "all_selected_pass": True, "cases": [
        {"case": "attention_kv_bucket24", "selected": "distributed_large_gram",
         "candidates": [cand("duplicated", 20.0), cand("distributed_large_gram", 4.0), cand("distributed_exchange", 5.0)]},
        {"case": "attention_q_gate", "selected": "duplicated", "candidates": [cand("duplicated", 1.0), cand("distributed_direct", 1.1)]},
        {"case": "too_small", "skipped": "needs 4 ranks"}]}
    (tmp_path / "a").mkdir()
    (tmp_path / "a" / "manifest.json").write_text(json.dumps(good))
    out = vm.analyze_muon_bench(tmp_path / "a")
    assert out["overall_gate"] and [r["selected"] for r in out["rows"]] == ["distributed_large_gram", "duplicated"]
    assert abs(out["rows"][0]["speedup_vs_duplicated"] - 5.0) < 1e-9
    assert vm.main(["analyze-muon", str(tmp_path / "a")]) == 0
    bad = json.loads(json.dumps(good))
    bad["cases"][0]["candidates"][1]["deterministic"] = False
    (tmp_path / "b").mkdir()
    (tmp_path / "b" / "manifest.json").write_text(json.dumps(bad))
    out = vm.analyze_muon_bench(tmp_path / "b")
    assert not out["overall_gate"] and "attention_kv_bucket24" in out["problems"][0]
    assert vm.main(["analyze-muon", str(tmp_path / "b")]) == 1
    with pytest.raises(ContractError, match="no Muon benchmark manifest"):
        vm.analyze_muon_bench(tmp_path / "none")
