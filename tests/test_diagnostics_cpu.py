"""Runtime diagnostics payload, telemetry through a fake NVML, metric enrichment and the preflight report."""

import json
import types
from pathlib import Path

import pytest
import torch

from research_b200.config import run_spec_from_mapping
from research_b200.runtime import diagnostics as D
from tests.helpers import tiny_dataset, tiny_raw_config, write_toml


class FakeNvml:
    """Three boards; the second one cannot report power, the third one cannot report utilisation."""

    NVML_TEMPERATURE_GPU = 0

    def __init__(self, fail_init=False):
        self.fail_init = fail_init
        self.handles = []

    def nvmlInit(self):
        if self.fail_init:
            raise RuntimeError("no driver")

    def nvmlDeviceGetHandleByIndex(self, i):
        self.handles.append(i)
        return i

    def nvmlDeviceGetMemoryInfo(self, h):
        return types.SimpleNamespace(used=(h + 1) * 10, total=100)

    def nvmlDeviceGetUtilizationRates(self, h):
        if h == 2:
            raise RuntimeError("not supported")
        return types.SimpleNamespace(gpu=50.0 + 20 * h, memory=10.0 * (h + 1))

    def nvmlDeviceGetPowerUsage(self, h):
        if h == 1:
            raise RuntimeError("not supported")
        return 400_000 + 100_000 * h

    def nvmlDeviceGetTemperature(self, h, kind):
        return 40 + 5 * h


def _spec(**kw):
    return run_spec_from_mapping(tiny_raw_config(Path("m.json"), **kw))


def test_nvml_sampling_sums_memory_and_power_averages_utilisation_and_takes_the_hottest_board():
    nvml = FakeNvml()
    out = D.sample_nvml([0, 1, 2], provider=nvml)
    assert nvml.handles == [0, 1, 2]
    assert out["gpu_memory_used_bytes"] == 60 and out["gpu_memory_total_bytes"] == 300
    assert out["gpu_utilization_pct"] == pytest.approx(60.0) and out["gpu_memory_utilization_pct"] == pytest.approx(15.0)
    assert out["gpu_power_w"] == pytest.approx(400.0 + 600.0) and out["gpu_temperature_c"] == 50.0


def test_nvml_sampling_degrades_to_nulls():
    empty = {k: None for k in D.TELEMETRY_KEYS[3:]}
    assert D.sample_nvml([0], provider=None) == empty
    assert D.sample_nvml([], provider=FakeNvml()) == empty
    assert D.sample_nvml([0], provider=FakeNvml(fail_init=True)) == empty
    cpu = D.sample_device_telemetry(torch.device("cpu"))
    assert set(cpu) == set(D.TELEMETRY_KEYS) and all(v is None for v in cpu.values())
    seen = D.sample_device_telemetry(torch.device("cpu"), nvml_provider=FakeNvml())
    assert seen["gpu_power_w"] == pytest.approx(400.0) and seen["device_memory_used_bytes"] is None


def test_execution_mode_names_the_state_mode_and_the_activation_axes():
    assert D.runtime_execution_mode(_spec()) == "replicated_data_parallel"
    tp = _spec(mesh={"fsdp": 2, "tp": 2}, parallelism={"mode": "fsdp", "tensor_parallel": True})
    assert D.runtime_execution_mode(tp) == "fsdp+tp"
    cp = _spec(mesh={"data": 1, "cp": 2}, parallelism={"mode": "ddp", "context_parallel": True})
    assert D.runtime_execution_mode(cp) == "replicated_data_parallel+cp"
    ep = _spec(kind="trinity", mesh={"fsdp": 1, "ep": 2, "tp": 2},
               parallelism={"mode": "zero2", "expert_parallel": True, "tensor_parallel": True})
    assert D.runtime_execution_mode(ep) == "zero2+ep+tp"


def test_phase_timer_accumulates_and_resets():
    t = D.PhaseTimer()
    with t.phase("a"):
        pass
    with t.phase("a"):
        pass
    t.add("b", 1.5)
    t.add("b", 0.5)
    assert t.get("b") == 2.0 and t.get("a") >= 0.0 and t.get("missing") == 0.0 and set(t.to_dict()) == {"a", "b"}
    assert t.total_sec() >= 0.0
    out = t.reset()
    assert out["b"] == 2.0 and t.to_dict() == {}
    with pytest.raises(ValueError):
        with t.phase("boom"):
            raise ValueError("x")
    assert "boom" in t.to_dict()                       # the time of a failed phase is still recorded


RUNTIME = {"performance": {"flops_per_token": 1000, "flops_per_token_exact": 800, "peak_flops_per_device": 1e6,
                           "peak_flops_total": 2e6, "device_kind": "B200", "device_count": 2},
           "parallelism": {"mode": "fsdp", "execution_mode": "fsdp+tp"},
           "device_telemetry": {"gpu_power_w": 900.0}}


def test_train_row_enrichment_rates_and_mfu():
    row = {"step": 3, "target_tokens": 400, "examples": 4, "loss": 2.0}
    out = D.enrich_train_metrics(row, timings={"data": 0.5, "train_step": 1.5, "metrics_sync": 0.5,
                                               "train_loop_step": 4.0}, runtime=RUNTIME)
    assert out["train_step_sec"] == 2.0 and out["step_sec"] == 4.0 and out["data_sec"] == 0.5
    assert out["train_tokens_per_sec"] == 200.0 and out["tokens_per_sec"] == 100.0 and out["examples_per_sec"] == 1.0
    assert out["flops_per_step"] == 400_000 and out["flops_per_sec"] == 200_000.0
    assert out["mfu"] == pytest.approx(10.0) and out["mfu_exact"] == pytest.approx(8.0)
    assert out["execution_mode"] == "fsdp+tp" and out["parallelism_mode"] == "fsdp"
    assert out["gpu_power_w"] == 900.0 and out["gpu_temperature_c"] is None and out["loss"] == 2.0
    # the reference's *_sec names are taken as well; a fresh telemetry sample wins over the one in the payload
    same = D.enrich_train_metrics(row, timings={"data_sec": 0.5, "train_dispatch_sec": 1.5, "metrics_sync_sec": 0.5,
                                                "step_sec": 4.0}, runtime=RUNTIME,
                                  telemetry={"gpu_power_w": 500.0})
    assert same["train_tokens_per_sec"] == 200.0 and same["step_sec"] == 4.0 and same["gpu_power_w"] == 500.0
    idle = D.enrich_train_metrics(row, timings={}, runtime=RUNTIME)
    assert idle["train_tokens_per_sec"] is None and idle["mfu"] is None and idle["flops_per_sec"] is None
    no_peak = dict(RUNTIME, performance=dict(RUNTIME["performance"], peak_flops_total=None))
    assert D.enrich_train_metrics(row, timings={"train_step": 1.0}, runtime=no_peak)["mfu"] is None


def test_eval_row_enrichment_and_run_summary():
    ev = D.enrich_eval_metrics({"loss": 1.0, "target_tokens": 300, "examples": 6}, eval_sec=2.0)
    assert ev["eval_tokens_per_sec"] == 150.0 and ev["eval_examples_per_sec"] == 3.0 and ev["eval_sec"] == 2.0
    assert D.enrich_eval_metrics({"target_tokens": 1, "examples": 1}, eval_sec=0.0)["eval_tokens_per_sec"] is None
    rows = [{"train_tokens_per_sec": 10.0, "mfu": 1.0, "batch_het": None},
            {"train_tokens_per_sec": 30.0, "mfu": None, "batch_het": 0.5},
            {"train_tokens_per_sec": 50.0, "mfu": 3.0, "batch_het": True}]
    s = D.training_diagnostics_summary(rows, total_wall_sec=9.0, runtime=RUNTIME)
    assert s["avg_train_tokens_per_sec"] == 30.0 and s["steady_train_tokens_per_sec"] == 40.0
    assert s["final_train_tokens_per_sec"] == 50.0 and s["avg_mfu"] == 2.0 and s["final_mfu"] == 3.0
    assert s["avg_batch_het"] == 0.5 and s["final_batch_het"] is None           # a boolean is not a number
    assert s["total_wall_sec"] == 9.0 and s["device_kind"] == "B200" and s["execution_mode"] == "fsdp+tp"
    assert s["runtime_diagnostics_path"] == "diagnostics/runtime.json"
    one = D.training_diagnostics_summary(rows[:1])
    assert one["steady_train_tokens_per_sec"] is None and "total_wall_sec" not in one
    none = D.training_diagnostics_summary([])
    assert none["avg_train_tokens_per_sec"] is None and none["final_mfu"] is None


def test_batch_and_compile_contract_arithmetic():
    spec = _spec(batch=8, seq_len=16, accum=3)
    b = D.batch_summary(spec, 4)
    assert b == {"global_batch_size": 8, "micro_global_batch_size": 8, "effective_global_batch_size": 24,
                 "gradient_accumulation_steps": 3, "per_device_batch_size": 2, "micro_tokens_per_step": 128,
                 "effective_tokens_per_step": 384, "global_tokens_per_step": 384, "per_device_tokens_per_step": 96}
    mesh = types.SimpleNamespace(size=lambda a: {"data": 2, "fsdp": 2}.get(a, 1))
    c = D.compile_contract_summary(spec, mesh)
    assert c["train"]["expected_batch_shape"] == [3, 8, 16] and c["eval"]["expected_batch_shape"] == [8, 16]
    assert c["train"]["donate_state"] is True and c["eval"]["donate_state"] is False
    assert c["train"]["input_shardings"]["input_ids"] == {"rows": ["data", "fsdp"], "sequence": []}
    assert D.moe_balance_payload(spec) == {"name": "none"}
    moe = D.moe_balance_payload(_spec(kind="trinity"))
    assert moe["name"] == "smebu" and set(moe) == {"name", "load_lr", "momentum", "clamp", "sequence_aux_loss_weight"}


def test_runtime_payload_and_preflight_report_of_a_tiny_run(tmp_path):
    from research_b200.runtime.preflight import format_preflight_report, preflight_report_to_json, run_preflight

    manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, kind="trinity", run_id="pf", output_dir=(tmp_path / "runs").as_posix(), evals=True,
                          accum=2, batch=4)
    report = run_preflight(write_toml(raw, tmp_path / "pf.toml"))
    assert not (tmp_path / "runs" / "pf").exists()                      # a preflight writes nothing
    assert report["status"] == "ok" and report["training"]["compile"] == "passed"
    tr = report["training"]
    assert tr["batch_tokens"] == 4 * 32 * 2 and tr["estimated_steps"] == 4 and tr["per_device_batch_size"] == 4
    assert tr["first_step_loss"] == pytest.approx(report["first_step"]["loss"])
    assert tr["first_step_moe_aux_loss"] is not None and tr["first_step_router_max_vio"] is not None
    fb = report["data"]["first_batch"]
    assert fb["target_tokens"] == 256 and fb["examples"] == 8 and fb["document_aware"] and fb["documents_touched"] >= 1
    assert report["data"]["train_split_tokens"] == report["data"]["train_split_end"] - report["data"]["train_split_start"]
    ev = report["eval"]
    assert ev["num_batches"] == 2 and ev["split"] == "val" and ev["target_tokens"] == 2 * 4 * 32 and ev["loss"] > 0
    diag = report["diagnostics"]
    for key in ("python", "packages", "runtime", "mesh", "model", "optimizer", "performance", "compile", "parallelism",
                "profiling", "kernels", "sharding", "data_pipeline", "device_telemetry"):
        assert key in diag, key
    assert diag["model"]["moe_balance"]["name"] == "smebu" and diag["model"]["parameter_leaves"] > 0
    assert diag["mesh"]["effective_tokens_per_step"] == 256 and diag["mesh"]["global_mesh_size"] == 1
    par = diag["parallelism"]
    assert par["execution_mode"] == "replicated_data_parallel" and par["tensor_parallel_policy"]["lm_head"] == "replicated"
    assert par["expert_parallel_policy"]["num_experts"] == 4 and par["expert_parallel_policy"]["enabled"] is False
    assert par["batch"]["per_device_batch_size"] == 4 and par["host_artifacts"]["writer"] == "single_host"
    kern = report["kernels"]
    assert kern["active_count"] == 0 and kern["fallback_count"] + kern["unavailable_count"] == len(kern["ops"])
    obs = report["observed_sharding"]
    assert obs["first_train_batch"]["input_ids"]["shape"] == [4, 32] and obs["train_state"]["mode"] == "ddp"
    text = format_preflight_report(report)
    for head in ("preflight: ok", "run: pf", "devices:", "mesh:", "parallelism:", "train data:", "model: trinity",
                 "optimizer: adamw", "training: estimated_steps=4", "first step: loss=", "compile contract:",
                 "profiling:", "kernels:", "eval: name=validation"):
        assert head in text, head
    assert json.loads(preflight_report_to_json(report))["run_id"] == "pf"
    no_eval = tiny_raw_config(manifest, run_id="pf2", output_dir=(tmp_path / "runs").as_posix())
    second = run_preflight(write_toml(no_eval, tmp_path / "pf2.toml"))
    assert second["eval"] is None and "eval: skipped" in format_preflight_report(second)


def test_run_inspection_sections_formatter_and_missing_checkpoint(tmp_path):
    import shutil

    from research_b200.errors import ContractError
    from research_b200.runtime.inspect import (format_run_inspection, inspect_run, profiling_summary,
                                               run_inspection_to_json, wandb_summary)
    from research_b200.runtime.training import run_training

    manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, kind="trinity", run_id="ins", output_dir=(tmp_path / "runs").as_posix(), evals=True,
                          steps=4, checkpoint_every=2)
    run_training(write_toml(raw, tmp_path / "ins.toml"))
    run_dir = tmp_path / "runs" / "ins"
    report = inspect_run(run_dir)
    assert report["status"] == "completed" and report["final"]["step"] == 4 and report["final"]["eval_loss"] > 0
    assert [c["step"] for c in report["checkpoints"]] == [2, 4] and all(c["exists"] for c in report["checkpoints"])
    assert report["latest_checkpoint"]["step"] == 4 and report["best_checkpoint"]["eval_loss"] is not None
    assert report["checkpoint_index"]["latest_step"] == 4
    diag = report["diagnostics"]
    assert diag["path"] == "diagnostics/runtime.json" and diag["backend"] == "cpu" and diag["device_count"] == 1
    assert diag["parallelism"]["batch"]["global_batch_size"] == 4 and diag["data_pipeline"]["order"] == "document_buffer"
    assert report["kernels"]["active_count"] == 0 and report["kernels"]["unavailable"] is not None
    assert report["wandb"] is None and report["profiling"]["enabled"] is False
    assert len(report["recent_train_metrics"]) == 4 and len(report["recent_eval_metrics"]) >= 2
    assert report["router_health"]["layer_count"] == 1 and report["optimizer_health"]["group_count"] > 0
    text = format_run_inspection(report)
    for head in ("run: ins", "status: completed", "final: step=4", "validation: loss=", "runtime: backend=cpu",
                 "parallelism: mode=replicated_data_parallel", "data pipeline: backend=blackwell_native", "kernels:",
                 "router health: layers=1", "optimizer health: groups=", "latest checkpoint: step=4",
                 "best checkpoint: step=", "checkpoints:", "  step=2 "):
        assert head in text, head
    assert "wandb:" not in text and "profiling:" not in text
    assert json.loads(run_inspection_to_json(report))["run_id"] == "ins"
    # sections that come from optional files
    wb = wandb_summary({"enabled": True, "wandb_run_id": "ins-abc", "project": "p", "url": None}, None)
    assert wb["wandb_run_id"] == "ins-abc" and wb["entity"] is None
    assert wandb_summary(None, {"wandb": {"project": "q"}})["project"] == "q" and wandb_summary(None, {}) is None
    prof = profiling_summary({"enabled": True, "status": "completed", "trace_files": ["profiles/a.trace.json.gz"],
                              "traced_step_range": {"start": 3, "end": 4}}, None)
    assert prof["perfetto_trace_available"] and prof["trace_step_range"] == {"start": 3, "end": 4}
    configured = profiling_summary(None, {"profiling": {"enabled": True, "trace_start_step": 3, "trace_steps": 2}})
    assert configured["status"] == "configured" and configured["trace_step_range"] is None
    # a run that never finished still inspects; a retained checkpoint that vanished is an error
    (run_dir / "summaries" / "final.json").unlink()
    partial = inspect_run(run_dir)
    assert partial["final"] is None and "progress: step=4" in format_run_inspection(partial)
    shutil.rmtree(run_dir / report["latest_checkpoint"]["checkpoint_path"])
    with pytest.raises(ContractError, match="retained path does not exist"):
        inspect_run(run_dir)


def test_checkpoint_eval_and_sample_payloads(tmp_path):
    from research_b200.errors import ContractError
    from research_b200.runtime.checkpoint_eval import (checkpoint_eval_to_json, evaluate_checkpoint,
                                                       format_checkpoint_eval)
    from research_b200.runtime.sampling import (checkpoint_sample_to_json, format_checkpoint_sample, parse_prompt_ids,
                                                sample_checkpoint)
    from research_b200.runtime.training import run_training

    manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, run_id="ce", output_dir=(tmp_path / "runs").as_posix(), evals=True, steps=2,
                          checkpoint_every=2)
    summary = run_training(write_toml(raw, tmp_path / "ce.toml"))
    run_dir = tmp_path / "runs" / "ce"
    payload = evaluate_checkpoint(run_dir, "latest")
    assert payload["status"] == "completed" and payload["checkpoint"]["step"] == 2
    assert payload["checkpoint"]["path"] == payload["checkpoint_path"] and len(payload["checkpoint"]["runtime_fingerprint"]) == 64
    row = payload["eval"]
    assert row["eval_name"] == "validation" and row["num_batches"] == 2 and row["target_tokens"] == 2 * 4 * 32
    assert row["loss"] == pytest.approx(summary.final_eval_loss, rel=1e-6) and row["eval_tokens_per_sec"] > 0
    assert row["token_start"] is not None and row["document_aware"] in (True, False)
    assert payload["data"]["manifest_path"] == manifest.as_posix() and len(payload["data"]["manifest_sha256"]) == 64
    stored = json.loads((run_dir / payload["artifact_path"]).read_text())
    assert stored["eval"]["loss"] == row["loss"] and stored["checkpoint"] == payload["checkpoint"]
    assert format_checkpoint_eval(payload).startswith("evaluated checkpoint step=2 path=checkpoints/")
    assert json.loads(checkpoint_eval_to_json(payload))["run_id"] == "ce"
    with pytest.raises(ContractError, match="needs checkpoint and eval objects"):
        format_checkpoint_eval({"checkpoint": 1})

    sample = sample_checkpoint(run_dir, "2", prompt_ids=[5, 6, 7], max_new_tokens=3, top_k=1)
    assert sample["checkpoint"]["selector"] == "2" and sample["checkpoint"]["step"] == 2
    assert sample["model"] == {"name": "decoder", "variant": "tiny", "vocab_size": 256, "max_seq_len": 64}
    assert sample["sampling"] == {"max_new_tokens": 3, "temperature": 1.0, "top_k": 1, "top_p": None}
    assert sample["prompt_ids"] == [5, 6, 7] and len(sample["generated_ids"]) == 3 and len(sample["full_ids"]) == 6
    assert "sampled checkpoint step=2" in format_checkpoint_sample(sample)
    assert json.loads(checkpoint_sample_to_json(sample))["status"] == "completed"
    lines = (run_dir / sample["artifact_path"]).read_text().splitlines()
    assert len(lines) == 1 and json.loads(lines[0])["generated_ids"] == sample["generated_ids"]
    with pytest.raises(ContractError, match="exceeds vocab size"):
        sample_checkpoint(run_dir, "latest", prompt_ids="1", max_new_tokens=1, top_k=1000)
    with pytest.raises(ContractError, match="outside the vocabulary"):
        sample_checkpoint(run_dir, "latest", prompt_ids="1,999", max_new_tokens=1)
    assert parse_prompt_ids(" 1, 2 ,3") == [1, 2, 3] and parse_prompt_ids((4, 5)) == [4, 5]
    for bad, match in (("", "non-empty"), ("1,,2", "invalid token id"), ("1,-2", "invalid token id"),
                       ("0x10", "invalid token id"), ([], "at least one"), ([1, True], "must be integers"),
                       ([1, 2.0], "must be integers"), ([-1], "non-negative")):
        with pytest.raises(ContractError, match=match):
            parse_prompt_ids(bad)
    with pytest.raises(ContractError, match="outside the vocabulary"):
        parse_prompt_ids([300], 256)


def test_lifecycle_events_and_summary_carry_the_run_level_fields(tmp_path):
    from research_b200.runtime.training import COMPLETED_EVENT_FIELDS, run_training

    manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, kind="trinity", run_id="ev", output_dir=(tmp_path / "runs").as_posix(), steps=3)
    summary = run_training(write_toml(raw, tmp_path / "ev.toml"))
    run_dir = tmp_path / "runs" / "ev"
    events = [json.loads(line) for line in (run_dir / "events.jsonl").read_text().splitlines()]
    started = next(e for e in events if e["type"] == "training_started")
    assert started["execution_mode"] == "replicated_data_parallel" and started["parallelism_mode"] == "ddp"
    assert started["data_pipeline_backend"] == "blackwell_native" and started["data_pipeline_order"] == "document_buffer"
    assert started["data_document_buffer_size"] == 8 and started["moe_balance_policy"] == "smebu"
    assert started["gradient_accumulation_steps"] == 1 and started["z_loss_weight"] == 0.0 and started["resume"] is False
    done = events[-1]
    assert done["type"] == "training_completed" and set(COMPLETED_EVENT_FIELDS) <= set(done)
    assert done["steps"] == 3 and done["final_loss"] == pytest.approx(summary.final_loss)
    assert done["final_moe_router_layers"][0]["layer_index"] == 1 and done["final_optimizer_groups"]
    final = json.loads((run_dir / "summaries" / "final.json").read_text())
    assert final["single_process"] is True and final["process_index"] == 0 and final["global_device_count"] == 1
    assert final["data_document_count"] == 300 and final["data_document_offsets_path"] == "document_offsets.u64"
    assert final["data_pipeline_state_schema_version"] == 2 and final["data_pipeline_version"].startswith("research_b200-")
    assert final["data_pipeline_worker_count"] == 0 and final["data_pipeline_prefetch"] is False
    assert final["data_document_buffer_size"] == 8 and final["data_document_refill_size"] == 8
    assert final["final_moe_router_layers"] == done["final_moe_router_layers"]
    assert final["execution_mode"] == "replicated_data_parallel"
    # a failing run says why in the same two keys the mirror and the inspector read
    bad = tiny_raw_config(manifest, run_id="evbad", output_dir=(tmp_path / "runs").as_posix(), steps=3)
    bad["training"]["target_tokens"] = 10 ** 9                                   # more than the data holds
    with pytest.raises(Exception):
        run_training(write_toml(bad, tmp_path / "evbad.toml"))
    failed = [json.loads(l) for l in (tmp_path / "runs" / "evbad" / "events.jsonl").read_text().splitlines()][-1]
    assert failed["type"] == "training_failed" and failed["error"] == failed["error_message"] and failed["error_type"]
