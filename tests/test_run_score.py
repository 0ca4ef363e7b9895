"""Run score arithmetic and the registry ledger."""

import math

import pytest

from research_b200.runtime import run_score as rs

BASE = {"core": 0.10, "final_val_bpb": 1.20, "domain_mean_bpb": 1.30, "domain_worst_bpb": 1.60,
        "train_epiplexity_bpb_auc_per_byte": 2.0, "steady_train_mfu": 0.30, "flops_per_token": 1e9,
        "peak_flops_total": 2.25e15, "tokens_seen": 1e9, "steady_train_tokens_per_sec": 5e4,
        "decode_tokens_per_sec": 1000.0, "prefill_tokens_per_sec": 50000.0, "ttft_sec": 0.2, "status": "complete"}


def test_baseline_scores_base_score():
    out = rs.run_score(BASE, BASE)
    assert out["score"] == pytest.approx(rs.BASE_SCORE)
    assert out["quality"] == pytest.approx(1.0) and out["health"] == 1.0


def test_components_are_clamped_and_weighted():
    run = dict(BASE, steady_train_mfu=0.90, decode_tokens_per_sec=5000.0, ttft_sec=0.02)
    out = rs.run_score(run, BASE)
    assert out["training_efficiency"] == pytest.approx(0.5 * 1.5 + 0.3 * 1.0 + 0.2 * 1.0)   # mfu ratio 3 -> 1.5
    assert out["inference_efficiency"] == pytest.approx(0.55 * 1.5 + 0.30 * 1.0 + 0.15 * 1.5)
    assert out["score"] > rs.BASE_SCORE


def test_missing_inputs_and_failures_are_unscored():
    run = dict(BASE)
    run.pop("core")
    out = rs.run_score(run, BASE)
    assert out["score"] is None and "core" in out["unscored_reason"]
    assert rs.run_score(dict(BASE, status="failed"), BASE)["score"] is None


def test_health_gates_and_penalties():
    assert rs.health({"status": "failed"}) == 0.0
    assert rs.health({"nan_count": 1}) == 0.0
    assert rs.health({"status": "incomplete"}) == 0.25
    h = rs.health({"status": "unstable", "loss_spike_count": 10, "grad_norm_spike_count": 2,
                   "best_val_bpb": 1.0, "final_val_bpb": 1.1})
    assert h == pytest.approx(0.75 - 0.25 - 0.06 - 0.10)


def test_bits_per_byte():
    assert rs.bits_per_byte(math.log(2.0) * 800, 100) == pytest.approx(8.0)
    with pytest.raises(ValueError):
        rs.bits_per_byte(1.0, 0)


def test_registry_upserts_by_run_name(tmp_path):
    path = tmp_path / "runs" / "registry.jsonl"
    rs.register_run({"run_name": "a", "score": 25.0, "status": "complete"}, path)
    rs.register_run({"run_name": "b", "score": None, "status": "failed"}, path)
    rs.register_run({"run_name": "a", "score": 26.5, "status": "complete"}, path)
    rows = rs.load_registry(path)
    assert [r["run_name"] for r in rows] == ["a", "b"] and rows[0]["score"] == 26.5
    text = rs.format_registry(rows)
    assert "run_name" in text and "26.5" in text
    assert rs.format_registry([]) == "no registered runs"
