"""``profile bench``: envelope, argument checks, forced routing, and the expert-parallel meshes over gloo ranks."""

import json

import pytest
import torch

from research_b200.errors import ContractError
from research_b200.runtime.profile_bench import (FixedRouter, benchmark_component, benchmark_to_json, format_benchmark,
                                                 percentile, routing_ids, timing_summary)
from tests.helpers import run_gloo


def test_timing_summary_and_percentiles():
    assert percentile([5.0], 0.9) == 5.0 and percentile([0.0, 10.0], 0.1) == pytest.approx(1.0)
    s = timing_summary([4.0, 1.0, 3.0, 2.0, 5.0])
    assert s == {"median": 3.0, "p10": pytest.approx(1.4), "p90": pytest.approx(4.6), "min": 1.0, "max": 5.0}


def test_forced_routing_is_balanced_or_fully_skewed():
    bal = routing_ids("balanced", 16, 2, 4, torch.device("cpu"))
    assert bal.shape == (1, 16, 2) and torch.bincount(bal.flatten(), minlength=4).tolist() == [8, 8, 8, 8]
    assert (bal[0, :, 0] != bal[0, :, 1]).all()                          # a token never picks one expert twice
    skew = routing_ids("skewed", 16, 2, 4, torch.device("cpu"))
    assert torch.bincount(skew.flatten(), minlength=4).tolist() == [16, 16, 0, 0]
    with pytest.raises(ContractError, match="unknown routing"):
        routing_ids("zipf", 16, 2, 4, torch.device("cpu"))
    router = FixedRouter(bal, 4)
    ids, w, scores = router(torch.zeros(1, 16, 8), torch.zeros(4))
    assert ids is bal and torch.allclose(w.sum(-1), torch.ones(1, 16)) and scores.shape == (1, 16, 4)


def test_argument_checks():
    for kwargs, match in ((dict(component="attention"), "unsupported profile benchmark component"),
                          (dict(component="moe", warmup=-1), "warmup must be non-negative"),
                          (dict(component="moe", iters=0), "iterations must be positive"),
                          (dict(component="muon", trace=True), "tracing requires --artifact-dir"),
                          (dict(component="moe", trace=True, artifact_dir="x"), "supported only for Muon")):
        with pytest.raises(ContractError, match=match):
            benchmark_component(**kwargs)


def test_moe_benchmark_single_process(tmp_path):
    report = benchmark_component("moe", warmup=0, iters=2, artifact_dir=str(tmp_path / "art"))
    assert report["kind"] == "directional_local_microbenchmark" and report["timing_is_acceptance_gate"] is False
    assert report["correctness_is_checked"] is False and report["device_count"] == 1 and report["iters"] == 2
    names = [c["name"] for c in report["cases"]]
    assert names == ["local_balanced_h32", "local_skewed_h32", "local_balanced_h256", "local_skewed_h256"]
    first = report["cases"][0]
    assert first["shape"] == {"tokens": 16, "hidden": 32, "intermediate": 64, "experts": 4, "top_k": 2}
    assert first["workload"] == "forward_backward" and first["timing_ms"]["min"] <= first["timing_ms"]["median"]
    assert first["max_tokens_on_one_expert"] == 8 and report["cases"][1]["max_tokens_on_one_expert"] == 16
    stored = json.loads((tmp_path / "art" / "moe_bench.json").read_text())
    assert stored["cases"][0]["name"] == names[0] and json.loads(benchmark_to_json(report))["component"] == "moe"
    text = format_benchmark(report)
    assert text.startswith("profile benchmark: component=moe backend=cpu") and "local_skewed_h256: first_call=" in text


def _bench_worker(rank, world):
    report = benchmark_component("moe", warmup=0, iters=1)
    return {"names": [c["name"] for c in report["cases"]], "meshes": [c["mesh"] for c in report["cases"]],
            "devices": report["device_count"], "finite": all(c["timing_ms"]["median"] > 0 for c in report["cases"])}


def test_moe_benchmark_shards_experts_over_the_ranks():
    two = run_gloo(2, _bench_worker)
    assert all(r == two[0] for r in two) and two[0]["devices"] == 2 and two[0]["finite"]
    assert two[0]["names"] == ["ep2_balanced_h32", "ep2_skewed_h32", "ep2_balanced_h256", "ep2_skewed_h256"]
    assert two[0]["meshes"][0] == {"data": 1, "ep": 2}
    four = run_gloo(4, _bench_worker)
    assert four[0]["devices"] == 4 and four[0]["finite"]
    assert {"ep4_balanced_h32", "ep2_efsdp2_balanced_h32", "ep2_efsdp2_skewed_h256"} <= set(four[0]["names"])
    assert {"fsdp": 1, "ep": 2, "expert_fsdp": 2} in four[0]["meshes"]


def test_muon_benchmark_envelope():
    report = benchmark_component("muon", warmup=0, iters=1)
    assert report["correctness_is_checked"] is True and report["component"] == "muon"
    assert report["known_correctness_constraint"] == "duplicated_five_step_calibrated_envelope"
    assert report["measurement_contract"]["reducer"] == "median" and report["timing_is_acceptance_gate"] is False
    text = format_benchmark(report)
    assert "component=muon" in text and "duplicated: median=" in text and "selected=" in text
