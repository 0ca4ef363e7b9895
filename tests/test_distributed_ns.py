"""Distributed Newton-Schulz over a tensor-parallel group: plans, Gram buckets, and the three executions against
the whole-matrix iteration (CPU ranks over gloo)."""

import pytest
import torch

from research_b200.config import run_spec_from_mapping
from research_b200.models.build import build_model
from research_b200.optim import distributed_ns as dns
from research_b200.optim import orthogonalize as orth
from research_b200.optim.build import build_optimizer, optimizer_policy_summary
from tests.helpers import run_gloo, tiny_dataset, tiny_raw_config, train_and_collect
from pathlib import Path


def test_execution_rule_and_buckets():
    assert dns.resolve_execution("duplicated", 1, (64, 256), 4) == ("duplicated", None)
    assert dns.resolve_execution("distributed", 1, (64, 256), 4) == ("distributed_direct", None)
    assert dns.resolve_execution("distributed", 0, (64, 256), 4) == ("distributed_exchange", None)
    assert dns.resolve_execution("distributed", 0, (64, 254), 4) == \
        ("duplicated", "exchange_long_dimension_not_divisible_by_tp")
    assert dns.resolve_execution("distributed_large_gram", 0, (64, 256), 4) == ("distributed_large_gram", None)
    # 2048-wide Grams are 8 MiB of bf16 each: four fill one 32 MiB bucket, the fifth opens the next
    plans = tuple(dns.MuonLeafPlan(f"layers.{i}.w", (2048, 8192), 1, False, 1, "distributed", "distributed_direct",
                                   None, -1, True) for i in range(5))
    plans += (dns.MuonLeafPlan("layers.0.o", (8192, 2048), 0, True, 1, "distributed", "distributed_direct", None, -1,
                               True),
              dns.MuonLeafPlan("layers.0.dup", (64, 64), 1, False, 1, "duplicated", "duplicated", None, -1, True))
    got = {p.name: p.bucket_id for p in dns.assign_bucket_ids(plans)}
    assert [got[f"layers.{i}.w"] for i in range(5)] == [1, 1, 1, 1, 2]       # "layers.0.o" sorts first: bucket 0
    assert got["layers.0.o"] == 0 and got["layers.0.dup"] == -1
    summary = dns.summarize_plans(dns.assign_bucket_ids(plans))
    assert summary["execution_counts"] == {"distributed_direct": 6, "duplicated": 1}
    assert summary["buckets"][1]["gram_payload_bytes"] == 4 * 2048 * 2048 * 2


def test_plans_come_with_the_optimizer_build():
    raw = tiny_raw_config(Path("m.json"), optimizer="muon")
    raw["optimizer"]["muon_tp_mode"] = "distributed"
    spec = run_spec_from_mapping(raw)
    res = build_model(spec.model, seed=0)
    built = build_optimizer(spec.optimizer, res.metadata, tp_size=2)
    plans = {p.name: p for p in built.muon_execution_plans}
    # hidden 64 -> intermediate 128: up/gate are split on the long (output) side, down on its long (input) side
    assert plans["layers.0.mlp.up.kernel"].execution == "distributed_direct"
    assert plans["layers.0.mlp.down.kernel"].execution == "distributed_direct"
    assert plans["layers.0.mlp.down.kernel"].transpose_for_shape
    assert plans["layers.0.attn.q.kernel"].execution in ("distributed_direct", "distributed_exchange")
    assert all(p.bucket_id >= 0 for p in plans.values())
    summary = optimizer_policy_summary(built)
    assert summary["muon_tp_execution"]["leaf_count"] == len(plans)
    assert optimizer_policy_summary(build_optimizer(spec.optimizer, res.metadata))["muon_tp_execution"] is None


def _bucket_worker(rank, world, execution, dtype_name):
    import torch.distributed as dist

    dtype = getattr(torch, dtype_name)
    torch.manual_seed(0)
    # storage orientation [out, in]; two shapes so that the bucket holds two stacks
    shapes = [(32, 96), (32, 96), (48, 64), (96, 32)]
    fulls = [torch.randn(s) * 0.05 for s in shapes]
    plans, axes, shards = [], [], []
    for k, (full, s) in enumerate(zip(fulls, shapes)):
        long_axis = 0 if s[0] > s[1] else 1
        axis = long_axis if execution == "distributed_direct" else 1 - long_axis
        plans.append(dns.MuonLeafPlan(f"w{k}", (s[1], s[0]), 1 - axis, s[1] > s[0], 1 if axis == long_axis else 0,
                                      "distributed", execution, None, 0, True))
        axes.append(axis)
        shards.append(full.chunk(world, dim=axis)[rank].contiguous())
    reducer = dns.TorchReducer(dist.group.WORLD)
    outs = dns.bucketed_distributed_zeropower(shards, plans, axes, dist.group.WORLD, reducer, dtype)
    again = dns.bucketed_distributed_zeropower(shards, plans, axes, dist.group.WORLD, dns.TorchReducer(dist.group.WORLD),
                                               dtype)
    errs = []
    for full, out, axis, rerun in zip(fulls, outs, axes, again):
        want = orth.zeropower_via_newton_schulz(full, precision="float32").chunk(world, dim=axis)[rank]
        assert out.shape == want.shape
        assert torch.equal(out, rerun)                       # run twice: same bits
        errs.append((out.float() - want).abs().max().item())
    return {"errs": errs, "reductions": reducer.reductions}


@pytest.mark.parametrize("execution", ["distributed_direct", "distributed_exchange", "distributed_large_gram"])
def test_bucketed_iteration_matches_the_whole_matrix(execution):
    exact = run_gloo(2, _bucket_worker, execution, "float32")
    for r in exact:
        assert max(r["errs"]) < 2e-5, r
        assert r["reductions"] == orth.MUON_NS_STEPS           # one packed reduction per step for four leaves
    envelope = run_gloo(2, _bucket_worker, execution, "bfloat16")
    for r in envelope:
        assert max(r["errs"]) < 2.5e-2, r                      # bf16 iteration against the fp32 one


@pytest.mark.parametrize("tp_mode", ["distributed"])
def test_training_with_distributed_muon_matches_one_process(tmp_path, tp_mode):
    manifest = tiny_dataset(tmp_path)
    base = tiny_raw_config(manifest, optimizer="muon", steps=4)
    ref = train_and_collect(0, 1, base, 3)
    raw = tiny_raw_config(manifest, optimizer="muon", mesh={"tp": 2},
                          parallelism={"mode": "ddp", "tensor_parallel": True}, steps=4)
    raw["optimizer"]["muon_tp_mode"] = tp_mode
    results = run_gloo(2, train_and_collect, raw, 3)
    for got in results:
        for a, b in zip(ref["loss_sum"], got["loss_sum"]):
            assert abs(a - b) <= 2e-3 * max(1.0, abs(a))
        for name, want in ref["model"].items():
            err = (got["model"][name] - want).abs().max().item()
            assert err <= 4e-3 * (1.0 + want.abs().max().item()), (name, err)
    for name, t in results[0]["model"].items():
        assert torch.equal(t, results[1]["model"][name]), name


def _selector_worker(rank, world):
    from research_b200.runtime.muon_bench import benchmark_muon

    return benchmark_muon(warmup=1, iters=2, cases="leaves")


def test_selector_checks_every_candidate_and_picks_one():
    from research_b200.runtime import muon_bench as mb

    assert mb.eligible_executions((1024, 256), 1, 4) == ("duplicated", "distributed_large_gram", "distributed_exchange")
    assert mb.eligible_executions((1024, 4096), 1, 4) == ("duplicated", "distributed_direct")
    assert mb.eligible_executions((4096, 1024), 0, 4) == ("duplicated", "distributed_direct")
    assert mb.eligible_executions((1024, 1024), 0, 4) == ("duplicated", "distributed_large_gram", "distributed_exchange")
    assert len(mb.calibration_bucket_cases()) == 14 and len(mb.PRODUCTION_BUCKETS) == 7
    assert mb.UPDATE_ATOL == pytest.approx(1.2e-2) and mb.PARAM_ATOL == pytest.approx(2.5e-2)
    reports = run_gloo(2, _selector_worker)
    report = reports[0]
    assert report["tp_size"] == 2 and len(report["cases"]) == 7 and report["all_selected_pass"]
    for case in report["cases"]:
        by = {c["execution"]: c for c in case["candidates"]}
        assert by["duplicated"]["max_update_abs_error"] == 0.0 and by["duplicated"]["correctness_gate"]
        for name, c in by.items():
            assert c["finite"] and c["momentum_exact"] and c["deterministic"], (case["case"], name, c)
            assert c["replica_max_abs_error"] == 0.0 and c["correctness_gate"], (case["case"], name, c)
            assert c["timing_ms"]["min"] <= c["timing_ms"]["median"] <= c["timing_ms"]["max"]
        assert case["selected"] in by and case["selection_reason"] in ("fastest_passing_candidate",
                                                                        "gain_below_selection_min_speedup")
        chosen, dup = by[case["selected"]], by["duplicated"]
        if case["selected"] != "duplicated":                                # a distributed pick needs a clear gain
            assert dup["timing_ms"]["median"] / chosen["timing_ms"]["median"] >= mb.SELECTION_MIN_SPEEDUP
        assert all(c["stability"] >= 0 and isinstance(c["stable"], bool) for c in by.values())
    kv = next(c for c in report["cases"] if c["case"] == "attention_kv")
    assert {c["execution"] for c in kv["candidates"]} == {"duplicated", "distributed_large_gram", "distributed_exchange"}
    assert reports[1]["selection"] == report["selection"]              # every rank reaches the same verdict
    contract = report["contract"]
    assert contract == mb.benchmark_contract() and contract["selection_min_speedup"] == 1.05
    assert contract["update_atol"] == mb.UPDATE_ATOL and contract["stability_limit"] == 0.05
    assert contract["timing_is_production_acceptance_gate"] is False and contract["correctness_steps"] == 5
