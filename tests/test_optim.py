"""Schedules, orthogonalisation, Dion2 selection, routing, AdamW against torch."""

import math

import pytest
import torch

from research_b200.config import run_spec_from_mapping
from research_b200.config.specs import OptimizerSpec, ParamRouteRule, ScheduleSpec
from research_b200.errors import ContractError
from research_b200.models.build import build_model
from research_b200.optim import orthogonalize as orth
from research_b200.optim.build import build_optimizer, optimizer_policy_summary, route_assignments
from research_b200.optim.schedules import build_lr_schedule
from tests.helpers import tiny_raw_config
from pathlib import Path


def test_schedules():
    const = build_lr_schedule(ScheduleSpec(peak_lr=1.0, warmup_steps=4))
    assert [const(i) for i in range(6)] == [0.25, 0.5, 0.75, 1.0, 1.0, 1.0]
    cos = build_lr_schedule(ScheduleSpec(peak_lr=1.0, name="cosine", warmup_steps=2, total_steps=6, min_lr_ratio=0.1))
    assert cos(0) == 0.5 and cos(1) == 1.0 and cos(2) == pytest.approx(1.0)
    assert cos(5) == pytest.approx(0.1) and cos(100) == pytest.approx(0.1)
    assert cos(3) == pytest.approx(0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi / 3)))
    wsd = build_lr_schedule(ScheduleSpec(peak_lr=2.0, name="wsd", warmup_steps=1, stable_steps=2, total_steps=6))
    assert [round(wsd(i), 6) for i in range(3)] == [2.0, 2.0, 2.0] and wsd(5) == pytest.approx(0.0)
    with pytest.raises(ContractError, match="total_steps is required"):
        build_lr_schedule(ScheduleSpec(peak_lr=1.0, name="cosine"))


@pytest.mark.parametrize("shape", [(48, 96), (96, 48), (3, 32, 64)])
def test_newton_schulz_pushes_singular_values_towards_one(shape):
    torch.manual_seed(0)
    x = torch.randn(shape)
    o = orth.zeropower_via_newton_schulz(x, precision="float32")
    s = torch.linalg.svdvals(o)
    assert s.max() < 1.3 and s.min() > 0.5
    # transposition commutes with the iteration (storage is [out, in], the reference's is [in, out])
    ot = orth.zeropower_via_newton_schulz(x.transpose(-1, -2).contiguous(), precision="float32")
    assert torch.allclose(ot.transpose(-1, -2), o, atol=1e-4)


def test_polar_express_and_dion2_selection():
    torch.manual_seed(1)
    x = torch.randn(32, 80)
    s = torch.linalg.svdvals(orth.polar_express(x).float())
    assert s.max() < 1.3 and s.min() > 0.4
    m = torch.zeros(8, 4)
    m[2] = 5.0
    m[5] = -3.0
    rows, idx = orth.select_dion2_slices(m, select_axis=0)
    assert sorted(idx.tolist()) == [2, 5] and rows.shape == (2, 4)
    cols, cidx = orth.select_dion2_slices(m.t().contiguous(), select_axis=1)
    assert sorted(cidx.tolist()) == [2, 5] and cols.shape == (4, 2)
    with pytest.raises(ValueError):
        orth.select_dion2_slices(m, select_axis=2)
    assert orth.rms_match_scale((64, 256)) == pytest.approx(0.2 * 16.0)


def test_routing_by_tag():
    spec = run_spec_from_mapping(tiny_raw_config(Path("m.json"), kind="trinity", optimizer="muon"))
    res = build_model(spec.model, seed=0)
    built = build_optimizer(spec.optimizer, res.metadata)
    by = {a.name: a for a in built.route_assignments}
    assert by["embed.embedding"].backend == "adamw" and by["embed.embedding"].fallback_reason == "embedding"
    assert by["lm_head.kernel"].backend == "adamw" and by["norm.scale"].fallback_reason == "norm"
    assert by["layers.0.attn.q.kernel"].backend == "muon" and by["layers.1.mlp.experts.gate"].backend == "muon"
    assert by["layers.1.mlp.router.proj.kernel"].backend == "adamw"
    assert by["layers.1.mlp.expert_bias"].weight_decay is False
    summary = optimizer_policy_summary(built)
    assert summary["backend_parameter_counts"]["muon"] > 0 and summary["muon"]["newton_schulz_steps"] == 5
    tp = route_assignments(spec.optimizer, res.metadata, tp_size=2)
    assert {a.name: a for a in tp}["layers.0.attn.o.kernel"].backend == "dist_muon"
    dion = build_optimizer(OptimizerSpec(name="dion", schedule=ScheduleSpec(peak_lr=1e-3)), res.metadata)
    assert {a.name: a for a in dion.route_assignments}["layers.0.mlp.down.kernel"].backend == "dion2"
    with pytest.raises(ContractError, match="does not match any model parameter"):
        route_assignments(OptimizerSpec(name="adamw", schedule=ScheduleSpec(peak_lr=1e-3),
                                        route_rules=(ParamRouteRule("nope", "adamw"),)), res.metadata)
    with pytest.raises(ContractError, match="no runtime adapter"):
        build_optimizer(OptimizerSpec(name="soap", schedule=ScheduleSpec(peak_lr=1e-3)), res.metadata)


def test_policy_summary_sections():
    from research_b200.optim.build import (describe_optimizer, dist_muon_policy_payload, distributed_policy_payload,
                                           route_distributed_policy, schedule_payload)

    raw = tiny_raw_config(Path("m.json"), kind="trinity", optimizer="muon")
    raw["optimizer"]["schedule"] = {"peak_lr": 2e-3, "name": "wsd", "warmup_steps": 2, "total_steps": 40,
                                    "stable_steps": 30, "min_lr_ratio": 0.1}
    raw["optimizer"]["adamw_fallback_schedule"] = {"peak_lr": 1e-3, "warmup_steps": 1}
    spec = run_spec_from_mapping(raw)
    res = build_model(spec.model, seed=0)
    built = build_optimizer(spec.optimizer, res.metadata, tp_size=2)
    s = optimizer_policy_summary(built, res.metadata)
    assert s["name"] == s["requested_name"] == "muon" and s["supported_runtime_backends"] == ["adamw", "dion", "muon"]
    assert s["schedule"] == {"name": "wsd", "peak_lr": 2e-3, "warmup_steps": 2, "total_steps": 40,
                             "min_lr_ratio": 0.1, "stable_steps": 30}
    assert s["adamw_fallback_schedule"]["peak_lr"] == 1e-3 and s["adamw_fallback_schedule"]["name"] == "constant"
    assert s["route_counts"] == s["backend_parameter_counts"] and sum(s["route_counts"].values()) == len(res.metadata)
    assert set(s["route_counts"]) == {"adamw", "dist_muon", "muon"}              # experts stay whole: plain muon
    assert s["fallback_counts"]["norm"] > 0 and s["fallback_counts"]["embedding"] == 1
    assert s["auto_routing"]["active"] is True and s["auto_routing"]["muon_tp_sharded_matrix_backend"] == "dist_muon"
    assert s["distributed_policy"]["zero2_fsdp"] == "owner_distributed_muon"
    assert s["muon"]["tp_mode"] == spec.optimizer.muon_tp_mode and "attention_q" in s["muon"]["hidden_matrix_tags"]
    assert "moe_gate" in s["muon"]["routed_expert_matrix_tags"] and s["dion2"] is None
    route = next(r for r in s["routes"] if r["path"] == "layers.0.attn.q.kernel")
    assert route["backend"] == "dist_muon" and route["logical_shape"] == [64, 64] and route["auto_resolved"]
    assert route["distributed_policy"] in ("duplicated_full_logical_matrix", "sharded_gram_collectives")
    plans = s["dist_muon"]["leaf_execution_plans"]
    assert len(plans) == s["route_counts"]["dist_muon"] and {"path", "execution", "bucket_id"} <= set(plans[0])
    assert optimizer_policy_summary(built)["routes"][0]["logical_shape"] is None      # shapes need the metadata
    # the fixed payloads
    dup = dist_muon_policy_payload(OptimizerSpec(name="muon", schedule=ScheduleSpec(peak_lr=1e-3), muon_tp_mode="duplicated"))
    dis = dist_muon_policy_payload(OptimizerSpec(name="muon", schedule=ScheduleSpec(peak_lr=1e-3), muon_tp_mode="distributed"))
    assert dup["exact"] is True and dup["execution"] == "duplicated" and dis["exact"] is False
    assert dis["distributed_policy"] == "sharded_gram_collectives"
    assert distributed_policy_payload("adamw")["zero2_fsdp"] == "supported"
    assert distributed_policy_payload("soap")["zero2_fsdp"] == "unsupported"
    assert route_distributed_policy("adamw", muon_tp_mode="distributed") == "elementwise_shard_safe"
    assert route_distributed_policy("dist_muon", muon_tp_mode="duplicated") == "duplicated_full_logical_matrix"
    assert route_distributed_policy("other", muon_tp_mode="duplicated") == "unknown" and schedule_payload(None) is None
    text = describe_optimizer(spec.optimizer)
    assert "schedule=wsd" in text and "stable_steps=30" in text and "adamw_fallback_schedule=constant:peak_lr=0.001" in text
    adamw = build_optimizer(OptimizerSpec(name="adamw", schedule=ScheduleSpec(peak_lr=1e-3)), res.metadata)
    plain = optimizer_policy_summary(adamw, res.metadata)
    assert plain["muon"] is None and plain["fallback_counts"] == {} and plain["auto_routing"]["active"] is False
    assert plain["muon_tp_execution"] is None and "leaf_execution_plans" not in plain["dist_muon"]


def test_adamw_step_matches_torch(tmp_path):
    from tests.helpers import tiny_dataset
    from research_b200.runtime.trainer import Trainer

    manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, clip=None)
    raw["optimizer"]["schedule"] = {"peak_lr": 1e-2}
    trainer = Trainer(run_spec_from_mapping(raw), device="cpu")
    params = [e.param for e in trainer.store.entries]
    ref = [p.detach().clone().requires_grad_(True) for p in params]
    opt = torch.optim.AdamW(ref, lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    for _ in range(2):
        trainer.store.zero_grads()
        for p, r in zip(params, ref):
            g = torch.randn_like(p)
            p.main_grad.copy_(g)
            r.grad = g.clone()
        trainer.optimizer.step()
        opt.step()
    for p, r in zip(params, ref):
        assert torch.allclose(p, r, atol=1e-6, rtol=1e-5)


def test_adamw_route_rule_without_weight_decay_is_not_decayed(tmp_path):
    """A route rule with ``weight_decay = false`` on an AdamW-routed tag masks the decay for those parameters only
    (reference: src/jaxtitan/optim/build.py:506-518)."""

    from tests.helpers import tiny_dataset
    from research_b200.runtime.trainer import Trainer

    manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, clip=None)
    raw["optimizer"]["schedule"] = {"peak_lr": 1e-2}
    raw["optimizer"]["weight_decay"] = 0.5
    import dataclasses

    spec = run_spec_from_mapping(raw)
    rule = ParamRouteRule("final_norm", "adamw", weight_decay=False)
    spec = dataclasses.replace(spec, optimizer=dataclasses.replace(spec.optimizer, route_rules=(rule,)))
    trainer = Trainer(spec, device="cpu")
    by_decay = {sec.decay for sec in trainer.store.sections if sec.backend == "adamw"}
    assert by_decay == {True, False}
    before = {e.name: e.param.detach().clone() for e in trainer.store.entries}
    trainer.store.zero_grads()                       # zero gradients: only the decay moves a parameter
    trainer.optimizer.step()
    for e in trainer.store.entries:
        moved = not torch.equal(e.param.detach(), before[e.name])
        is_norm = all(m.tag == "final_norm" for m in e.metas)
        assert moved != is_norm, (e.name, moved)


def _newton_schulz_restated(x):
    """The quintic iteration spelled out (bf16, left Gram of the wide orientation)."""

    x = x.to(torch.bfloat16)
    x = x / torch.clamp(torch.linalg.matrix_norm(x.float()).to(torch.bfloat16), min=1e-7)
    wide = x.shape[0] <= x.shape[1]
    if not wide:
        x = x.t()
    a, b, c = 3.4445, -4.7750, 2.0315
    for _ in range(5):
        gram = x @ x.t()
        x = a * x + (b * gram + c * (gram @ gram)) @ x
    return (x if wide else x.t()).float()


@pytest.mark.parametrize("kind", ["decoder", "trinity"])
def test_muon_step_matches_the_update_rule(tmp_path, kind):
    """``m <- 0.95 m + 0.05 g``; Nesterov input ``0.05 g + 0.95 m``; five Newton-Schulz steps in bf16; step
    ``lr * 0.2 * sqrt(max(rows, cols))``; decoupled decay ``lr * wd * p`` (reference: src/jaxtitan/optim/muon.py:97-127)."""

    from tests.helpers import tiny_dataset
    from research_b200.runtime.trainer import Trainer

    manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, kind=kind, optimizer="muon", clip=None)
    raw["optimizer"]["schedule"] = {"peak_lr": 2e-2}
    raw["optimizer"]["weight_decay"] = 0.1
    trainer = Trainer(run_spec_from_mapping(raw), device="cpu")
    lr, wd = 2e-2, 0.1
    entries = [e for e in trainer.store.entries if e.backend == "muon"]
    assert entries and any(e.param.dim() == 3 for e in entries) == (kind == "trinity")
    torch.manual_seed(0)
    momentum = {e.name: torch.zeros_like(e.param) for e in entries}
    expected = {e.name: e.param.detach().clone() for e in entries}
    for _ in range(2):
        trainer.store.zero_grads()
        grads = {}
        for e in trainer.store.entries:
            g = torch.randn_like(e.param) * 0.1
            e.param.main_grad.copy_(g)
            grads[e.name] = g
        for e in entries:
            g, m, w = grads[e.name], momentum[e.name], expected[e.name]
            m.mul_(0.95).add_(g, alpha=0.05)
            inp = 0.05 * g + 0.95 * m
            for meta in e.metas:
                rows = slice(None) if meta.rows is None else slice(*meta.rows)
                blocks = [(inp[x, rows], w[x, rows]) for x in range(w.shape[0])] if w.dim() == 3 else [(inp[rows], w[rows])]
                for block_in, block_w in blocks:
                    step = lr * 0.2 * math.sqrt(max(block_in.shape))
                    block_w.mul_(1.0 - lr * wd).add_(_newton_schulz_restated(block_in), alpha=-step)
        trainer.optimizer.step()
    for e in entries:
        step = lr * 0.2 * math.sqrt(max(e.param.shape[-2:]))
        # a momentum of 0.90 instead of 0.95 already moves entries by 0.02 of a step after two updates
        assert torch.allclose(e.param.detach(), expected[e.name], atol=0.004 * step, rtol=0), e.name
    # everything else took AdamW: embedding, head, norms, router
    others = {m.tag for e in trainer.store.entries if e.backend == "adamw" for m in e.metas}
    assert {"embedding", "lm_head", "final_norm"} <= others


def _polar_express_restated(x):
    x = x.to(torch.bfloat16)
    x = x / (torch.linalg.matrix_norm(x.float()).to(torch.bfloat16) * 1.02 + 1e-8)
    tall = x.shape[0] > x.shape[1]
    for a, b, c in orth.DION2_POLAR_EXPRESS_COEFFICIENTS:
        gram = x.t() @ x if tall else x @ x.t()
        poly = b * gram + c * (gram @ gram)
        x = a * x + (x @ poly if tall else poly @ x)
    return x.float()


def test_dion2_step_matches_the_update_rule(tmp_path):
    """Momentum takes the whole gradient; the quarter of the rows (or columns) with the largest L1 norm is
    orthogonalised with Polar Express, applied with ``lr * sqrt(fan_in / fan_out)`` and kept in the momentum at 0.95
    of its value; the rest of the momentum stays (reference: src/jaxtitan/optim/dion2.py:62-98)."""

    from tests.helpers import tiny_dataset
    from research_b200.runtime.trainer import Trainer

    manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, optimizer="dion", clip=None)
    raw["optimizer"]["schedule"] = {"peak_lr": 1e-2}
    raw["optimizer"]["weight_decay"] = 0.1
    trainer = Trainer(run_spec_from_mapping(raw), device="cpu")
    lr, wd = 1e-2, 0.1
    routes = {a.name: a for a in trainer.optimizer_build.route_assignments}
    entries = [e for e in trainer.store.entries if e.backend == "dion2"]
    assert entries
    torch.manual_seed(0)
    momentum = {e.name: torch.zeros_like(e.param) for e in entries}
    expected = {e.name: e.param.detach().clone() for e in entries}
    for _ in range(3):
        trainer.store.zero_grads()
        grads = {}
        for e in trainer.store.entries:
            g = torch.randn_like(e.param) * 0.1
            e.param.main_grad.copy_(g)
            grads[e.name] = g
        for e in entries:
            momentum[e.name].add_(grads[e.name])
            for meta in e.metas:
                rows = slice(None) if meta.rows is None else slice(*meta.rows)
                m, w = momentum[e.name][rows], expected[e.name][rows]
                logical_axis = routes[meta.name].matrix_axis or 0
                axis = (1 - logical_axis) if meta.transposed else logical_axis      # in the stored orientation
                k = max(1, math.ceil(0.25 * m.shape[axis]))
                idx = m.abs().sum(dim=1 - axis).topk(k).indices
                picked = m.index_select(axis, idx)
                fan_in, fan_out = meta.shape                                         # logical [in, out]
                w.mul_(1.0 - lr * wd)
                w.index_add_(axis, idx, _polar_express_restated(picked), alpha=-lr * math.sqrt(fan_in / fan_out))
                m.index_copy_(axis, idx, picked * 0.95)
        trainer.optimizer.step()
    for e in entries:
        assert torch.allclose(e.param.detach(), expected[e.name], atol=2e-5, rtol=0), e.name
    # the error-feedback part of the momentum: rows never picked hold the plain sum of their gradients
    probe = entries[0]
    state_mom = None
    for i, sec in enumerate(trainer.store.sections):
        if probe in sec.entries:
            lo, _ = trainer.store.local_master_range(sec)
            state_mom = trainer.optimizer.state[i]["momentum"][probe.offset - lo:probe.offset - lo + probe.numel]
    assert torch.allclose(state_mom.view(probe.param.shape), momentum[probe.name], atol=1e-6)
