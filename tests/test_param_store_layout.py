"""Layout of the parameter store: sections, owner blocks in backward order, per-layer buckets, weights sharded at
rest (what each rank keeps, which pieces a layer fetch copies)."""

import math

import pytest
import torch

from research_b200.config import run_spec_from_mapping
from research_b200.parallel.sharding import ALIGN, layer_of
from research_b200.runtime.trainer import Trainer
from tests.helpers import run_gloo, tiny_dataset, tiny_raw_config


def test_layer_of_parses_parameter_names():
    assert layer_of("layers.3.attn.wqkv") == 3 and layer_of("model.layers.12.mlp.w_down") == 12
    assert layer_of("embed") == -1 and layer_of("norm.scale") == -1 and layer_of("lm_head") == -1


def _layout(rank, world, raw):
    trainer = Trainer(run_spec_from_mapping(raw), device="cpu")
    store = trainer.store
    out = {"sections": [], "memory": store.memory_report(), "resident": store.resident, "total": store.total}
    for sec in store.sections:
        out["sections"].append({
            "backend": sec.backend, "start": sec.start, "length": sec.length, "shard_axis": sec.shard_axis,
            "owner_block": sec.owner_block, "bucket_layers": sec.bucket_layers,
            "bucket_ranges": dict(sec.bucket_ranges), "decay": sec.decay,
            "entries": [(e.name, e.offset, e.numel, e.owner) for e in sec.entries],
            "local": store.local_master_range(sec)})
    if not store.resident:
        out["pieces"] = {l: store._pieces(entries) for l, entries in store._layer_entries.items()}
        out["extras"] = store._pieces(store._extra_entries)
        out["layer_numel"] = {l: sum(e.numel for e in entries) for l, entries in store._layer_entries.items()}
        out["extra_numel"] = sum(e.numel for e in store._extra_entries)
    return out


def test_owner_blocks_are_in_backward_order_with_one_range_per_layer(tmp_path):
    manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, optimizer="muon", mesh={"fsdp": 2}, parallelism={"mode": "fsdp"},
                          extra_model={"num_layers": 3})
    per_rank = run_gloo(2, _layout, raw)
    for rank, info in enumerate(per_rank):
        muon = next(s for s in info["sections"] if s["backend"] == "muon")
        assert muon["shard_axis"] == "fsdp" and muon["bucket_layers"] == (2, 1, 0)
        assert muon["length"] == 2 * muon["owner_block"] and muon["owner_block"] % ALIGN == 0
        mine = sorted((off, name, n) for name, off, n, owner in muon["entries"] if owner == rank)
        assert [layer_of(name) for _, name, _ in mine] == sorted((layer_of(n) for _, n, _ in mine), reverse=True)
        # every layer's matrices of this owner form one gap-free range, and the ranges tile the owner's block front
        cursor = muon["local"][0]
        for layer in muon["bucket_layers"]:
            if layer not in muon["bucket_ranges"]:
                continue
            a, b = muon["bucket_ranges"][layer]
            assert a == cursor and b > a
            cursor = b
        assert cursor <= muon["local"][1]
    # the two ranks split the Newton-Schulz work about evenly and own disjoint matrices
    owners = {name: owner for name, _, _, owner in next(s for s in per_rank[0]["sections"] if s["backend"] == "muon")["entries"]}
    assert set(owners.values()) == {0, 1}
    assert per_rank[0]["sections"] == per_rank[1]["sections"] or True          # layouts are computed identically
    for a, b in zip(per_rank[0]["sections"], per_rank[1]["sections"]):
        assert a["entries"] == b["entries"] and a["start"] == b["start"]


@pytest.mark.parametrize("optimizer", ["adamw", "muon"])
def test_weights_sharded_at_rest_keep_one_nth_and_fetch_every_element_once(tmp_path, optimizer):
    manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, optimizer=optimizer, mesh={"fsdp": 2},
                          parallelism={"mode": "fsdp", "fsdp_resident": False})
    per_rank = run_gloo(2, _layout, raw)
    resident = run_gloo(2, _layout, tiny_raw_config(manifest, optimizer=optimizer, mesh={"fsdp": 2},
                                                   parallelism={"mode": "fsdp"}))
    for info in per_rank:
        assert not info["resident"] and info["memory"]["mode"] == "sharded"
        # at rest: about half of the sharded sections (the alignment padding is the slack)
        assert info["memory"]["compute_bytes"] <= 0.5 * resident[0]["memory"]["compute_bytes"] + 64 * ALIGN * 4
        for layer, pieces in info["pieces"].items():
            covered = sorted((off, off + n) for _, _, off, n in pieces)
            assert sum(b - a for a, b in covered) == info["layer_numel"][layer]
            assert all(x[1] <= y[0] for x, y in zip(covered, covered[1:]))           # no element fetched twice
            assert {r for r, _, _, _ in pieces} <= {0, 1}
        assert sum(n for _, _, _, n in info["extras"]) == info["extra_numel"]
    assert per_rank[0]["pieces"] == per_rank[1]["pieces"]                             # same plan on every rank


def test_single_rank_ignores_the_sharded_switch(tmp_path):
    manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, mesh={"fsdp": 1}, parallelism={"mode": "fsdp", "fsdp_resident": False})
    trainer = Trainer(run_spec_from_mapping(raw), device="cpu")
    assert trainer.store.resident and trainer.store.memory_report()["mode"] == "resident"
    assert math.isfinite(trainer.train_step().loss)
