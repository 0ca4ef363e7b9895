"""Mesh specs, axis policies, batch slicing and, over gloo ranks, the process groups of every axis."""

import numpy as np
import pytest
import torch

from research_b200.config.specs import (ExpertFSDPPolicy, MeshSpec, ParallelismSpec, resolve_expert_fsdp_axis,
                                        resolve_expert_parallel_axis)
from research_b200.errors import ContractError
from research_b200.parallel.mesh import (MeshContext, build_mesh_context, execution_context_for,
                                         require_single_node_runtime)
from research_b200.steps.train import local_batch_slices
from tests.helpers import run_gloo


def _ctx(names, sizes, rank):
    coords = dict(zip(names, (int(c) for c in np.unravel_index(rank, sizes))))
    return MeshContext(tuple(names), tuple(sizes), rank, int(np.prod(sizes)), coords)


def test_mesh_spec_validation_and_aliases():
    spec = MeshSpec(axis_names=("data", "tensor", "context", "expert"), axis_sizes=(2, 2, 1, 2))
    assert spec.axis_names == ("data", "tp", "cp", "ep") and spec.device_count == 8
    assert spec.sizes == {"data": 2, "tp": 2, "cp": 1, "ep": 2}
    assert MeshSpec().axis_names == ("data",) and MeshSpec().device_count == 1
    for kwargs, match in ((dict(axis_names=("data", "tp"), axis_sizes=(2,)), "same length"),
                          (dict(axis_names=(), axis_sizes=()), "at least one axis"),
                          (dict(axis_names=("data", "data"), axis_sizes=(1, 2)), "must be unique"),
                          (dict(axis_names=("tp", "tensor"), axis_sizes=(1, 2)), "must be unique"),
                          (dict(axis_names=("data", ""), axis_sizes=(1, 2)), "non-empty"),
                          (dict(axis_names=("data",), axis_sizes=(0,)), "must be positive")):
        with pytest.raises(ContractError, match=match):
            MeshSpec(**kwargs)


def test_mesh_context_accessors():
    ctx = _ctx(("data", "fsdp", "tp"), (2, 2, 2), rank=5)
    assert ctx.coords == {"data": 1, "fsdp": 0, "tp": 1} and ctx.size("tp") == 2 and ctx.size("cp") == 1
    assert ctx.coord("fsdp") == 0 and ctx.coord("ep") == 0 and ctx.group("tp") is None
    assert ctx.sizes == {"data": 2, "fsdp": 2, "tp": 2} and ctx.replica_axes() == ("data", "fsdp")
    assert _ctx(("data", "tp"), (1, 4), 2).replica_axes() == ()
    d = ctx.describe()
    assert d["axis_names"] == ["data", "fsdp", "tp"] and d["device_count"] == 8 and d["rank"] == 5


def test_unknown_axis_and_wrong_device_count_are_refused():
    with pytest.raises(ContractError, match="unsupported mesh axis 'pipeline'"):
        build_mesh_context(MeshSpec(axis_names=("pipeline",), axis_sizes=(1,)))
    with pytest.raises(ContractError, match=r"need 4 devices but the job has 1 ranks"):
        build_mesh_context(MeshSpec(axis_names=("data", "tp"), axis_sizes=(2, 2)))
    one = build_mesh_context(MeshSpec(axis_names=("data", "tp"), axis_sizes=(1, 1)), device=torch.device("cpu"))
    assert one.world_size == 1 and one.rank == 0 and one.groups == {} and one.device.type == "cpu"


def test_multi_node_launches_are_refused(monkeypatch):
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "4")
    require_single_node_runtime(4)
    with pytest.raises(ContractError, match="multi-node runs are not supported: world_size=8 but LOCAL_WORLD_SIZE=4"):
        require_single_node_runtime(8)
    monkeypatch.delenv("LOCAL_WORLD_SIZE")
    require_single_node_runtime(8)


def test_expert_axis_resolution():
    off = resolve_expert_parallel_axis(ParallelismSpec(), {"data": 2})
    assert off.enabled is False
    ep = resolve_expert_parallel_axis(ParallelismSpec(expert_parallel=True), {"data": 1, "ep": 4})
    assert (ep.enabled, ep.axis, ep.axis_size, ep.axis_sharing) == (True, "ep", 4, "dedicated_ep")
    folded = resolve_expert_parallel_axis(ParallelismSpec(mode="fsdp", expert_parallel=True), {"fsdp": 4})
    assert (folded.axis, folded.axis_sharing) == ("fsdp", "shared_with_fsdp")
    prefers_ep = resolve_expert_parallel_axis(ParallelismSpec(mode="fsdp", expert_parallel=True), {"fsdp": 2, "ep": 2})
    assert prefers_ep.axis == "ep"
    data = resolve_expert_parallel_axis(ParallelismSpec(expert_parallel=True, expert_parallel_axis="data"), {"data": 4})
    assert (data.axis, data.axis_sharing, data.axis_size) == ("data", "shared_with_data", 4)
    for par, sizes, match in (
            (ParallelismSpec(expert_parallel=True), {"data": 4}, "requires a mesh ep axis or"),
            (ParallelismSpec(expert_parallel=True, expert_parallel_axis="fsdp"), {"fsdp": 2}, "requires parallelism.mode='fsdp'"),
            (ParallelismSpec(expert_parallel=True, expert_parallel_axis="ep"), {"data": 2}, "requires a mesh ep axis")):
        with pytest.raises(ContractError, match=match):
            resolve_expert_parallel_axis(par, sizes)
    with pytest.raises(ContractError, match="expert_parallel_axis must be one of"):
        ParallelismSpec(expert_parallel=True, expert_parallel_axis="tp")


def test_expert_fsdp_axis_resolution():
    assert resolve_expert_fsdp_axis(ParallelismSpec(), {"data": 2}) == ExpertFSDPPolicy(enabled=False)
    assert resolve_expert_fsdp_axis(ParallelismSpec(), {"expert_fsdp": 1}).enabled is False
    on = resolve_expert_fsdp_axis(ParallelismSpec(mode="fsdp", expert_parallel=True), {"fsdp": 1, "ep": 2, "expert_fsdp": 2})
    assert on.enabled and on.axis == "expert_fsdp" and on.axis_size == 2
    for par, sizes, match in (
            (ParallelismSpec(expert_parallel=True), {"ep": 2, "expert_fsdp": 2}, "requires parallelism.mode='fsdp'"),
            (ParallelismSpec(mode="fsdp"), {"fsdp": 2, "expert_fsdp": 2}, "requires parallelism.expert_parallel=true"),
            (ParallelismSpec(mode="fsdp", expert_parallel=True), {"fsdp": 2, "expert_fsdp": 2}, "dedicated expert_parallel_axis='ep'")):
        with pytest.raises(ContractError, match=match):
            resolve_expert_fsdp_axis(par, sizes)


def test_parallelism_spec_rules():
    for kwargs, match in ((dict(mode="pipeline"), "parallelism.mode"),
                          (dict(vocab_parallel_head=True), "requires parallelism.tensor_parallel=true"),
                          (dict(fsdp_resident=False), "requires parallelism.mode='fsdp'"),
                          (dict(context_attention="ring2"), "parallelism.context_attention"),
                          (dict(tensor_parallel="yes"), "parallelism.tensor_parallel")):
        with pytest.raises(ContractError, match=match):
            ParallelismSpec(**kwargs)
    ok = ParallelismSpec(mode="fsdp", fsdp_resident=False, tensor_parallel=True, vocab_parallel_head=True)
    assert ok.fsdp_resident is False and ok.vocab_parallel_head is True


def test_execution_context_follows_the_mesh_and_the_switches():
    mesh = _ctx(("data", "tp", "ep"), (1, 1, 1), 0)
    ex = execution_context_for(mesh, ParallelismSpec())
    assert (ex.tp_size, ex.cp_size, ex.ep_size, ex.efsdp_size, ex.sp) == (1, 1, 1, 1, False)
    assert ex.ep_dispatcher == "all_to_all" and ex.ep_axis_name is None and ex.vocab_parallel is False
    moe = execution_context_for(mesh, ParallelismSpec(expert_parallel=True))
    assert moe.ep_axis_name == "ep" and moe.ep_axis_sharing == "dedicated_ep" and moe.ep_dispatcher == "all_to_all"
    shared = execution_context_for(_ctx(("data",), (1,), 0), ParallelismSpec(expert_parallel=True, expert_parallel_axis="data"))
    assert shared.ep_dispatcher == "rdep_static" and shared.ep_axis_sharing == "shared_with_data"
    uly = execution_context_for(_ctx(("data", "cp"), (1, 1), 0), ParallelismSpec(context_parallel=True, context_attention="ulysses"))
    assert uly.cp_attention == "ulysses"
    head = execution_context_for(_ctx(("data", "tp"), (1, 1), 0), ParallelismSpec(tensor_parallel=True, vocab_parallel_head=True))
    assert head.vocab_parallel is True and execution_context_for(mesh, ParallelismSpec(), fused=False).fused is False


@pytest.mark.parametrize("rank, rows, dp_rank", [(0, 4, 0), (1, 4, 0), (2, 4, 1), (5, 4, 2), (7, 4, 3)])
def test_batch_rows_split_over_data_then_fsdp(rank, rows, dp_rank):
    mesh = _ctx(("data", "fsdp", "tp"), (2, 2, 2), rank)
    r, c = local_batch_slices(mesh, 16, 32)
    assert (r.start, r.stop) == (dp_rank * rows, (dp_rank + 1) * rows) and c == slice(0, 32)


def test_context_parallel_ranks_take_zigzag_halves_that_tile_the_sequence():
    seen = []
    for rank in range(4):
        rows, cols = local_batch_slices(_ctx(("data", "cp"), (1, 4), rank), 8, 64)
        assert (rows.start, rows.stop) == (0, 8) and len(cols) == 16
        seen.append(np.asarray(cols))
    assert sorted(np.concatenate(seen).tolist()) == list(range(64))
    first = seen[0].tolist()
    assert first[:8] == list(range(0, 8)) and first[8:] == list(range(56, 64))         # one early and one late chunk


def _groups_worker(rank, world):
    import torch.distributed as dist

    mesh = build_mesh_context(MeshSpec(axis_names=("data", "tp", "cp"), axis_sizes=(2, 2, 1)), device=torch.device("cpu"))
    out = {"coords": mesh.coords, "sizes": {a: mesh.size(a) for a in ("data", "tp", "cp", "ep")}}
    for axis in ("data", "tp"):
        group = mesh.group(axis)
        members = [None] * dist.get_world_size(group)
        dist.all_gather_object(members, rank, group=group)
        total = torch.tensor([float(rank)])
        dist.all_reduce(total, group=group)
        out[axis] = (members, float(total))
    out["cp_group"] = mesh.group("cp")
    return out


def test_process_groups_follow_row_major_coordinates():
    got = run_gloo(4, _groups_worker)
    assert [g["coords"] for g in got] == [{"data": 0, "tp": 0, "cp": 0}, {"data": 0, "tp": 1, "cp": 0},
                                          {"data": 1, "tp": 0, "cp": 0}, {"data": 1, "tp": 1, "cp": 0}]
    assert got[0]["tp"] == ([0, 1], 1.0) and got[3]["tp"] == ([2, 3], 5.0)              # tp is the fastest axis
    assert got[0]["data"] == ([0, 2], 2.0) and got[1]["data"] == ([1, 3], 4.0)
    assert all(g["cp_group"] is None and g["sizes"] == {"data": 2, "tp": 2, "cp": 1, "ep": 1} for g in got)
