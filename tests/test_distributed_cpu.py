"""Parity of distributed layouts against one process, on CPU ranks over gloo (the reference checks the same
thing on four fake devices: tests/jaxtitan/test_train_step.py:943-1051): same global batch, same token count,
loss sums within 1e-4 and the whole updated parameter tree close after a few optimizer steps."""

import math

import pytest
import torch

from tests.helpers import run_gloo, tiny_dataset, tiny_raw_config, train_and_collect

STEPS = 3


def _single(raw):
    from research_b200.parallel import mesh  # noqa: F401

    return train_and_collect(0, 1, raw, STEPS)


def _compare(ref, got, tol=2e-4):
    assert ref["token_count"] == got["token_count"]
    for a, b in zip(ref["loss_sum"], got["loss_sum"]):
        assert abs(a - b) <= 1e-3 * max(1.0, abs(a)), (ref["loss_sum"], got["loss_sum"])
    for name, want in ref["model"].items():
        have = got["model"][name]
        assert have.shape == want.shape, name
        err = (have - want).abs().max().item()
        assert err <= tol * (1.0 + want.abs().max().item()), (name, err)


CASES = [
    ("fsdp2_sharded_params", "decoder", "adamw", {"fsdp": 2}, {"mode": "fsdp", "fsdp_resident": False}),
    ("fsdp2_sharded_params_muon", "decoder", "muon", {"fsdp": 2}, {"mode": "fsdp", "fsdp_resident": False}),
    ("ddp2", "decoder", "adamw", {"data": 2}, {"mode": "ddp"}),
    ("zero2", "decoder", "adamw", {"fsdp": 2}, {"mode": "zero2"}),
    ("fsdp2_muon", "decoder", "muon", {"fsdp": 2}, {"mode": "fsdp"}),
    ("tp2", "decoder", "adamw", {"tp": 2}, {"mode": "ddp", "tensor_parallel": True}),
    # compositions on four ranks
    ("hsdp_data2_fsdp2", "decoder", "adamw", {"data": 2, "fsdp": 2}, {"mode": "fsdp"}),
    ("hsdp_data2_fsdp2_muon", "decoder", "muon", {"data": 2, "fsdp": 2}, {"mode": "fsdp"}),
    ("fsdp2_tp2", "decoder", "adamw", {"fsdp": 2, "tp": 2}, {"mode": "fsdp", "tensor_parallel": True}),
    ("cp2_tp2", "decoder", "adamw", {"cp": 2, "tp": 2},
     {"mode": "ddp", "context_parallel": True, "tensor_parallel": True}),
    ("tp2_ep2_moe", "trinity", "adamw", {"tp": 2, "ep": 2},
     {"mode": "ddp", "tensor_parallel": True, "expert_parallel": True}),
    ("fsdp2_sharded_params_tp2", "decoder", "adamw", {"fsdp": 2, "tp": 2},
     {"mode": "fsdp", "tensor_parallel": True, "fsdp_resident": False}),
    ("tp2_vocab_parallel_head", "decoder", "adamw", {"tp": 2},
     {"mode": "ddp", "tensor_parallel": True, "vocab_parallel_head": True}),
    ("tp2_muon_duplicated", "decoder", "muon", {"tp": 2}, {"mode": "ddp", "tensor_parallel": True}),
    ("cp2", "decoder", "adamw", {"cp": 2}, {"mode": "ddp", "context_parallel": True}),
    ("cp2_ulysses", "decoder", "adamw", {"cp": 2},
     {"mode": "ddp", "context_parallel": True, "context_attention": "ulysses"}),
    ("ep2_moe", "trinity", "adamw", {"ep": 2}, {"mode": "ddp", "expert_parallel": True}),
    ("fsdp2_folded_ep_moe", "trinity", "adamw", {"fsdp": 2}, {"mode": "fsdp", "expert_parallel": True}),
    # expert FSDP: routed experts split over ep (expert index) and expert_fsdp (intermediate dimension)
    ("ep2_expert_fsdp2_moe", "trinity", "adamw", {"fsdp": 1, "ep": 2, "expert_fsdp": 2},
     {"mode": "fsdp", "expert_parallel": True}),
]


@pytest.mark.parametrize("name,kind,optimizer,mesh,parallelism", CASES, ids=[c[0] for c in CASES])
def test_layout_matches_single_process(tmp_path, name, kind, optimizer, mesh, parallelism):
    manifest = tiny_dataset(tmp_path)
    base = tiny_raw_config(manifest, kind=kind, optimizer=optimizer, steps=STEPS + 1)
    ref = _single(base)
    raw = tiny_raw_config(manifest, kind=kind, optimizer=optimizer, mesh=mesh, parallelism=parallelism,
                          steps=STEPS + 1)
    world = 1
    for size in mesh.values():
        world *= size
    results = run_gloo(world, train_and_collect, raw, STEPS)
    tol = 2e-3 if optimizer == "muon" else 2e-4
    for got in results:
        _compare(ref, got, tol)
    # every rank ends with the same logical parameters, all of them finite
    for name_, t in results[0]["model"].items():
        assert torch.isfinite(t).all(), name_
        for other in results[1:]:
            assert torch.equal(t, other["model"][name_]), name_


def _idle_rank_worker(rank, world, routing):
    """One MoE layer, experts over all ranks, routing forced; returns the output and the input gradient."""

    import torch

    from research_b200.config.specs import MeshSpec, ModelSpec, MoeBalanceSpec, ParallelismSpec, TrinityMoeSpec, TrinitySpec
    from research_b200.models.moe import SparseMoE
    from research_b200.parallel.mesh import build_mesh_context, execution_context_for
    from research_b200.runtime.profile_bench import FixedRouter, routing_ids

    device = torch.device("cpu")
    axes = {"data": 1} if world == 1 else {"data": 1, "ep": world}
    mesh = build_mesh_context(MeshSpec(axis_names=tuple(axes), axis_sizes=tuple(axes.values())), device=device)
    ex = execution_context_for(mesh, ParallelismSpec(mode="ddp", expert_parallel=world > 1))
    experts, top_k, tokens, hidden, inter = 4, 2, 16, 32, 48
    moe = TrinityMoeSpec(num_experts=experts, top_k=top_k, expert_intermediate_size=inter, capacity_factor=None,
                         balance=MoeBalanceSpec())
    spec = ModelSpec(name="trinity", variant="t", vocab_size=64, hidden_size=hidden, intermediate_size=inter,
                     num_layers=2, num_heads=2, max_seq_len=tokens,
                     trinity=TrinitySpec(initial_dense_layers=1, local_window=8, local_layers_per_global=1, moe=moe))
    layer = SparseMoE(spec, moe, ex)
    local = experts // world
    gen = torch.Generator().manual_seed(7)
    w_gate_up = torch.randn(experts, 2 * inter, hidden, generator=gen) * 0.1
    w_down = torch.randn(experts, hidden, inter, generator=gen) * 0.1
    with torch.no_grad():
        layer.experts.w_gate_up.copy_(w_gate_up[rank * local:(rank + 1) * local])
        layer.experts.w_down.copy_(w_down[rank * local:(rank + 1) * local])
    layer.router = FixedRouter(routing_ids(routing, tokens, top_k, experts, device), experts)
    x = torch.randn(1, tokens, hidden, generator=gen).requires_grad_(True)
    y, _, _ = layer(x, ex, name="l", layer_index=0)
    (y.square().sum()).backward()
    grads = layer.experts.w_gate_up.grad
    return {"y": y.detach(), "dx": x.grad.clone(), "dw_norm": None if grads is None else float(grads.norm())}


@pytest.mark.parametrize("routing", ["skewed", "balanced"])
def test_expert_parallel_backward_completes_when_a_rank_receives_no_token(routing):
    """With every token routed to the experts of rank 0, rank 1 computes nothing, yet it must run the same exchanges
    in its backward pass as rank 0 does: the run finishes and matches the single-process layer."""

    (ref,) = run_gloo(1, _idle_rank_worker, routing)
    got = run_gloo(2, _idle_rank_worker, routing)
    for r in got:
        assert torch.allclose(r["y"], ref["y"], atol=1e-5) and torch.allclose(r["dx"], ref["dx"], atol=1e-5)
    if routing == "skewed":
        assert got[0]["dw_norm"] > 0 and not got[1]["dw_norm"]          # the idle rank's experts get no gradient


def _bf16_balance_worker(rank, world, raw):
    import torch

    from research_b200.config import run_spec_from_mapping
    from research_b200.runtime.trainer import Trainer

    trainer = Trainer(run_spec_from_mapping(raw), device="cpu")
    losses = [trainer.train_step(diagnostics=True).loss for _ in range(3)]
    mlp = trainer.result.model.layers[1].mlp
    return {"losses": losses, "master": mlp.bias_master.clone(), "copy": mlp.expert_bias.data.clone(),
            "momentum": trainer.moe_balance.layers[0].momentum.clone()}


@pytest.mark.parametrize("mesh, parallelism", [
    ({"ep": 2}, {"mode": "ddp", "expert_parallel": True}),
    ({"fsdp": 2}, {"mode": "fsdp", "expert_parallel": True}),
    ({"fsdp": 2}, {"mode": "fsdp", "fsdp_resident": False}),
], ids=["ep2", "fsdp2_folded_ep", "fsdp2_sharded_at_rest"])
def test_balance_bias_stays_fp32_and_identical_on_every_rank_with_bf16_compute(tmp_path, mesh, parallelism):
    manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, kind="trinity", mesh=mesh, parallelism=parallelism, steps=4)
    raw["model"]["compute_dtype"] = "bfloat16"
    raw["training"]["precision"] = "bf16"
    a, b = run_gloo(2, _bf16_balance_worker, raw)
    for r in (a, b):
        assert r["master"].dtype == torch.float32 and r["copy"].dtype == torch.bfloat16
        assert torch.equal(r["copy"], r["master"].to(torch.bfloat16)) and float(r["master"].abs().max()) > 0
        assert all(math.isfinite(x) for x in r["losses"])
    assert torch.equal(a["master"], b["master"]) and torch.equal(a["momentum"], b["momentum"])


def _seeds_that_order_two_strings_both_ways(a, b):
    """A hash seed under which a set iterates ``a`` before ``b`` and one under which it iterates ``b`` first."""

    import subprocess
    import sys

    found = {}
    for seed in range(64):
        out = subprocess.run([sys.executable, "-c", f"print(list({{{a!r}, {b!r}}})[0])"], capture_output=True, text=True,
                             env={"PYTHONHASHSEED": str(seed), "PATH": ""})
        found.setdefault(out.stdout.strip(), seed)
        if len(found) == 2:
            return found[a], found[b]
    raise AssertionError("no pair of seeds found")


@pytest.mark.parametrize("kind, axes, parallelism", [
    ("decoder", ("fsdp", "tp"), {"mode": "fsdp", "tensor_parallel": True}),
    ("trinity", ("tp", "ep"), {"mode": "ddp", "tensor_parallel": True, "expert_parallel": True}),
], ids=["fsdp2_tp2", "tp2_ep2_moe"])
def test_collectives_over_two_axes_do_not_depend_on_the_string_hash_seed(tmp_path, kind, axes, parallelism):
    """Ranks must reduce over the mesh axes in one order.  With the ranks' hash seeds chosen so that a set of the two
    axis names iterates one name first on ranks 0 and 3 and the other first on ranks 1 and 2, code that walks such a
    set makes every rank wait for a peer that waits for someone else: this run would end in the collective timeout.
    The result must also be the single-process one whatever the seeds are."""

    first, second = _seeds_that_order_two_strings_both_ways(*axes)
    manifest = tiny_dataset(tmp_path)
    ref = _single(tiny_raw_config(manifest, kind=kind, steps=STEPS + 1))
    raw = tiny_raw_config(manifest, kind=kind, mesh={axes[0]: 2, axes[1]: 2}, parallelism=parallelism, steps=STEPS + 1)
    results = run_gloo(4, train_and_collect, raw, STEPS, hash_seeds=[first, second, second, first])
    for got in results:
        _compare(ref, got, 2e-4)


def test_no_loop_over_a_set_in_modules_that_issue_collectives():
    """The order of a loop that contains a collective must not come from a set (its order is per process)."""

    import re
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent / "research_b200"
    loop_over_set = re.compile(r"for\s+[\w,\s()]+\s+in\s+(\{|set\(|frozenset\()")
    offenders = []
    for path in root.rglob("*.py"):
        text = path.read_text()
        if "torch.distributed" not in text and "import dist" not in text:
            continue
        for n, line in enumerate(text.splitlines(), 1):
            if loop_over_set.search(line):
                offenders.append(f"{path.relative_to(root)}:{n}")
    assert offenders == []


def _divergent_layout_worker(rank, world, raw):
    from research_b200.config import run_spec_from_mapping
    from research_b200.errors import ContractError
    from research_b200.parallel.sharding import ParamStore
    from research_b200.runtime.trainer import Trainer

    ok = Trainer(run_spec_from_mapping(raw), device="cpu")
    agreed = ok.layout_fingerprint()
    if rank == 1:
        original = ParamStore.describe
        ParamStore.describe = lambda self: {**original(self), "arena_elements": original(self)["arena_elements"] + 1}
    try:
        Trainer(run_spec_from_mapping(raw), device="cpu")
    except ContractError as exc:
        return {"agreed": agreed, "error": str(exc)}
    return {"agreed": agreed, "error": None}


def test_ranks_that_lay_the_run_out_differently_fail_at_start_up_instead_of_waiting(tmp_path):
    manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, mesh={"fsdp": 2}, parallelism={"mode": "fsdp"})
    a, b = run_gloo(2, _divergent_layout_worker, raw)
    assert a["agreed"] == b["agreed"] and 0 < a["agreed"] < 2 ** 62
    for r in (a, b):
        assert r["error"] is not None and "laid the run out differently" in r["error"]
        assert "would deadlock" in r["error"]


def _generate_worker(rank, world, raw):
    import torch

    from research_b200.config import run_spec_from_mapping
    from research_b200.infer.generation import generate_tokens
    from research_b200.runtime.trainer import Trainer

    trainer = Trainer(run_spec_from_mapping(raw), device="cpu", build_data=False)
    prompts = torch.tensor([[3, 1, 4, 1, 5], [9, 2, 6, 5, 3]])
    out = generate_tokens(trainer.result.model, prompts, max_new_tokens=5, top_k=1, page_size=4)
    return {"ids": out.generated_ids, "logprobs": out.logprobs}


@pytest.mark.parametrize("kind, mesh, parallelism", [
    ("decoder", {"tp": 2}, {"mode": "ddp", "tensor_parallel": True}),
    ("trinity", {"tp": 2}, {"mode": "ddp", "tensor_parallel": True}),
    ("decoder", {"tp": 2}, {"mode": "ddp", "tensor_parallel": True, "vocab_parallel_head": True}),
    ("trinity", {"ep": 2}, {"mode": "ddp", "expert_parallel": True}),
    ("decoder", {"cp": 2}, {"mode": "ddp", "context_parallel": True}),
], ids=["tp2", "tp2_moe", "tp2_vocab_parallel_head", "ep2_moe", "cp2"])
def test_generation_on_a_split_model_matches_one_process(tmp_path, kind, mesh, parallelism):
    """Decoding runs a row at a time: no sequence to split, so tensor-parallel ranks hold whole activations and sum
    their row-parallel products.  Every rank must produce the tokens one process produces."""

    manifest = tiny_dataset(tmp_path)
    (ref,) = run_gloo(1, _generate_worker, tiny_raw_config(manifest, kind=kind))
    got = run_gloo(2, _generate_worker, tiny_raw_config(manifest, kind=kind, mesh=mesh, parallelism=parallelism))
    for r in got:
        assert r["ids"] == ref["ids"]
        assert torch.allclose(torch.tensor(r["logprobs"]), torch.tensor(ref["logprobs"]), atol=1e-4)


def _first_step_gradients(rank, world, raw):
    """The reduced gradient of every parameter as the optimizer first sees it."""

    from research_b200.config import run_spec_from_mapping
    from research_b200.optim.optimizer import Optimizer
    from research_b200.runtime.trainer import Trainer

    trainer = Trainer(run_spec_from_mapping(raw), device="cpu")
    seen = {}
    step = Optimizer.step

    def spy(self, *args, **kwargs):
        if not seen:
            seen.update({e.name: e.param.main_grad.clone() for e in self.store.entries if e.param.main_grad is not None})
        return step(self, *args, **kwargs)

    Optimizer.step = spy
    try:
        trainer.train_on(trainer.next_accumulated_batch())
    finally:
        Optimizer.step = step
    return seen


def _trinity_with_loud_balance_losses(manifest, **layout):
    raw = tiny_raw_config(manifest, kind="trinity", steps=2, **layout)
    moe = raw["model"]["trinity"]["moe"]
    # weights a thousand times the usual ones: an error in these terms' gradients shows in the router's
    moe["balance"]["sequence_aux_loss_weight"] = 0.1
    moe["aux_loss_coef"] = 0.1
    return raw


@pytest.mark.parametrize("mesh, parallelism", [
    ({"cp": 2}, {"mode": "ddp", "context_parallel": True, "context_attention": "gather"}),
    ({"cp": 2}, {"mode": "ddp", "context_parallel": True, "context_attention": "ulysses"}),
    ({"tp": 2}, {"mode": "ddp", "tensor_parallel": True}),
], ids=["cp2_gather", "cp2_ulysses", "tp2_sequence_parallel"])
def test_trinity_gradients_on_a_split_sequence_match_one_process(tmp_path, mesh, parallelism):
    """Sliding-window and global layers, gated attention, the scaled embedding and both balance losses (statistics of
    whole sequences) over a split sequence.  Compared on the gradients: after AdamW an element whose gradient is a
    rounding error away from zero moves by a visible fraction of the learning rate in either direction, which says
    nothing about the layout.  Tensors a layout splits are left to the parameter comparison above."""

    manifest = tiny_dataset(tmp_path)
    (ref,) = run_gloo(1, _first_step_gradients, _trinity_with_loud_balance_losses(manifest))
    got = run_gloo(2, _first_step_gradients,
                   _trinity_with_loud_balance_losses(manifest, mesh=mesh, parallelism=parallelism))
    assert ref and set(ref) == set(got[0])
    compared = 0
    for name, want in ref.items():
        for r in got:
            if r[name].shape != want.shape:
                continue
            compared += 1
            err = (r[name] - want).abs().max().item()
            assert err <= 1e-4 * max(want.abs().max().item(), 1e-3), (name, err)
    assert compared >= len(got) * 6 and any("router" in name for name in ref)


@pytest.mark.parametrize("kind, mesh, parallelism", [
    ("decoder", {"tp": 2}, {"mode": "ddp", "tensor_parallel": True}),
    ("trinity", {"tp": 2}, {"mode": "ddp", "tensor_parallel": True}),
    ("trinity", {"fsdp": 1, "ep": 2, "expert_fsdp": 2}, {"mode": "fsdp", "expert_parallel": True}),
], ids=["tp2", "tp2_moe", "ep2_expert_fsdp2"])
def test_dion2_on_a_shard_selects_over_the_logical_matrix(tmp_path, kind, mesh, parallelism):
    """Dion2 keeps the quarter of a matrix's rows or columns with the largest norms.  On a tensor-parallel shard, and
    on a routed expert whose intermediate dimension is split over ``expert_fsdp``, that choice is made over the whole
    logical matrix: one step moves every parameter where one process moves it (a choice made shard by shard is off by
    a third of the learning rate in a tenth of the elements)."""

    manifest = tiny_dataset(tmp_path)
    (ref,) = run_gloo(1, train_and_collect, tiny_raw_config(manifest, kind=kind, optimizer="dion", steps=2), 1)
    raw = tiny_raw_config(manifest, kind=kind, optimizer="dion", steps=2, mesh=mesh, parallelism=parallelism)
    for got in run_gloo(math.prod(mesh.values()), train_and_collect, raw, 1):
        _compare(ref, got, 2e-4)
