"""Grouped expert GEMMs and a Trinity MoE training step on the GPU."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_grouped_expert_ffn_matches_per_expert_loop():
    from research_b200.ops import functional as Fn
    from research_b200.ops import native
    from research_b200.ops.grouped import grouped_expert_ffn

    torch.manual_seed(0)
    E, H, I = 6, 256, 384
    counts = torch.tensor([130, 0, 517, 64, 1, 300], device="cuda")
    R = int(counts.sum())
    rows = (torch.randn(R, H, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    w1 = torch.nn.Parameter((torch.randn(E, 2 * I, H, device="cuda") * 0.05))
    w2 = torch.nn.Parameter((torch.randn(E, H, I, device="cuda") * 0.05))
    w1.main_grad = torch.zeros_like(w1)
    w2.main_grad = torch.zeros_like(w2)
    y = grouped_expert_ffn(rows, counts, w1, w2)
    g = (torch.randn_like(y.float()) * 0.1).bfloat16()
    y.backward(g)
    native.check_status()

    rows_ref = rows.detach().float().requires_grad_(True)
    w1r = w1.detach().bfloat16().float().requires_grad_(True)
    w2r = w2.detach().bfloat16().float().requires_grad_(True)
    outs, off = [], 0
    for e in range(E):
        n = int(counts[e])
        seg = rows_ref[off:off + n]
        off += n
        gu = seg @ w1r[e].t()
        h = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
        outs.append(h.bfloat16().float() @ w2r[e].t() if False else h @ w2r[e].t())
    y_ref = torch.cat(outs, dim=0)
    y_ref.backward(g.float())
    assert torch.allclose(y.float(), y_ref, atol=3e-2, rtol=3e-2), (y.float() - y_ref).abs().max().item()
    assert torch.allclose(rows.grad.float(), rows_ref.grad, atol=2e-2, rtol=5e-2)
    for mg, rg in ((w1.main_grad, w1r.grad), (w2.main_grad, w2r.grad)):
        assert (mg - rg).abs().max().item() <= 0.03 * rg.abs().max().item() + 1e-3
    assert Fn.use_native(rows)


def test_trinity_moe_training_step_reduces_loss():
    import numpy as np

    from research_b200.config import run_spec_from_mapping
    from research_b200.contracts import Batch
    from research_b200.ops import native
    from research_b200.runtime.trainer import Trainer

    raw = {
        "run": {"id": "moe-gpu"},
        "model": {"name": "trinity", "variant": "t", "vocab_size": 1024, "hidden_size": 256, "intermediate_size": 512,
                  "num_layers": 3, "num_heads": 4, "n_kv_heads": 2, "max_seq_len": 256,
                  "trinity": {"initial_dense_layers": 1, "local_window": 128, "local_layers_per_global": 2,
                              "norm_policy": "afmoe_dual",
                              "moe": {"num_experts": 8, "top_k": 2, "expert_intermediate_size": 256,
                                      "num_shared_experts": 1, "balance": {"name": "smebu"}}}},
        "optimizer": {"name": "muon", "grad_clip_norm": 1.0, "schedule": {"peak_lr": 2e-3}},
        "data": {"train_manifest": "unused.json"},
        "training": {"seq_len": 256, "global_batch_size": 4, "target_tokens": 4 * 256 * 16, "precision": "bf16"},
    }
    trainer = Trainer(run_spec_from_mapping(raw), build_data=False)
    rng = np.random.default_rng(0)
    ids = rng.integers(0, 1024, size=(4, 257)).astype(np.int32)
    batch = Batch(input_ids=ids[:, :-1], target_ids=ids[:, 1:], loss_mask=np.ones((4, 256), dtype=bool))
    losses = [float(trainer.train_on([batch]).loss) for _ in range(6)]
    native.check_status()
    assert all(np.isfinite(losses)), losses
    assert losses[-1] < losses[0] - 0.05, losses


@pytest.mark.parametrize("capacity", [None, 300])
def test_native_routing_plan_matches_sort_based_dispatch(capacity):
    from research_b200.models.moe import apply_capacity
    from research_b200.ops import native
    from research_b200.ops.grouped import RoutingPlan, routed_expert_ffn

    torch.manual_seed(0)
    T, k, E, H, I = 3000, 4, 16, 256, 128
    logits = torch.randn(T, E, device="cuda")
    logits[:, 3] += 2.0                                   # a hot expert, so that the capacity drops something
    w_full, ids = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    x = (torch.randn(T, H, device="cuda") * 0.5).bfloat16()
    w1 = torch.nn.Parameter(torch.randn(E, 2 * I, H, device="cuda") * 0.05)
    w2 = torch.nn.Parameter(torch.randn(E, H, I, device="cuda") * 0.05)

    plan = RoutingPlan(ids, E, capacity)
    # ranks and counts against the one-hot formulation
    onehot = torch.nn.functional.one_hot(ids.reshape(-1), E)
    pos_ref = (onehot.cumsum(0) * onehot).sum(-1) - 1
    assert torch.equal(plan.pos.long(), pos_ref)
    assert torch.equal(plan.counts.long(), onehot.sum(0))
    keep = plan.kept_mask
    if capacity is None:
        assert bool(keep.all())
    else:
        assert torch.equal(keep.reshape(-1), pos_ref < capacity)
        assert int((~keep).sum()) > 0
    # every kept assignment owns a distinct row inside its expert's block
    d = plan.dest[plan.dest >= 0].long()
    assert d.unique().numel() == d.numel()
    e_of = ids.reshape(-1)[plan.dest >= 0].long()
    assert bool(((d >= plan.k_range[e_of, 0]) & (d < plan.k_range[e_of, 1])).all())

    def run(native_path):
        xr = x.clone().requires_grad_(True)
        wr = (w_full * keep.to(w_full.dtype)).detach().clone().requires_grad_(True)
        w1.main_grad = torch.zeros_like(w1)
        w2.main_grad = torch.zeros_like(w2)
        if native_path:
            y = routed_expert_ffn(xr, wr, plan, w1, w2)
        else:
            from research_b200.models.moe import Experts
            from research_b200.parallel.expert import _local_dispatch

            experts = Experts(H, I, E)
            experts.w_gate_up, experts.w_down = w1, w2
            y = _local_dispatch(experts, xr, ids, wr, E)
        g = torch.sin(torch.arange(y.numel(), device="cuda").view_as(y) * 0.01).bfloat16() * 0.1
        y.backward(g)
        native.check_status()
        # a dropped assignment has no row on the native path, so its weight gets no gradient there; in the model
        # the capacity mask multiplies the weights, which zeroes that gradient on either path
        return (y.float(), xr.grad.float(), wr.grad.float() * keep.float(), w1.main_grad.clone(),
                w2.main_grad.clone())

    a, b = run(True), run(False)
    names = ("y", "dx", "dw_route", "dW1", "dW2")
    for name, u, v in zip(names, a, b):
        tol = 0.03 * v.abs().max().item() + 1e-3
        assert (u - v).abs().max().item() <= tol, (name, (u - v).abs().max().item(), tol)
