"""Run-twice checks: kernels that claim a fixed reduction order must reproduce their output bit for bit."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bf(shape, scale=1.0):
    return (torch.randn(shape, device="cuda") * scale).to(torch.bfloat16)


def test_attention_forward_and_backward_are_bitwise_reproducible():
    from research_b200.ops import native

    torch.manual_seed(0)
    B, S, H, Hkv, D = 2, 1024, 8, 4, 128
    q, k, v, d_o = _bf((B, S, H, D)), _bf((B, S, Hkv, D)), _bf((B, S, Hkv, D)), _bf((B, S, H, D))
    runs = []
    for _ in range(2):
        o, lse = native.attn_fwd(q, k, v, causal=True)
        dq, dk, dv = native.attn_bwd(q, k, v, o, d_o, lse, causal=True)
        runs.append((o.clone(), lse.clone(), dq.clone(), dk.clone(), dv.clone()))
    native.check_status()
    for a, b in zip(*runs):
        assert torch.equal(a, b)          # the backward accumulates dQ, dK and dV without atomics


def test_gemm_and_router_are_bitwise_reproducible():
    from research_b200.ops import native
    from research_b200.ops.router import route

    torch.manual_seed(1)
    a, b = _bf((2048, 1024)), _bf((512, 1024))
    assert torch.equal(native.gemm(a, b), native.gemm(a, b))
    logits = _bf((4096, 64), 1.5)
    bias = torch.zeros(64, device="cuda")
    first, second = route(logits, bias, 8, "sigmoid", 1.0), route(logits, bias, 8, "sigmoid", 1.0)
    native.check_status()
    for x, y in zip(first, second):
        assert torch.equal(x, y)


def test_routing_plan_and_dispatch_are_bitwise_reproducible():
    from research_b200.ops import native
    from research_b200.ops.grouped import RoutingPlan, _combine_rows, _gather_rows

    torch.manual_seed(2)
    T, k, E, H = 4096, 4, 16, 256
    ids = torch.topk(torch.randn(T, E, device="cuda"), k, dim=-1).indices.to(torch.int32)
    x = _bf((T, H))
    w = torch.rand(T * k, device="cuda")
    outs = []
    for _ in range(2):
        plan = RoutingPlan(ids, E, int(1.25 * T * k / E))
        pad = _gather_rows(x, None, plan)
        outs.append((plan.dest.clone(), pad.clone(), _combine_rows(pad, w, plan).clone()))
    native.check_status()
    for a, b in zip(*outs):
        assert torch.equal(a, b)          # ranks follow token order, so capacity drops the same assignments


@pytest.mark.parametrize("family,optimizer", [("decoder", "muon"), ("decoder", "adamw"), ("trinity", "dion")])
def test_whole_training_steps_repeat_bit_for_bit_in_deterministic_mode(family, optimizer):
    """With the debugging switch on, every arrival-ordered sum (split-K weight gradients, the atomics behind the norm
    scale and embedding gradients, Muon's norm, router importance) takes a fixed-order form: two runs from the same
    seed end with identical master weights and identical losses."""

    import numpy as np

    from research_b200.config import run_spec_from_mapping
    from research_b200.contracts import Batch
    from research_b200.ops import native
    from research_b200.runtime.trainer import Trainer

    raw = {
        "run": {"id": "repeatable"},
        "model": {"name": "decoder", "variant": "t", "vocab_size": 1024, "hidden_size": 256, "intermediate_size": 512,
                  "num_layers": 2, "num_heads": 2, "n_kv_heads": 1, "max_seq_len": 256, "init": "normal_0.02",
                  "qk_norm": True},
        "optimizer": {"name": optimizer, "weight_decay": 0.1, "grad_clip_norm": 1.0, "schedule": {"peak_lr": 1e-3}},
        "data": {"train_manifest": "unused.json"},
        "training": {"seq_len": 256, "global_batch_size": 4, "target_tokens": 4 * 256 * 4, "precision": "bf16"},
    }
    if family == "trinity":
        raw["model"].pop("qk_norm")
        raw["model"].update(name="trinity", trinity={
            "initial_dense_layers": 1, "local_window": 128, "local_layers_per_global": 1, "norm_policy": "afmoe_dual",
            "moe": {"num_experts": 4, "top_k": 2, "expert_intermediate_size": 256, "num_shared_experts": 1}})
    rng = np.random.default_rng(0)
    ids = rng.integers(0, 1024, size=(4, 257)).astype(np.int32)
    batch = Batch(input_ids=ids[:, :-1], target_ids=ids[:, 1:], loss_mask=np.ones((4, 256), dtype=bool))
    native.set_deterministic(True)
    try:
        runs = []
        for _ in range(2):
            trainer = Trainer(run_spec_from_mapping(raw), build_data=False)
            losses = [float(trainer.train_on([batch]).loss) for _ in range(3)]
            native.check_status()
            runs.append((losses, {e.name: trainer.store.master_view(trainer.store.section_of(e), e).clone()
                                  for e in trainer.store.entries}))
    finally:
        native.set_deterministic(False)
    assert runs[0][0] == runs[1][0]
    for name, w in runs[0][1].items():
        assert torch.equal(w, runs[1][1][name]), name
