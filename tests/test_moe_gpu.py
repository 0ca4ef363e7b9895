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
