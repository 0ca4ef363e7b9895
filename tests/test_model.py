"""Model semantics against straightforward restatements, KV-cache consistency, MoE routing."""

from pathlib import Path

import pytest
import torch

from research_b200.config import run_spec_from_mapping
from research_b200.infer.generation import generate_tokens, sample_next_token
from research_b200.models.build import build_model
from research_b200.models.moe import apply_capacity, sequence_balance_loss, switch_balance_loss
from research_b200.ops import functional as Fn
from tests.helpers import tiny_raw_config


def _model(kind="decoder", **extra):
    spec = run_spec_from_mapping(tiny_raw_config(Path("m.json"), kind=kind, extra_model=extra or None))
    return build_model(spec.model, seed=0), spec


def test_parameter_table_uses_reference_paths_and_shapes():
    res, spec = _model()
    names = {m.name: m for m in res.metadata}
    assert names["layers.0.attn.q.kernel"].shape == (64, 64) and names["layers.0.attn.k.kernel"].shape == (64, 32)
    assert names["layers.0.mlp.gate.kernel"].shape == (64, 128) and names["layers.0.mlp.down.kernel"].shape == (128, 64)
    assert names["lm_head.kernel"].tag == "lm_head" and names["embed.embedding"].shape == (256, 64)
    assert names["layers.1.pre_norm.scale"].tag == "block_pre_norm"
    q = res.logical_view(names["layers.0.attn.q.kernel"])
    assert q.shape == (64, 64) and torch.equal(q, res.model.layers[0].attn.wqkv.data[:64].t())
    assert res.parameter_count() == sum(p.numel() for p in res.model.parameters())
    tied, _ = _model(tied_embeddings=True)
    assert "lm_head.kernel" not in {m.name for m in tied.metadata}


def test_rope_is_interleaved_and_norm_preserving():
    x = torch.randn(1, 5, 2, 8)
    pos = torch.arange(5)[None]
    y = Fn.rope_reference(x, pos, 10000.0)
    assert torch.allclose(y[:, 0], x[:, 0], atol=1e-6)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    ang = 3 * 10000.0 ** (-2 / 8)
    a, b = x[0, 3, 0, 2], x[0, 3, 0, 3]
    assert torch.allclose(y[0, 3, 0, 2], a * torch.cos(torch.tensor(ang)) - b * torch.sin(torch.tensor(ang)), atol=1e-5)


def test_attention_masks_causal_documents_and_window():
    torch.manual_seed(0)
    q, k, v = torch.randn(1, 6, 2, 4), torch.randn(1, 6, 1, 4), torch.randn(1, 6, 1, 4)
    out = Fn.attention_reference(q, k, v, causal=True, lo=None, scale=0.5)
    v2 = v.clone()
    v2[:, 4:] += 100.0
    out2 = Fn.attention_reference(q, k, v2, causal=True, lo=None, scale=0.5)
    assert torch.allclose(out[:, :4], out2[:, :4]) and not torch.allclose(out[:, 4:], out2[:, 4:])
    lo = torch.tensor([[0, 0, 0, 3, 3, 3]], dtype=torch.int32)
    v3 = v.clone()
    v3[:, :3] += 100.0
    a = Fn.attention_reference(q, k, v, causal=True, lo=lo, scale=0.5)
    b = Fn.attention_reference(q, k, v3, causal=True, lo=lo, scale=0.5)
    assert torch.allclose(a[:, 3:], b[:, 3:])


@pytest.mark.parametrize("kind", ["decoder", "trinity"])
def test_kv_cache_decode_matches_full_forward(kind):
    res, spec = _model(kind)
    model = res.model.eval()
    ids = torch.randint(0, 256, (2, 12))
    with torch.no_grad():
        full = model(ids.to(torch.int32)).logits
        from research_b200.infer.generation import init_kv_cache

        cache = init_kv_cache(model, 2, 16, page_size=4)
        pos = torch.arange(8, dtype=torch.int32).expand(2, 8).contiguous()
        pre = model.run_with_cache(ids[:, :8].to(torch.int32), pos, cache)
        assert torch.allclose(pre, full[:, :8], atol=2e-4, rtol=1e-4)
        for t in range(8, 12):
            step = model.run_with_cache(ids[:, t:t + 1].to(torch.int32), torch.full((2, 1), t, dtype=torch.int32), cache)
            assert torch.allclose(step[:, 0], full[:, t], atol=2e-4, rtol=1e-4), t


def test_sampler_and_generation():
    logits = torch.tensor([[0.0, 2.0, 1.0, -1.0]])
    tok, lp = sample_next_token(logits, temperature=1.0, top_k=1, top_p=None, generator=None)
    assert tok.item() == 1 and lp.item() == pytest.approx(0.0)
    g = torch.Generator().manual_seed(0)
    draws = {sample_next_token(logits, temperature=1.0, top_k=2, top_p=None, generator=g)[0].item() for _ in range(50)}
    assert draws <= {1, 2}
    from research_b200.errors import ContractError

    with pytest.raises(ContractError, match="top_p"):
        sample_next_token(logits, temperature=1.0, top_k=None, top_p=0.9, generator=None)
    res, _ = _model()
    out = generate_tokens(res.model, torch.tensor([[1, 2, 3]]), max_new_tokens=5, top_k=1)
    again = generate_tokens(res.model, torch.tensor([[1, 2, 3]]), max_new_tokens=5, top_k=1)
    assert out.generated_ids == again.generated_ids and len(out.full_ids[0]) == 8 and len(out.logprobs[0]) == 5
    with pytest.raises(ContractError, match="exceeds model.max_seq_len"):
        generate_tokens(res.model, torch.tensor([[1] * 60]), max_new_tokens=10)


def test_router_weights_bias_and_capacity():
    res, _ = _model("trinity")
    moe = res.model.layers[1].mlp
    x = torch.randn(2, 8, 64)
    ids, w, scores = moe.router(x, moe.expert_bias)
    assert ids.shape == (2, 8, 2) and torch.allclose(w.sum(-1), torch.ones(2, 8), atol=1e-5)
    top = scores.gather(-1, ids)
    assert torch.allclose(w, top / top.sum(-1, keepdim=True), atol=1e-6)
    bias = torch.zeros(4)
    bias[3] = 10.0
    ids_b, w_b, _ = moe.router(x, bias)
    assert (ids_b == 3).any(dim=-1).all()                       # the bias steers selection...
    assert torch.allclose(w_b.sum(-1), torch.ones(2, 8), atol=1e-5)  # ...but weights come from unbiased scores
    e = torch.zeros(6, 1, dtype=torch.long)
    kept, dropped = apply_capacity(e, torch.ones(6, 1), num_experts=2, capacity_factor=1.0)
    assert kept[:3].sum() == 3 and kept[3:].sum() == 0 and dropped.item() == 3
    uniform = torch.full((1, 4, 4), 0.25)
    sel = torch.tensor([[[0, 1], [2, 3], [0, 1], [2, 3]]])
    assert sequence_balance_loss(sel, uniform, 2).item() == pytest.approx(1.0)
    assert switch_balance_loss(sel, uniform, 2).item() == pytest.approx(1.0)
    # every pick on one expert whose probability is 1: E times the balanced value
    one_hot = torch.zeros(1, 4, 4)
    one_hot[..., 0] = 1.0
    assert switch_balance_loss(torch.zeros(1, 4, 1, dtype=torch.long), one_hot, 1).item() == pytest.approx(4.0)


def test_moe_layer_matches_dense_loop():
    res, _ = _model("trinity")
    moe = res.model.layers[1].mlp
    x = torch.randn(1, 6, 64)
    y, aux, stats = moe(x, res.execution, name="l", layer_index=1)
    ids, w, _ = moe.router(x, moe.expert_bias)
    want = torch.zeros_like(x)
    for t in range(6):
        for j in range(2):
            e = ids[0, t, j].item()
            h = Fn.swiglu(torch.nn.functional.linear(x[0, t], moe.experts.w_gate_up[e]))
            want[0, t] += w[0, t, j] * torch.nn.functional.linear(h, moe.experts.w_down[e])
    want = want + moe.shared_experts(x, res.execution)
    assert torch.allclose(y, want, atol=1e-5)
    assert stats[0].expert_counts.sum().item() == 12 and aux[0].name == "moe_sequence_balance"
