"""The models against a from-scratch restatement that reads only the logical parameter table.

The restatement below shares no code with the model: it takes every parameter in the reference's ``[in, out]``
layout from ``ModelBuildResult.logical_view`` and spells the forward pass out with plain tensor operations."""

import math
from pathlib import Path

import pytest
import torch
import torch.nn.functional as F

from research_b200.config import run_spec_from_mapping
from research_b200.models.build import build_model
from research_b200.models.transformer import trinity_layer_attention_kind, trinity_post_norm_scale
from tests.helpers import tiny_raw_config


def _build(kind="decoder", seed=0, **extra):
    spec = run_spec_from_mapping(tiny_raw_config(Path("m.json"), kind=kind, extra_model=extra or None))
    return build_model(spec.model, seed=seed), spec.model


def _params(res):
    return {m.name: res.logical_view(m).detach().double() for m in res.metadata}


def rms(x, scale, eps=1e-6):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * scale


def rope(x, theta):
    """Interleaved pairs (2i, 2i+1) rotated by ``pos * theta^(-2i/D)``; x: [S, heads, D]."""

    S, _, D = x.shape
    inv = theta ** (-torch.arange(0, D, 2, dtype=torch.float64) / D)
    ang = torch.arange(S, dtype=torch.float64)[:, None] * inv[None]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2], out[..., 1::2] = a * cos - b * sin, a * sin + b * cos
    return out


def attention(p, prefix, x, spec, *, use_rope, window, gate, doc_ids=None):
    S, H = x.shape
    hq, hkv, D = spec.num_heads, spec.n_kv_heads, spec.hidden_size // spec.num_heads
    q = (x @ p[f"{prefix}.q.kernel"]).view(S, hq, D)
    k = (x @ p[f"{prefix}.k.kernel"]).view(S, hkv, D)
    v = (x @ p[f"{prefix}.v.kernel"]).view(S, hkv, D)
    if f"{prefix}.q_norm.scale" in p:
        q, k = rms(q, p[f"{prefix}.q_norm.scale"]), rms(k, p[f"{prefix}.k_norm.scale"])
    if use_rope:
        q, k = rope(q, spec.rope_theta), rope(k, spec.rope_theta)
    k, v = k.repeat_interleave(hq // hkv, dim=1), v.repeat_interleave(hq // hkv, dim=1)
    scores = torch.einsum("shd,thd->hst", q, k) / math.sqrt(D)
    i, j = torch.arange(S)[:, None], torch.arange(S)[None, :]
    allowed = j <= i
    if window is not None:
        allowed &= j > i - window
    if doc_ids is not None:
        allowed &= doc_ids[:, None] == doc_ids[None, :]
    scores = scores.masked_fill(~allowed, float("-inf"))
    out = torch.einsum("hst,thd->shd", scores.softmax(-1), v).reshape(S, hq * D)
    if gate:
        out = out * torch.sigmoid(x @ p[f"{prefix}.gate.kernel"])
    return out @ p[f"{prefix}.o.kernel"]


def swiglu(x, gate, up, down):
    return (F.silu(x @ gate) * (x @ up)) @ down


def decoder_oracle(p, spec, ids, doc_ids=None):
    x = p["embed.embedding"][ids]
    for i in range(spec.num_layers):
        L = f"layers.{i}"
        x = x + attention(p, f"{L}.attn", rms(x, p[f"{L}.pre_norm.scale"]), spec, use_rope=True, window=None,
                          gate=False, doc_ids=doc_ids)
        x = x + swiglu(rms(x, p[f"{L}.post_norm.scale"]), p[f"{L}.mlp.gate.kernel"], p[f"{L}.mlp.up.kernel"],
                       p[f"{L}.mlp.down.kernel"])
    head = p["lm_head.kernel"] if "lm_head.kernel" in p else p["embed.embedding"].t()
    return rms(x, p["norm.scale"]) @ head


def moe_oracle(p, prefix, x, moe):
    scores = torch.sigmoid(x @ p[f"{prefix}.router.proj.kernel"])
    pick = (scores + p[f"{prefix}.expert_bias"]).topk(moe.top_k, dim=-1).indices
    chosen = scores.gather(-1, pick)
    weights = chosen / chosen.sum(-1, keepdim=True) * moe.route_scale
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for slot in range(moe.top_k):
            e = int(pick[t, slot])
            out[t] += weights[t, slot] * swiglu(x[t], p[f"{prefix}.experts.gate"][e], p[f"{prefix}.experts.up"][e],
                                                p[f"{prefix}.experts.down"][e])
    if f"{prefix}.shared_experts.gate.kernel" in p:
        out = out + swiglu(x, p[f"{prefix}.shared_experts.gate.kernel"], p[f"{prefix}.shared_experts.up.kernel"],
                           p[f"{prefix}.shared_experts.down.kernel"])
    return out


def trinity_oracle(p, spec, ids):
    tr = spec.trinity
    x = p["embed.embedding"][ids] * math.sqrt(spec.hidden_size)
    for i in range(spec.num_layers):
        L = f"layers.{i}"
        is_global = (i + 1) % (tr.local_layers_per_global + 1) == 0
        a = attention(p, f"{L}.attn", rms(x, p[f"{L}.attn_pre_norm.scale"]), spec, use_rope=not is_global,
                      window=None if is_global else tr.local_window, gate=tr.attention_gate)
        x = x + rms(a, p[f"{L}.attn_post_norm.scale"])
        h = rms(x, p[f"{L}.ffn_pre_norm.scale"])
        if tr.moe is not None and i >= tr.initial_dense_layers:
            m = moe_oracle(p, f"{L}.mlp", h, tr.moe)
        else:
            m = swiglu(h, p[f"{L}.mlp.gate.kernel"], p[f"{L}.mlp.up.kernel"], p[f"{L}.mlp.down.kernel"])
        x = x + rms(m, p[f"{L}.ffn_post_norm.scale"])
    return rms(x, p["norm.scale"]) @ p["lm_head.kernel"]


@pytest.mark.parametrize("extra", [{}, {"tied_embeddings": True}, {"qk_norm": False}, {"n_kv_heads": 4},
                                   {"n_kv_heads": 1}, {"rope_theta": 1000000.0}])
def test_decoder_matches_the_restatement(extra):
    res, spec = _build("decoder", **extra)
    torch.manual_seed(1)
    for m in res.metadata:                                 # norms start at one: move them so that they matter
        if m.tag.endswith("norm"):
            res.logical_view(m).data.add_(0.2 * torch.randn(m.shape))
    ids = torch.randint(0, spec.vocab_size, (2, 24))
    with torch.no_grad():
        got = res.model.eval()(ids.to(torch.int32)).logits.double()
    p = _params(res)
    for b in range(2):
        assert torch.allclose(got[b], decoder_oracle(p, spec, ids[b]), atol=2e-4, rtol=1e-4)


def test_decoder_document_mask_matches_the_restatement_and_can_be_switched_off():
    res, spec = _build("decoder")
    ids = torch.randint(0, spec.vocab_size, (1, 20))
    docs = torch.tensor([[0] * 7 + [1] * 9 + [2] * 4])
    with torch.no_grad():
        masked = res.model.eval()(ids.to(torch.int32), docs).logits.double()
        plain = res.model(ids.to(torch.int32)).logits.double()
    p = _params(res)
    assert torch.allclose(masked[0], decoder_oracle(p, spec, ids[0], docs[0]), atol=2e-4, rtol=1e-4)
    assert torch.allclose(masked[0, :7], plain[0, :7], atol=1e-5) and not torch.allclose(masked[0, 7:], plain[0, 7:], atol=1e-3)
    off, _ = _build("decoder", attention_doc_mask=False)
    with torch.no_grad():
        assert torch.equal(off.model.eval()(ids.to(torch.int32), docs).logits, off.model(ids.to(torch.int32)).logits)


@pytest.mark.parametrize("layers, per_global", [(2, 1), (4, 1), (4, 3), (3, 2)])
def test_trinity_matches_the_restatement(layers, per_global):
    raw = tiny_raw_config(Path("m.json"), kind="trinity", extra_model={"num_layers": layers})
    raw["model"]["trinity"]["local_layers_per_global"] = per_global
    raw["model"]["trinity"]["local_window"] = 5
    spec = run_spec_from_mapping(raw).model
    res = build_model(spec, seed=3)
    torch.manual_seed(2)
    for m in res.metadata:
        if m.tag == "moe_expert_bias":
            res.logical_view(m).data.copy_(0.3 * torch.randn(m.shape))      # the bias steers selection only
    ids = torch.randint(0, spec.vocab_size, (1, 18))
    with torch.no_grad():
        got = res.model.eval()(ids.to(torch.int32)).logits.double()
    assert torch.allclose(got[0], trinity_oracle(_params(res), spec, ids[0]), atol=5e-4, rtol=1e-3)


def test_trinity_layer_pattern_and_norm_scales():
    kinds = [trinity_layer_attention_kind(i, 3) for i in range(8)]
    assert kinds == ["local", "local", "local", "global"] * 2
    assert [trinity_layer_attention_kind(i, 0) for i in range(3)] == ["global"] * 3
    res, spec = _build("trinity", num_layers=4)
    assert trinity_post_norm_scale(spec) == pytest.approx(0.5)
    by = {m.name: res.logical_view(m) for m in res.metadata}
    assert torch.allclose(by["layers.2.attn_post_norm.scale"], torch.full((64,), 0.5))
    assert torch.allclose(by["layers.2.ffn_post_norm.scale"], torch.full((64,), 0.5))
    assert torch.allclose(by["layers.2.attn_pre_norm.scale"], torch.ones(64)) and torch.allclose(by["norm.scale"], torch.ones(64))
    layer_kinds = [(layer.attn.cfg.position, layer.attn.cfg.mask, layer.attn.cfg.local_window, layer.is_moe)
                   for layer in res.model.layers]
    assert layer_kinds == [("rope", "sliding_window", 8, False), ("none", "causal", None, True),
                           ("rope", "sliding_window", 8, True), ("none", "causal", None, True)]
    raw = tiny_raw_config(Path("m.json"), kind="trinity")
    raw["model"]["trinity"]["norm_policy"] = "afmoe_dual"
    dual = run_spec_from_mapping(raw).model
    assert trinity_post_norm_scale(dual) == 1.0


def test_trinity_initialisation_statistics_and_untrained_bias():
    res, spec = _build("trinity", hidden_size=256, num_heads=4, intermediate_size=512)
    by = {m.name: (m, res.logical_view(m)) for m in res.metadata}
    want = 0.5 / math.sqrt(256)
    for name in ("layers.0.attn.q.kernel", "layers.1.mlp.experts.gate", "layers.0.mlp.down.kernel", "lm_head.kernel",
                 "embed.embedding"):
        w = by[name][1]
        # a normal cut at two (or three) standard deviations keeps 88-99 % of its spread
        assert 0.8 * want < float(w.std()) < 1.05 * want, (name, float(w.std()), want)
        assert float(w.abs().max()) <= 3.01 * want and abs(float(w.mean())) < 0.1 * want
    bias_meta, bias = by["layers.1.mlp.expert_bias"]
    assert torch.count_nonzero(bias) == 0 and bias.dtype == torch.float32
    assert res.model.layers[1].mlp.expert_bias.requires_grad is False
    again, _ = _build("trinity", hidden_size=256, num_heads=4, intermediate_size=512)
    other, _ = _build("trinity", seed=1, hidden_size=256, num_heads=4, intermediate_size=512)
    assert torch.equal(again.model.embed, res.model.embed) and not torch.equal(other.model.embed, res.model.embed)


def test_parameters_are_fp32_masters_with_no_biases():
    for kind in ("decoder", "trinity"):
        res, _ = _build(kind)
        assert all(p.dtype == torch.float32 for p in res.model.parameters())
        assert not any(m.name.endswith(".bias") for m in res.metadata)
        shapes = {m.name: m.shape for m in res.metadata}
        assert sum(math.prod(s) for s in shapes.values()) == res.parameter_count()
    moe, _ = _build("trinity")
    shapes = {m.name: m.shape for m in moe.metadata}
    assert shapes["layers.1.mlp.experts.gate"] == (4, 64, 32) and shapes["layers.1.mlp.experts.down"] == (4, 32, 64)
    assert shapes["layers.1.mlp.shared_experts.up.kernel"] == (64, 32) and shapes["layers.1.mlp.expert_bias"] == (4,)
