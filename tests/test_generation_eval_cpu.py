"""Generation cache and sampler, evaluation loss, learning-rate schedules and SMEBU balancing on the CPU paths."""

import math
from pathlib import Path

import pytest
import torch

from research_b200.config import run_spec_from_mapping
from research_b200.config.specs import MoeBalanceSpec, ScheduleSpec
from research_b200.errors import ContractError
from research_b200.infer.generation import PagedKVCache, generate_tokens, init_kv_cache, sample_next_token
from research_b200.models.build import build_model
from research_b200.optim.schedules import build_lr_schedule
from research_b200.steps.eval import causal_lm_loss
from research_b200.steps.moe_balance import apply_moe_balance_update, init_moe_balance, router_diagnostics
from tests.helpers import tiny_raw_config


def _model(kind="decoder", **extra):
    spec = run_spec_from_mapping(tiny_raw_config(Path("m.json"), kind=kind, extra_model=extra or None))
    return build_model(spec.model, seed=0), spec


def _cache(batch=2, max_len=10, page=4, heads=2, dim=4, layers=1):
    return PagedKVCache(layers=layers, batch=batch, max_len=max_len, kv_heads=heads, head_dim=dim, page_size=page,
                        dtype=torch.float32, device=torch.device("cpu"))


# ---------------------------------------------------------------------------------------------- paged cache


def test_cache_rounds_capacity_up_to_whole_pages_and_owns_disjoint_pages():
    c = _cache(batch=3, max_len=10, page=4)
    assert c.pages_per_seq == 3 and c.max_len == 12
    assert c.k.shape == (1, 9, 2, 4, 4) and c.v.shape == c.k.shape
    assert c.page_table.tolist() == [[0, 1, 2], [3, 4, 5], [6, 7, 8]]
    assert c.lengths.tolist() == [0, 0, 0]


@pytest.mark.parametrize("prompt", [3, 4, 7, 8])
def test_cache_prefill_block_copy_equals_scatter_write(prompt):
    """A prompt written from row 0 takes the page-wise block copy; any other start takes the indexed write."""

    torch.manual_seed(prompt)
    B, H, D = 2, 2, 4
    k, v, q = torch.randn(B, prompt, H, D), torch.randn(B, prompt, H, D), torch.randn(B, prompt, 4, D)
    pos = torch.arange(prompt, dtype=torch.int32).expand(B, prompt).contiguous()
    blocked = _cache()
    out_a = blocked.update_and_attend(0, q, k, v, pos, None)
    scattered = _cache()
    outs = [scattered.update_and_attend(0, q[:, t:t + 1], k[:, t:t + 1], v[:, t:t + 1], pos[:, t:t + 1], None)
            for t in range(prompt)]
    assert torch.equal(blocked.k, scattered.k) and torch.equal(blocked.v, scattered.v)
    assert torch.allclose(out_a, torch.cat(outs, dim=1), atol=1e-5)
    assert torch.equal(blocked._rows(blocked.k, 0, prompt), k)


def test_cache_window_limits_the_keys_a_query_sees():
    torch.manual_seed(0)
    B, T, H, D = 1, 8, 1, 4
    k, v, q = torch.randn(B, T, H, D), torch.randn(B, T, H, D), torch.randn(B, T, 2, D)
    pos = torch.arange(T, dtype=torch.int32)[None]
    base = _cache(batch=1).update_and_attend(0, q, k, v, pos, 3)
    v2 = v.clone()
    v2[:, :5] += 50.0                                   # rows 0..4 are outside the window of query 7 (keys 5, 6, 7)
    moved = _cache(batch=1).update_and_attend(0, q, k, v2, pos, 3)
    assert torch.allclose(base[:, 7], moved[:, 7]) and not torch.allclose(base[:, 6], moved[:, 6])


def test_cache_advance_keeps_the_longest_length_seen():
    c = _cache()
    c.advance(torch.tensor([[0, 1, 2], [0, 1, 2]], dtype=torch.int32))
    assert c.lengths.tolist() == [3, 3]
    c.advance(torch.tensor([[1], [5]], dtype=torch.int32))
    assert c.lengths.tolist() == [3, 6] and c.lengths.dtype == torch.int32


def test_init_kv_cache_takes_geometry_from_the_model():
    res, spec = _model()
    c = init_kv_cache(res.model, 3, 20, page_size=8)
    assert c.k.shape == (spec.model.num_layers, 3 * 3, 2, 8, spec.model.head_dim)
    assert c.k.dtype == next(res.model.parameters()).dtype


# ---------------------------------------------------------------------------------------------- sampler


def test_sampler_rejects_bad_settings():
    logits = torch.zeros(1, 4)
    for kwargs, match in ((dict(temperature=0.0, top_k=None), "temperature"),
                          (dict(temperature=-1.0, top_k=None), "temperature"),
                          (dict(temperature=1.0, top_k=0), "top_k"),
                          (dict(temperature=1.0, top_k=-3), "top_k")):
        with pytest.raises(ContractError, match=match):
            sample_next_token(logits, top_p=None, generator=None, **kwargs)


def test_sampler_logprob_is_of_the_truncated_tempered_distribution():
    logits = torch.tensor([[1.0, 3.0, 2.0, 0.0], [0.5, 0.5, 4.0, 1.0]])
    g = torch.Generator().manual_seed(3)
    tok, lp = sample_next_token(logits, temperature=0.5, top_k=2, top_p=None, generator=g)
    for b in range(2):
        scaled = logits[b] / 0.5
        keep = torch.topk(scaled, 2).indices
        want = scaled[tok[b]] - torch.logsumexp(scaled[keep], 0)
        assert tok[b].item() in keep.tolist() and lp[b].item() == pytest.approx(want.item(), abs=1e-6)


def test_sampler_top_k_larger_than_the_vocabulary_is_the_full_distribution():
    logits = torch.tensor([[0.1, 0.2, 0.3]])
    a = sample_next_token(logits, temperature=1.0, top_k=100, top_p=None, generator=torch.Generator().manual_seed(5))
    b = sample_next_token(logits, temperature=1.0, top_k=None, top_p=None, generator=torch.Generator().manual_seed(5))
    assert a[0].item() == b[0].item() and a[1].item() == pytest.approx(b[1].item())


def test_sampler_frequencies_follow_the_softmax():
    logits = torch.log(torch.tensor([[0.6, 0.3, 0.1]])).expand(4000, 3).contiguous()
    tok, _ = sample_next_token(logits, temperature=1.0, top_k=None, top_p=None, generator=torch.Generator().manual_seed(0))
    freq = torch.bincount(tok, minlength=3).float() / 4000
    assert torch.allclose(freq, torch.tensor([0.6, 0.3, 0.1]), atol=0.03)


def test_sampler_low_temperature_approaches_greedy():
    logits = torch.tensor([[0.0, 1.0, 0.9]]).expand(200, 3).contiguous()
    tok, _ = sample_next_token(logits, temperature=0.01, top_k=None, top_p=None, generator=torch.Generator().manual_seed(1))
    assert (tok == 1).all()


# ---------------------------------------------------------------------------------------------- generation


def test_generation_seed_controls_the_draws():
    res, _ = _model()
    prompt = torch.tensor([[5, 6, 7, 8]])
    a = generate_tokens(res.model, prompt, max_new_tokens=6, temperature=1.5, seed=11, page_size=4)
    b = generate_tokens(res.model, prompt, max_new_tokens=6, temperature=1.5, seed=11, page_size=4)
    seeds = {tuple(generate_tokens(res.model, prompt, max_new_tokens=6, temperature=1.5, seed=s).generated_ids[0])
             for s in range(6)}
    assert a.generated_ids == b.generated_ids and a.logprobs == b.logprobs and len(seeds) > 1


def test_generation_page_size_does_not_change_greedy_output():
    res, _ = _model()
    prompt = torch.tensor([[9, 3, 200, 17, 4]])
    outs = [generate_tokens(res.model, prompt, max_new_tokens=7, top_k=1, page_size=p).generated_ids for p in (2, 5, 128)]
    assert outs[0] == outs[1] == outs[2]


@pytest.mark.parametrize("kind", ["decoder", "trinity"])
def test_generation_batch_rows_are_independent(kind):
    res, _ = _model(kind)
    prompts = torch.tensor([[1, 2, 3, 4], [40, 30, 20, 10]])
    both = generate_tokens(res.model, prompts, max_new_tokens=5, top_k=1, page_size=4)
    for b in range(2):
        alone = generate_tokens(res.model, prompts[b:b + 1], max_new_tokens=5, top_k=1, page_size=4)
        assert both.generated_ids[b] == alone.generated_ids[0]
        assert both.logprobs[b] == pytest.approx(alone.logprobs[0], abs=1e-4)


def test_generation_greedy_logprobs_match_a_full_forward():
    res, _ = _model()
    out = generate_tokens(res.model, torch.tensor([[3, 1, 4, 1, 5]]), max_new_tokens=4, top_k=1, page_size=4)
    full = torch.tensor(out.full_ids, dtype=torch.int32)
    with torch.no_grad():
        logits = res.model.eval()(full).logits[0].float()
    for j, (tok, lp) in enumerate(zip(out.generated_ids[0], out.logprobs[0])):
        row = logits[5 + j - 1]
        assert int(row.argmax()) == tok
        assert lp == pytest.approx(0.0)                 # top_k=1 renormalises over one token
    sampled = generate_tokens(res.model, torch.tensor([[3, 1, 4, 1, 5]]), max_new_tokens=3, temperature=1.0, seed=2)
    full = torch.tensor(sampled.full_ids, dtype=torch.int32)
    with torch.no_grad():
        logp = torch.log_softmax(res.model(full).logits[0].float(), -1)
    for j, (tok, lp) in enumerate(zip(sampled.generated_ids[0], sampled.logprobs[0])):
        assert lp == pytest.approx(logp[5 + j - 1, tok].item(), abs=2e-4)


def test_generation_restores_training_mode_and_checks_arguments():
    res, _ = _model()
    res.model.train()
    generate_tokens(res.model, torch.tensor([[1, 2]]), max_new_tokens=1, top_k=1)
    assert res.model.training
    with pytest.raises(ContractError, match="max_new_tokens"):
        generate_tokens(res.model, torch.tensor([[1, 2]]), max_new_tokens=0)
    exact = generate_tokens(res.model, torch.tensor([[1] * 60]), max_new_tokens=4, top_k=1)    # 64 == max_seq_len
    assert len(exact.full_ids[0]) == 64


# ---------------------------------------------------------------------------------------------- evaluation loss


def test_causal_lm_loss_is_a_masked_sum_and_a_count():
    torch.manual_seed(0)
    logits, targets = torch.randn(2, 5, 7), torch.randint(0, 7, (2, 5))
    mask = torch.tensor([[1, 1, 0, 1, 0], [0, 0, 0, 0, 1]])
    total, count = causal_lm_loss(logits, targets, mask)
    want = torch.nn.functional.cross_entropy(logits.reshape(-1, 7), targets.reshape(-1), reduction="none").view(2, 5)
    assert count.item() == 4 and total.item() == pytest.approx((want * mask).sum().item(), rel=1e-6)
    zero, none = causal_lm_loss(logits, targets, torch.zeros(2, 5))
    assert zero.item() == 0.0 and none.item() == 0.0
    half, _ = causal_lm_loss(logits.bfloat16(), targets.int(), mask)       # reduced-precision logits, int32 targets
    assert half.dtype == torch.float32 and half.item() == pytest.approx(total.item(), rel=2e-2)


# ---------------------------------------------------------------------------------------------- schedules


def test_constant_schedule_warms_up_linearly_from_one_step():
    lr = build_lr_schedule(ScheduleSpec(peak_lr=2.0, name="constant", warmup_steps=4))
    assert [lr(i) for i in range(6)] == pytest.approx([0.5, 1.0, 1.5, 2.0, 2.0, 2.0])
    flat = build_lr_schedule(ScheduleSpec(peak_lr=0.3, name="constant"))
    assert flat(0) == flat(10 ** 6) == 0.3


def test_cosine_schedule_hits_peak_midpoint_and_floor():
    lr = build_lr_schedule(ScheduleSpec(peak_lr=1.0, name="cosine", warmup_steps=2, total_steps=12, min_lr_ratio=0.1))
    assert lr(0) == pytest.approx(0.5) and lr(1) == pytest.approx(1.0) and lr(2) == pytest.approx(1.0)
    assert lr(11) == pytest.approx(0.1) and lr(500) == pytest.approx(0.1)
    mid = 0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * 4.5 / 9))
    assert lr(2 + 4.5) == pytest.approx(mid)
    values = [lr(i) for i in range(2, 12)]
    assert all(a >= b for a, b in zip(values, values[1:]))
    one = build_lr_schedule(ScheduleSpec(peak_lr=1.0, name="cosine", warmup_steps=3, total_steps=4, min_lr_ratio=0.25))
    assert one(3) == pytest.approx(0.25)                # a single decay step sits on the floor


def test_wsd_schedule_has_a_plateau_and_a_default_decay_tenth():
    lr = build_lr_schedule(ScheduleSpec(peak_lr=1.0, name="wsd", warmup_steps=2, total_steps=20, stable_steps=10))
    assert lr(1) == 1.0 and lr(2) == 1.0 and lr(11) == 1.0 and lr(12) == pytest.approx(1.0) and lr(13) < 1.0
    assert lr(19) == pytest.approx(0.0, abs=1e-12)
    auto = build_lr_schedule(ScheduleSpec(peak_lr=1.0, name="wsd", warmup_steps=10, total_steps=100))
    assert auto(89) == 1.0 and auto(90) == pytest.approx(1.0) and auto(91) < 1.0 and auto(99) == pytest.approx(0.0, abs=1e-12)


def test_schedule_contract_errors():
    with pytest.raises(ContractError, match="total_steps is required"):
        build_lr_schedule(ScheduleSpec(peak_lr=1.0, name="cosine", warmup_steps=1))
    with pytest.raises(ContractError, match="total_steps > warmup_steps"):
        build_lr_schedule(ScheduleSpec(peak_lr=1.0, name="cosine", warmup_steps=5, total_steps=5))
    with pytest.raises(ContractError, match="warmup_steps \\+ stable_steps"):
        build_lr_schedule(ScheduleSpec(peak_lr=1.0, name="wsd", warmup_steps=5, total_steps=10, stable_steps=5))
    with pytest.raises(ContractError):
        ScheduleSpec(peak_lr=0.0)
    with pytest.raises(ContractError):
        ScheduleSpec(peak_lr=1.0, name="linear")


# ---------------------------------------------------------------------------------------------- SMEBU


def test_smebu_state_covers_only_moe_layers():
    res, spec = _model("trinity")
    state = init_moe_balance(res.model, MoeBalanceSpec(name="smebu"))
    assert [l.path for l in state.layers] == ["layers.1.mlp.expert_bias"]
    assert state.layers[0].bias.data_ptr() == res.model.layers[1].mlp.expert_bias.data_ptr()
    assert init_moe_balance(res.model, None) is None and init_moe_balance(res.model, MoeBalanceSpec()) is None
    dense, _ = _model("decoder")
    assert init_moe_balance(dense.model, MoeBalanceSpec(name="smebu")) is None


def test_smebu_update_follows_the_formula_and_stays_centred():
    res, _ = _model("trinity")
    spec = MoeBalanceSpec(name="smebu", load_lr=0.1, momentum=0.5, clamp=2.0)
    state = init_moe_balance(res.model, spec)
    counts = torch.tensor([[10.0, 2.0, 4.0, 0.0]])
    bias0 = state.layers[0].bias.clone()
    out = apply_moe_balance_update(state, counts)
    violation = (4.0 - counts[0]) / 4.0
    delta = 0.1 * torch.tanh(2.0 * violation)
    delta = delta - delta.mean()
    assert torch.allclose(state.layers[0].momentum, 0.5 * delta, atol=1e-7)
    assert torch.allclose(state.layers[0].bias, bias0 + 0.5 * delta, atol=1e-7)
    assert state.layers[0].momentum.sum().abs().item() < 1e-6
    assert state.layers[0].bias[0] < bias0[0] and state.layers[0].bias[3] > bias0[3]   # overloaded down, idle up
    assert out["smebu_momentum_norm"].item() == pytest.approx((0.5 * delta).norm().item(), rel=1e-5)
    apply_moe_balance_update(state, counts)
    assert torch.allclose(state.layers[0].momentum, 0.75 * delta, atol=1e-7)
    assert torch.allclose(state.layers[0].bias, bias0 + 1.25 * delta, atol=1e-6)


def test_smebu_balanced_counts_and_missing_inputs_change_nothing():
    res, _ = _model("trinity")
    state = init_moe_balance(res.model, MoeBalanceSpec(name="smebu"))
    before = state.layers[0].bias.clone()
    apply_moe_balance_update(state, torch.full((1, 4), 6.0))
    assert torch.equal(state.layers[0].bias, before)
    assert apply_moe_balance_update(state, None) == {} and apply_moe_balance_update(None, torch.ones(1, 4)) == {}
    with pytest.raises(ContractError, match="router count shape"):
        apply_moe_balance_update(state, torch.ones(2, 4))


def test_router_diagnostics_on_known_loads():
    counts = torch.tensor([[4.0, 4.0, 4.0, 4.0], [8.0, 0.0, 4.0, 4.0]])
    d = router_diagnostics(counts, counts.clone())
    assert d["router_max_vio"].item() == pytest.approx(1.0)
    assert d["router_load_min"].item() == 0.0 and d["router_load_max"].item() == 8.0
    assert d["router_dead_experts_count"].item() == 1.0 and d["router_experts_active_mean"].item() == pytest.approx(3.5)
    uniform = math.log(4.0)
    skew = -(0.5 * math.log(0.5) + 2 * 0.25 * math.log(0.25))
    assert d["router_mean_load_entropy"].item() == pytest.approx((uniform + skew) / 2, rel=1e-5)
    assert d["router_min_load_entropy"].item() == pytest.approx(skew, rel=1e-5)
    cv = math.sqrt(8.0) / 4.0
    assert d["router_mean_load_cv"].item() == pytest.approx(cv / 2, rel=1e-5)
    assert d["router_mean_importance_cv"].item() == pytest.approx(cv / 2, rel=1e-5)
