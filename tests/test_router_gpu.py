"""Router kernels (csrc/router.cu) against their PyTorch fp32 restatements."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", ["sigmoid", "softmax"])
@pytest.mark.parametrize("experts,top_k,dtype", [(64, 8, torch.float32), (64, 8, torch.bfloat16),
                                                 (8, 2, torch.float32), (160, 6, torch.float32),
                                                 (1024, 4, torch.float32)])
def test_route_matches_reference_forward_and_backward(kind, experts, top_k, dtype):
    from research_b200.ops import native
    from research_b200.ops.router import _RouteFn, route, route_reference

    torch.manual_seed(experts + top_k)
    T = 3000
    logits = (torch.randn(T, experts, device="cuda") * 1.5).to(dtype)
    bias = torch.randn(experts, device="cuda") * 0.1
    a = logits.clone().requires_grad_(True)
    b = logits.float().clone().requires_grad_(True)
    ids, w, s = route(a, bias, top_k, kind, 2.5)
    native.check_status()
    assert ids.dtype == torch.int64 and w.dtype == torch.float32
    ids_r, w_r, s_r = route_reference(b, bias, top_k, kind, 2.5)
    torch.testing.assert_close(s, s_r, rtol=2e-5, atol=1e-7)
    # the picks carry the same selection values in the same (descending) order; ties may name another expert
    sel, sel_r = (s + bias).gather(-1, ids), (s_r + bias).gather(-1, ids_r)
    torch.testing.assert_close(sel, sel_r, rtol=2e-5, atol=1e-7)
    assert (sel[:, :-1] >= sel[:, 1:]).all()
    assert (ids.sort(dim=-1).values.diff(dim=-1) > 0).all()          # k distinct experts per token
    same = (ids == ids_r).all(dim=-1)
    assert same.float().mean() > (0.9 if dtype == torch.bfloat16 else 0.999)
    torch.testing.assert_close(w[same], w_r[same], rtol=3e-5, atol=1e-7)
    # backward through the weights and the scores (an auxiliary loss reads the scores)
    gw = torch.randn_like(w)
    gs = torch.randn_like(s) * 0.1
    keep = same[:, None].float()
    ((w * gw * keep).sum() + (s * gs).sum()).backward()
    ((w_r * gw * keep).sum() + (s_r * gs).sum()).backward()
    native.check_status()
    tol = dict(rtol=2e-2, atol=2e-3) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(a.grad.float(), b.grad, **tol)
    # weights only (dscores absent)
    a2 = logits.clone().requires_grad_(True)
    ids2, w2, _ = _RouteFn.apply(a2, bias, top_k, kind == "softmax", 2.5)
    (w2 * gw * keep).sum().backward()
    b2 = logits.float().clone().requires_grad_(True)
    _, w2r, _ = route_reference(b2, bias, top_k, kind, 2.5)
    (w2r * gw * keep).sum().backward()
    torch.testing.assert_close(a2.grad.float(), b2.grad, **tol)


def test_route_breaks_ties_towards_the_lower_expert():
    from research_b200.ops.router import route

    logits = torch.zeros(5, 64, device="cuda")
    ids, w, _ = route(logits, torch.zeros(64, device="cuda"), 4, "sigmoid", 1.0)
    assert ids.tolist() == [[0, 1, 2, 3]] * 5
    torch.testing.assert_close(w, torch.full_like(w, 0.25))


@pytest.mark.parametrize("experts", [64, 257])
def test_load_statistics_match_reference(experts):
    from research_b200.ops import native
    from research_b200.ops.router import load_statistics, load_statistics_reference

    torch.manual_seed(1)
    ids = torch.randint(0, experts - 1, (20000, 8), device="cuda")     # the last expert stays empty
    w = torch.rand(20000, 8, device="cuda")
    got = load_statistics(ids, w, experts)
    native.check_status()
    want = load_statistics_reference(ids, w, experts)
    torch.testing.assert_close(got[0], want[0], rtol=0, atol=0)
    torch.testing.assert_close(got[1], want[1], rtol=1e-4, atol=1e-3)
    for g, r in zip(got[2:], want[2:]):
        torch.testing.assert_close(g, r, rtol=1e-5, atol=1e-6)


def test_smebu_kernel_matches_reference_update():
    from research_b200.ops import native
    from research_b200.steps.moe_balance import MoeBalanceLayer, MoeBalanceState, apply_moe_balance_update

    torch.manual_seed(2)
    L, E = 5, 96
    counts = torch.randint(0, 4000, (L, E), device="cuda").float()

    def fresh(device):
        g = torch.Generator().manual_seed(3)
        layers = [MoeBalanceLayer(f"layers.{i}.mlp.expert_bias", (torch.randn(E, generator=g) * 0.01).to(device),
                                  (torch.randn(E, generator=g) * 0.001).to(device)) for i in range(L)]
        return MoeBalanceState("smebu", 1e-2, 0.9, 3.0, layers)

    gpu, cpu = fresh("cuda"), fresh("cpu")
    for _ in range(2):
        m_gpu = apply_moe_balance_update(gpu, counts)
        m_cpu = apply_moe_balance_update(cpu, counts.cpu())
    native.check_status()
    assert gpu.kernel is not None                                       # the native path ran
    for a, b in zip(gpu.layers, cpu.layers):
        torch.testing.assert_close(a.bias.cpu(), b.bias, rtol=1e-5, atol=1e-7)
        torch.testing.assert_close(a.momentum.cpu(), b.momentum, rtol=1e-5, atol=1e-7)
    for key in m_cpu:
        torch.testing.assert_close(m_gpu[key].cpu(), m_cpu[key], rtol=1e-5, atol=1e-7)
