"""Dion2's selection / gather / apply kernels against a plain PyTorch fp32 restatement of the same rules
(reference transform: src/jaxtitan/optim/dion2.py:34-125)."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

EPS, EF = 1e-8, 0.95


def _reference(g, m, w, clip, axis, k, decay, step, o_of, idx=None):
    """g, m, w: [n, rows, cols] fp32 (copies).  ``o_of(stack)`` supplies the orthogonalised stack.  ``idx``: the
    selection to apply (default: the reference's own order, norm descending then index ascending)."""

    m = m + clip * g
    norms = m.double().abs().sum(dim=2 if axis == 0 else 1)
    dim = norms.shape[1]
    if idx is None:
        idx = torch.argsort(norms, dim=1, descending=True, stable=True)[:, :k]
    idx = idx.long()
    n, rows, cols = m.shape
    gidx = idx[:, :, None].expand(n, k, cols) if axis == 0 else idx[:, None, :].expand(n, rows, k)
    sel = torch.gather(m, 1 + axis, gidx)
    stack = sel.to(torch.bfloat16)
    sq = stack.float().pow(2).sum(dim=(1, 2))
    stack = stack / (sq.sqrt().to(torch.bfloat16)[:, None, None] * 1.02 + EPS)
    o = o_of(stack)
    w = w * decay
    w = w.scatter_add(1 + axis, gidx, o.float() * (-step))
    m = m.scatter(1 + axis, gidx, sel * EF)
    inv = torch.full((n, dim), -1, dtype=torch.int32, device=m.device)
    inv.scatter_(1, idx, torch.arange(k, dtype=torch.int32, device=m.device)[None].expand(n, k))
    return m, w, stack, idx.to(torch.int32), inv, norms


@pytest.mark.parametrize("axis", [0, 1])
@pytest.mark.parametrize("n,rows,cols,pad_rows", [(1, 64, 128, 0), (3, 96, 72, 0), (4, 128, 256, 64), (2, 1024, 520, 0)])
def test_dion2_kernels_match_the_plain_rules(axis, n, rows, cols, pad_rows):
    from research_b200.ops import native

    torch.manual_seed(axis * 10 + n)
    dev = torch.device("cuda")
    total = rows + pad_rows                                   # matrices are row ranges of a larger fused entry
    g_full = torch.randn(n, total, cols, device=dev)
    m_full = torch.randn(n, total, cols, device=dev) * 0.3
    w_full = torch.randn(n, total, cols, device=dev)
    sh_full = torch.zeros(n, total, cols, device=dev, dtype=torch.bfloat16)
    r0 = pad_rows // 2
    g, m, w, sh = (t[:, r0:r0 + rows] for t in (g_full, m_full, w_full, sh_full))
    clip = torch.tensor([0.5], device=dev)
    k = max(1, math.ceil(0.25 * (rows if axis == 0 else cols)))
    stride = total * cols
    assert native.dion2_supported(n, rows, cols, stride, axis)
    decay, step = 1.0 - 3e-4 * 0.1, 2e-3
    gen = torch.Generator(device=dev).manual_seed(5)
    o = torch.randn((n, k, cols) if axis == 0 else (n, rows, k), device=dev, generator=gen).to(torch.bfloat16)
    before = m_full.clone(), w_full.clone()
    g0, m0, w0 = g.clone(), m.clone(), w.clone()

    stack, idx, inv = native.dion2_select_stack(g, m, clip, n, rows, cols, stride, axis, k, EPS)
    # the kernel's order against float64 norms: non-increasing, and nothing left out is larger than what was taken,
    # both up to the rounding of an fp32 sum (two slices whose norms agree to 1e-5 may come in either order)
    *_, norms = _reference(g0, m0, w0, 0.5, axis, k, decay, step, lambda s: o)
    taken = torch.gather(norms, 1, idx.long())
    tol = 2e-5 * norms.max().item()
    assert (taken[:, 1:] <= taken[:, :-1] + tol).all()
    left = norms.scatter(1, idx.long(), float("-inf"))
    assert (left.max(dim=1).values <= taken[:, -1] + tol).all()
    assert all(len(set(row.tolist())) == k for row in idx)
    m_ref, w_ref, stack_ref, idx_ref, inv_ref, _ = _reference(g0, m0, w0, 0.5, axis, k, decay, step, lambda s: o, idx=idx)
    assert torch.equal(inv, inv_ref)
    assert torch.allclose(stack.float(), stack_ref.float(), rtol=2 ** -7, atol=1e-6)      # at most one bf16 step
    assert (stack.float() - stack_ref.float()).abs().gt(0).float().mean() < 0.02           # and nearly always none
    native.dion2_apply(w, m, o, inv, sh, n, rows, cols, k, stride, axis, decay, step, EF)
    torch.cuda.synchronize()
    assert torch.allclose(m, m_ref, rtol=1e-6, atol=1e-7)
    assert torch.allclose(w, w_ref, rtol=1e-6, atol=1e-6)
    assert torch.equal(sh, w.to(torch.bfloat16))
    if pad_rows:                                                                             # rows outside stay untouched
        outside = torch.ones(total, dtype=torch.bool, device=dev)
        outside[r0:r0 + rows] = False
        assert torch.equal(m_full[:, outside], before[0][:, outside])
        assert torch.equal(w_full[:, outside], before[1][:, outside])
        assert not sh_full[:, outside].any()


def test_dion2_selection_is_repeatable_and_breaks_ties_by_index():
    from research_b200.ops import native

    dev = torch.device("cuda")
    rows, cols = 64, 32
    m = torch.zeros(1, rows, cols, device=dev)
    m[0, :, 0] = torch.tensor([float(i % 4) for i in range(rows)], device=dev)              # 16-way ties
    g = torch.zeros_like(m)
    k = 16
    out = [native.dion2_select_stack(g, m, None, 1, rows, cols, rows * cols, 0, k, EPS) for _ in range(2)]
    assert torch.equal(out[0][1], out[1][1]) and torch.equal(out[0][0], out[1][0])
    assert out[0][1][0].tolist() == [i for i in range(rows) if i % 4 == 3]


def test_dion2_rejects_sizes_outside_its_rules():
    from research_b200.ops import native

    assert not native.dion2_supported(1, 64, 66, 64 * 66, 0)
    assert not native.dion2_supported(1, 64, 16384, 64 * 16384, 1)
    assert native.dion2_supported(1, 16384, 64, 64 * 16384, 1)
