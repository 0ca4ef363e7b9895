"""Flash attention kernels against a naive fp32 attention with the same masks."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bf(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def naive_attention(q, k, v, causal, lo, scale):
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    g = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    s = torch.einsum("bhqd,bhkd->bhqk", qf, kf) * scale
    idx = torch.arange(S, device=q.device)
    allowed = torch.ones(B, 1, S, S, dtype=torch.bool, device=q.device)
    if causal:
        allowed = allowed & (idx[None, None, :, None] >= idx[None, None, None, :])
    if lo is not None:
        allowed = allowed & (idx[None, None, None, :] >= lo.long()[:, None, :, None])
    s = s.masked_fill(~allowed, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("bhqk,bhkd->bhqd", p, vf).permute(0, 2, 1, 3)
    return o, lse


def doc_lo(B, S, mean_len, seed):
    g = torch.Generator().manual_seed(seed)
    lo = torch.zeros(B, S, dtype=torch.int32)
    for b in range(B):
        pos = 0
        while pos < S:
            n = int(torch.empty(1).exponential_(1.0 / mean_len, generator=g).item()) + 1
            lo[b, pos:pos + n] = pos
            pos += n
    return lo.cuda()


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("S,causal,docs", [(256, True, False), (512, True, True), (384, False, False), (1000, True, True)])
def test_attn_fwd(D, S, causal, docs):
    from research_b200.ops import native

    B, Hq, Hkv = 2, 4, 2
    packed = _bf((B, S, (Hq + 2 * Hkv) * D), 1)
    q = packed[..., : Hq * D].view(B, S, Hq, D)
    k = packed[..., Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D)
    v = packed[..., (Hq + Hkv) * D:].view(B, S, Hkv, D)
    lo = doc_lo(B, S, 150, 3) if docs else None
    o, lse = native.attn_fwd(q, k, v, causal=causal, lo=lo)
    native.check_status()
    ref_o, ref_lse = naive_attention(q, k, v, causal, lo, D ** -0.5)
    assert torch.allclose(lse, ref_lse, atol=2e-2, rtol=1e-3), (lse - ref_lse).abs().max()
    assert torch.allclose(o.float(), ref_o, atol=2e-2, rtol=2e-2), (o.float() - ref_o).abs().max()


def test_attn_fwd_sliding_window_and_speed():
    from research_b200.ops import native

    B, S, Hq, Hkv, D, W = 1, 2048, 4, 4, 128, 300
    q, k, v = _bf((B, S, Hq, D), 1), _bf((B, S, Hkv, D), 2), _bf((B, S, Hkv, D), 3)
    lo = (torch.arange(S, device="cuda", dtype=torch.int32) - (W - 1)).clamp_min(0)[None].contiguous()
    o, lse = native.attn_fwd(q, k, v, causal=True, lo=lo)
    native.check_status()
    ref_o, ref_lse = naive_attention(q, k, v, True, lo, D ** -0.5)
    assert torch.allclose(o.float(), ref_o, atol=2e-2, rtol=2e-2)
    B, S, Hq, Hkv = 8, 4096, 16, 8
    q, k, v = _bf((B, S, Hq, D), 4), _bf((B, S, Hkv, D), 5), _bf((B, S, Hkv, D), 6)
    for _ in range(3):
        native.attn_fwd(q, k, v, causal=True)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(10):
        native.attn_fwd(q, k, v, causal=True)
    e.record()
    torch.cuda.synchronize()
    native.check_status()
    ms = s.elapsed_time(e) / 10
    flops = 4 * B * Hq * S * S * D / 2
    print(f"attn fwd causal B8 S4096 H16 D128: {ms:.3f} ms, {flops / ms / 1e9:.1f} TFLOP/s")


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("S,causal,docs", [(256, True, False), (512, True, True), (384, False, False), (1000, True, True)])
def test_attn_bwd(D, S, causal, docs):
    from research_b200.ops import native

    B, Hq, Hkv = 2, 4, 2
    q, k, v = _bf((B, S, Hq, D), 1), _bf((B, S, Hkv, D), 2), _bf((B, S, Hkv, D), 3)
    d_o = _bf((B, S, Hq, D), 4, 0.5)
    lo = doc_lo(B, S, 150, 3) if docs else None
    o, lse = native.attn_fwd(q, k, v, causal=causal, lo=lo)
    dq, dk, dv = native.attn_bwd(q, k, v, o, d_o, lse, causal=causal, lo=lo)
    native.check_status()
    qr, kr, vr = (t.float().requires_grad_(True) for t in (q, k, v))
    ref_o, _ = naive_attention(qr, kr, vr, causal, lo, D ** -0.5)
    ref_o.backward(d_o.float())
    for name, got, ref in (("dq", dq, qr.grad), ("dk", dk, kr.grad), ("dv", dv, vr.grad)):
        err = (got.float() - ref).abs().max().item()
        scale = ref.abs().max().item()
        assert err <= 2e-2 * scale + 2e-2, (name, err, scale)


def test_attn_bwd_speed():
    from research_b200.ops import native

    B, S, Hq, Hkv, D = 8, 4096, 16, 8, 128
    q, k, v = _bf((B, S, Hq, D), 4), _bf((B, S, Hkv, D), 5), _bf((B, S, Hkv, D), 6)
    d_o = _bf((B, S, Hq, D), 7)
    o, lse = native.attn_fwd(q, k, v, causal=True)
    for _ in range(3):
        native.attn_bwd(q, k, v, o, d_o, lse, causal=True)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(10):
        native.attn_bwd(q, k, v, o, d_o, lse, causal=True)
    e.record()
    torch.cuda.synchronize()
    native.check_status()
    ms = s.elapsed_time(e) / 10
    flops = 10 * B * Hq * S * S * D / 2
    print(f"attn bwd causal B8 S4096 H16 D128: {ms:.3f} ms, {flops / ms / 1e9:.1f} TFLOP/s (5-GEMM count)")


@pytest.mark.parametrize("docs", [False, True])
def test_attn_context_parallel_offsets(docs):
    """Queries of a later sequence chunk against all earlier keys: the same numbers as the full computation."""

    from research_b200.ops import native

    B, S, Hq, Hkv, D, chunks = 1, 1024, 4, 2, 128, 4
    q, k, v = _bf((B, S, Hq, D), 1), _bf((B, S, Hkv, D), 2), _bf((B, S, Hkv, D), 3)
    d_o = _bf((B, S, Hq, D), 4, 0.5)
    lo = doc_lo(B, S, 200, 5) if docs else None
    o_full, lse_full = native.attn_fwd(q, k, v, causal=True, lo=lo)
    dq_full, dk_full, dv_full = native.attn_bwd(q, k, v, o_full, d_o, lse_full, causal=True, lo=lo)
    n = S // chunks
    dk_sum, dv_sum = torch.zeros_like(k, dtype=torch.float32), torch.zeros_like(v, dtype=torch.float32)
    for r in range(chunks):
        qs = slice(r * n, (r + 1) * n)
        kv_len = (r + 1) * n
        lo_r = None if lo is None else lo[:, qs].contiguous()
        o, lse = native.attn_fwd(q[:, qs], k[:, :kv_len], v[:, :kv_len], causal=True, lo=lo_r, q_offset=r * n)
        assert torch.allclose(o.float(), o_full[:, qs].float(), atol=2e-2, rtol=2e-2)
        assert torch.allclose(lse, lse_full[:, :, qs], atol=2e-2, rtol=1e-3)
        hi = None if lo_r is None else native.kv_visibility_upper_bound(lo_r, kv_len, r * n)
        dq, dk, dv = native.attn_bwd(q[:, qs], k[:, :kv_len], v[:, :kv_len], o, d_o[:, qs], lse, causal=True, lo=lo_r,
                                     hi=hi, q_offset=r * n)
        assert torch.allclose(dq.float(), dq_full[:, qs].float(), atol=3e-2, rtol=3e-2)
        dk_sum[:, :kv_len] += dk.float()
        dv_sum[:, :kv_len] += dv.float()
    native.check_status()
    assert (dk_sum - dk_full.float()).abs().max() <= 3e-2 * dk_full.float().abs().max() + 3e-2
    assert (dv_sum - dv_full.float()).abs().max() <= 3e-2 * dv_full.float().abs().max() + 3e-2
