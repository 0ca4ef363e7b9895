"""tcgen05 GEMM against a plain fp32 PyTorch reference, all four operand layouts, tails, batch, accumulate."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, trans_a, trans_b):
    af = a.float().transpose(-1, -2) if trans_a else a.float()
    bf = b.float().transpose(-1, -2) if trans_b else b.float()
    return af @ bf


def _rand(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * 0.5).to(torch.bfloat16)


@pytest.mark.parametrize("trans_a,trans_b", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("mnk", [(128, 256, 64), (256, 512, 256), (384, 320, 192), (200, 136, 72), (1024, 2048, 512)])
def test_gemm_layouts(trans_a, trans_b, mnk):
    from research_b200.ops import native

    M, N, K = mnk
    a = _rand((K, M) if trans_a else (M, K), 1)
    b = _rand((N, K) if trans_b else (K, N), 2)
    out = native.gemm(a, b, trans_a=trans_a, trans_b=trans_b)
    native.check_status()
    ref = _ref(a, b, trans_a, trans_b)
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, (err, scale)


@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_fp32_out_and_accumulate(bn):
    from research_b200.ops import native

    M, N, K = 512, 768, 320
    a, b = _rand((M, K), 3), _rand((N, K), 4)
    out = native.gemm(a, b, out_dtype=torch.float32, bn=bn)
    ref = _ref(a, b, False, True)
    assert (out - ref).abs().max().item() <= 2e-3 * ref.abs().max().item() + 1e-3
    native.gemm(a, b, out=out, accumulate=True, bn=bn)
    native.check_status()
    assert (out - 2 * ref).abs().max().item() <= 4e-3 * ref.abs().max().item() + 2e-3


def test_gemm_batched_and_strided_rows():
    from research_b200.ops import native

    B, M, N, K = 3, 256, 384, 128
    a, b = _rand((B, M, K), 5), _rand((B, N, K), 6)
    out = native.gemm(a, b)
    ref = _ref(a, b, False, True)
    assert (out.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2
    wide = _rand((M, 2 * K), 7)
    a2 = wide[:, :K]  # row stride 2K
    out2 = native.gemm(a2, b[0])
    native.check_status()
    ref2 = _ref(a2, b[0], False, True)
    assert (out2.float() - ref2).abs().max().item() <= 1e-2 * ref2.abs().max().item() + 1e-2


def test_gemm_large_matches_and_is_timed():
    from research_b200.ops import native

    M = N = K = 4096
    a, b = _rand((M, K), 8), _rand((N, K), 9)
    out = native.gemm(a, b)
    ref = (a @ b.t()).float()
    assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
    for _ in range(3):
        native.gemm(a, b, out=out)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(10):
        native.gemm(a, b, out=out)
    e.record()
    torch.cuda.synchronize()
    native.check_status()
    tflops = 10 * 2 * M * N * K / (s.elapsed_time(e) * 1e-3) / 1e12
    print(f"gemm 4096^3: {tflops:.1f} TFLOP/s")
    assert tflops > 50


def test_skinny_splitk_gemm_matches_reference():
    from research_b200.ops import native

    torch.manual_seed(0)
    # the shapes share one fp32 workspace that every call must leave zeroed: large after small and back again
    for rows, n, k in ((32, 2048, 2048), (32, 2048, 5632), (7, 11264, 2048), (64, 4096, 2048), (3, 512, 256),
                       (64, 11264, 2048), (32, 2048, 2048)):
        a = (torch.randn(rows, k, device="cuda") * 0.5).bfloat16()
        b = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
        ref = a.float() @ b.float().t()
        for fused in (False, True):       # finishing pass as its own kernel / inside the product
            y = native.gemm_skinny(a, b, fused_finish=fused)
            native.check_status()
            assert y.shape == (rows, n) and y.dtype == torch.bfloat16
            assert torch.allclose(y.float(), ref, atol=3e-2, rtol=3e-2), (rows, n, k, fused, (y.float() - ref).abs().max().item())
    assert native.splitk_factor(2048, 2048) > 1


def test_weight_gradient_split_k_accumulates_like_one_pass():
    from research_b200.ops import native

    torch.manual_seed(0)
    for tokens, m, n in ((8192, 2048, 2048), (4096, 2048, 5632), (2048, 512, 256)):
        dy = (torch.randn(tokens, m, device="cuda") * 0.1).bfloat16()
        x = (torch.randn(tokens, n, device="cuda") * 0.5).bfloat16()
        grad = torch.full((m, n), 0.25, dtype=torch.float32, device="cuda")
        native.gemm_wgrad(dy, x, grad)
        native.check_status()
        ref = 0.25 + dy.float().t() @ x.float()
        assert (grad - ref).abs().max().item() <= 2e-3 * ref.abs().max().item() + 1e-3
    assert native.wave_splits(2048, 2048, 32768) > 1
