"""Decode attention kernel and GPU generation against fp32 restatements."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("D,Hq,Hkv", [(128, 16, 8), (128, 8, 8), (64, 16, 4), (64, 32, 4), (128, 4, 1)])
def test_decode_attention_matches_reference(D, Hq, Hkv):
    from research_b200.ops import native
    from research_b200.ops.decode import decode_attention, decode_attention_reference

    torch.manual_seed(0)
    B, rows = 5, 700
    q = torch.randn(B, Hq, D, device="cuda").bfloat16()
    # caches as views into a wider packed buffer, like the paged pool
    kc = torch.randn(B, rows, Hkv, D, device="cuda").bfloat16()
    vc = torch.randn(B, rows, Hkv, D, device="cuda").bfloat16()
    lengths = torch.tensor([1, 17, 256, 699, 700], device="cuda", dtype=torch.int32)
    for lo in (None, torch.tensor([0, 3, 100, 650, 0], device="cuda", dtype=torch.int32)):
        out = decode_attention(q, kc, vc, lengths, lo)
        ref = decode_attention_reference(q, kc, vc, lengths, lo)
        native.check_status()
        assert out.shape == (B, Hq * D)
        assert torch.allclose(out.float(), ref.float(), atol=2e-2, rtol=2e-2), (out.float() - ref.float()).abs().max()


def test_paged_decode_and_append_match_dense_cache():
    from research_b200.ops import native
    from research_b200.ops.decode import decode_attention_paged, decode_attention_reference, kv_append_paged

    torch.manual_seed(1)
    B, pages, Hkv, ps, D, Hq = 3, 5, 4, 128, 128, 8
    kp = torch.randn(B, pages, Hkv, ps, D, device="cuda").bfloat16()
    vp = torch.randn(B, pages, Hkv, ps, D, device="cuda").bfloat16()
    pos = torch.tensor([0, 300, 639], device="cuda", dtype=torch.int32)
    packed = torch.randn(B, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()   # new k / v as views of a packed row
    k_new = packed[:, Hq * D:(Hq + Hkv) * D].view(B, Hkv, D)
    v_new = packed[:, (Hq + Hkv) * D:].view(B, Hkv, D)
    kv_append_paged(k_new, v_new, kp, vp, pos)
    dense_k = kp.permute(0, 1, 3, 2, 4).reshape(B, pages * ps, Hkv, D)
    dense_v = vp.permute(0, 1, 3, 2, 4).reshape(B, pages * ps, Hkv, D)
    for b in range(B):
        assert torch.equal(dense_k[b, int(pos[b])], k_new[b]) and torch.equal(dense_v[b, int(pos[b])], v_new[b])
    q = torch.randn(B, Hq, D, device="cuda").bfloat16()
    out = decode_attention_paged(q, kp, vp, pos + 1, None)
    native.check_status()
    ref = decode_attention_reference(q, dense_k, dense_v, pos + 1, None)
    assert torch.allclose(out.float(), ref.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("D,Hq,Hkv,page_rows", [(128, 16, 8, 128), (128, 8, 8, 64), (64, 16, 4, 128), (128, 16, 2, 64)])
def test_streaming_paged_decode_matches_reference_and_register_kernel(D, Hq, Hkv, page_rows):
    """The tile-streaming kernel (bulk copies into shared memory) against the fp32 restatement and the
    register-resident kernel, with ragged lengths, a lower bound that does not sit on a tile edge, an empty
    window and a sequence that ends on the first row of a page."""
    from research_b200.ops import native
    from research_b200.ops.decode import decode_attention_paged, decode_attention_reference

    torch.manual_seed(D + Hq + page_rows)
    B, pages = 5, 1024 // page_rows
    q = (torch.randn(B, Hq, D, device="cuda") * 0.7).bfloat16()
    kp = (torch.randn(B, pages, Hkv, page_rows, D, device="cuda") * 0.7).bfloat16()
    vp = torch.randn(B, pages, Hkv, page_rows, D, device="cuda").bfloat16()
    lengths = torch.tensor([1024, 517, 1, page_rows + 1, 300], device="cuda", dtype=torch.int32)
    lo = torch.tensor([0, 45, 0, 3, 300], device="cuda", dtype=torch.int32)       # the last window is empty
    dense_k = kp.permute(0, 1, 3, 2, 4).reshape(B, pages * page_rows, Hkv, D)
    dense_v = vp.permute(0, 1, 3, 2, 4).reshape(B, pages * page_rows, Hkv, D)
    for bounds in (None, lo):
        want = decode_attention_reference(q, dense_k, dense_v, lengths, bounds).float()
        got = decode_attention_paged(q, kp, vp, lengths, bounds, kernel="stream").float()
        regs = decode_attention_paged(q, kp, vp, lengths, bounds, kernel="registers").float()
        native.check_status()
        torch.testing.assert_close(got, want, atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(got, regs, atol=1e-2, rtol=1e-2)
        # queries left where the projection wrote them: rows of a packed q|k buffer, read without a copy
        packed = torch.zeros(B, (Hq + Hkv) * D, device="cuda", dtype=torch.bfloat16)
        packed[:, : Hq * D] = q.reshape(B, Hq * D)
        strided = packed[:, : Hq * D].view(B, Hq, D)
        assert not strided.is_contiguous()
        assert torch.equal(decode_attention_paged(strided, kp, vp, lengths, bounds, kernel="stream").float(), got)
    assert torch.count_nonzero(got[4]) == 0


def test_decode_attention_empty_window_gives_zeros():
    from research_b200.ops.decode import decode_attention

    q = torch.randn(2, 4, 64, device="cuda").bfloat16()
    kc = torch.randn(2, 64, 4, 64, device="cuda").bfloat16()
    vc = torch.randn(2, 64, 4, 64, device="cuda").bfloat16()
    out = decode_attention(q, kc, vc, torch.tensor([0, 5], device="cuda", dtype=torch.int32),
                           torch.tensor([0, 9], device="cuda", dtype=torch.int32))
    assert torch.count_nonzero(out) == 0


def test_generation_native_decode_matches_masked_attention(monkeypatch):
    """Teacher-forced logits with the native prefill/decode kernels against the dense masked-attention path."""

    from research_b200.config import run_spec_from_mapping
    from research_b200.infer import generation
    from research_b200.ops import native
    from research_b200.runtime.trainer import Trainer

    raw = {
        "run": {"id": "gen-parity"},
        "model": {"name": "decoder", "variant": "t", "vocab_size": 512, "hidden_size": 256, "intermediate_size": 512,
                  "num_layers": 2, "num_heads": 4, "n_kv_heads": 2, "max_seq_len": 512, "init": "normal_0.02"},
        "optimizer": {"name": "adamw", "schedule": {"peak_lr": 1e-3}},
        "data": {"train_manifest": "unused.json"},
        "training": {"seq_len": 256, "global_batch_size": 2, "target_tokens": 2 * 256 * 4, "precision": "bf16"},
    }
    trainer = Trainer(run_spec_from_mapping(raw), build_data=False)
    model = trainer.result.model
    prompts = torch.randint(0, 512, (3, 200), device="cuda", dtype=torch.int32)
    follow = torch.randint(0, 512, (3, 6), device="cuda", dtype=torch.int32)

    real_cache = generation.PagedKVCache

    class _NoNative(generation.PagedKVCache):
        def update_and_attend(self, layer, q, k, v, positions, window):
            B, T = positions.shape
            kp, vp = self._pages(self.k, layer), self._pages(self.v, layer)
            idx = positions.long()
            b_idx = torch.arange(B, device=q.device)[:, None].expand(B, T)
            kp[b_idx, idx // self.page_size, :, idx % self.page_size] = k.to(kp.dtype)
            vp[b_idx, idx // self.page_size, :, idx % self.page_size] = v.to(vp.dtype)
            end = int(positions.max().item()) + 1
            kpos = torch.arange(end, device=q.device)
            allowed = kpos[None, None, :] <= idx[:, :, None]
            return generation._masked_attention(q, self._rows(self.k, layer, end), self._rows(self.v, layer, end),
                                                allowed)

    def teacher_forced(cache_cls):
        monkeypatch.setattr(generation, "PagedKVCache", cache_cls)
        cache = generation.init_kv_cache(model, 3, 256)
        pos = torch.arange(200, device="cuda", dtype=torch.int32).expand(3, 200).contiguous()
        outs = []
        with torch.no_grad():
            outs.append(model.run_with_cache(prompts, pos, cache)[:, -1].float())
            cache.advance(pos)
            for t in range(follow.shape[1]):
                p1 = torch.full((3, 1), 200 + t, device="cuda", dtype=torch.int32)
                outs.append(model.run_with_cache(follow[:, t:t + 1], p1, cache)[:, -1].float())
                cache.advance(p1)
        return torch.stack(outs)

    model.eval()
    fast = teacher_forced(real_cache)
    native.check_status()
    slow = teacher_forced(_NoNative)
    lp_fast, lp_slow = torch.log_softmax(fast, -1), torch.log_softmax(slow, -1)
    assert (lp_fast - lp_slow).abs().max().item() < 5e-2, (lp_fast - lp_slow).abs().max().item()
    # and the sampling loop runs end to end on the native path
    monkeypatch.setattr(generation, "PagedKVCache", real_cache)
    res = generation.generate_tokens(model, prompts, max_new_tokens=8, temperature=1.0, top_k=50, seed=0)
    native.check_status()
    assert len(res.generated_ids) == 3 and all(len(g) == 8 for g in res.generated_ids)


def test_sampler_kernel_threshold_logprob_and_distribution():
    from research_b200.ops import native

    torch.manual_seed(0)
    B, V = 4, 50304
    logits = (torch.randn(B, V, device="cuda") * 2.0).bfloat16()
    # argmax
    tok, lp = native.sample_topk(logits, torch.rand(B, device="cuda"), 1.0, 1)
    assert torch.equal(tok, logits.float().argmax(-1)) and bool((lp == 0).all())
    # threshold with ties: kept set and log-probabilities against the PyTorch formulation
    for T, k in ((1.0, 50), (0.7, 8), (1.3, None)):
        scaled = logits.float() / T
        if k is not None:
            thr = torch.topk(scaled, k, dim=-1).values[:, -1:]
            scaled = torch.where(scaled >= thr, scaled, torch.full_like(scaled, float("-inf")))
        ref_logp = torch.log_softmax(scaled, -1)
        for trial in range(8):
            u = torch.rand(B, device="cuda")
            tok, lp = native.sample_topk(logits, u, T, k)
            chosen = ref_logp.gather(1, tok[:, None])[:, 0]
            assert bool(torch.isfinite(chosen).all()), "sampled a token outside the kept set"
            assert torch.allclose(lp, chosen, atol=2e-3, rtol=1e-3), (lp, chosen)
    # distribution: small vocabulary, many draws of one row
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0, 3.0, 0.5, -2.0, 1.5]], device="cuda").repeat(4096, 1)
    tok, _ = native.sample_topk(small, torch.rand(4096, device="cuda"), 1.0, 4)
    freq = torch.bincount(tok, minlength=8).float() / 4096
    kept = torch.tensor([2.0, 1.0, 3.0, 1.5])
    probs = torch.zeros(8)
    probs[[0, 1, 4, 7]] = torch.softmax(kept, 0)
    assert float((freq.cpu() - probs).abs().max()) < 0.03, (freq, probs)
    native.check_status()
