"""KV-cache generation: prefill, per-token decode, sampling.

Sampler semantics follow the reference (src/jaxtitan/infer/generation.py:225-242, 420-432): logits / temperature;
top-k keeps values >= the k-th largest (a threshold, so ties survive); ``top_k == 1`` is argmax; otherwise a
categorical draw; the log-probability of the chosen token under the filtered distribution is returned; ``top_p`` is
rejected.  The cache is paged: fixed-size pages per sequence, appended in place, and decode attention reads only
the pages in use (the reference attends over the whole padded cache every step, generation.py:302,
components/attention.py:213-218).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from research_b200.errors import ContractError
from research_b200.ops import functional as Fn


class PagedKVCache:
    """``[layers, pages, kv_heads, page_size, head_dim]`` K and V pools (head-major pages) + a page table."""

    def __init__(self, *, layers: int, batch: int, max_len: int, kv_heads: int, head_dim: int, page_size: int,
                 dtype: torch.dtype, device: torch.device):
        self.page_size = page_size
        self.pages_per_seq = (max_len + page_size - 1) // page_size
        self.max_len = self.pages_per_seq * page_size
        total_pages = batch * self.pages_per_seq
        shape = (layers, total_pages, kv_heads, page_size, head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.page_table = torch.arange(total_pages, device=device, dtype=torch.int32).view(batch, self.pages_per_seq)
        self.lengths = torch.zeros(batch, dtype=torch.int32, device=device)
        self.batch = batch

    def _pages(self, pool: torch.Tensor, layer: int) -> torch.Tensor:
        # with the identity page table, sequence b owns pages [b * pages_per_seq, (b + 1) * pages_per_seq)
        return pool[layer].view(self.batch, self.pages_per_seq, pool.shape[2], self.page_size, pool.shape[4])

    def _rows(self, pool: torch.Tensor, layer: int, end: int) -> torch.Tensor:
        """Dense ``[B, end, Hkv, D]`` copy of the first ``end`` rows (fallback paths only)."""

        pg = self._pages(pool, layer)
        return pg.permute(0, 1, 3, 2, 4).reshape(self.batch, self.max_len, pg.shape[2], pg.shape[4])[:, :end]

    def update_and_attend(self, layer: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                          positions: torch.Tensor, window: int | None) -> torch.Tensor:
        """Write k, v at ``positions`` ([B,T]) and attend q over everything written so far (causal)."""

        B, T = positions.shape
        kp, vp = self._pages(self.k, layer), self._pages(self.v, layer)
        native_ok = q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128)
        if T == 1 and native_ok:
            from research_b200.ops.decode import decode_attention_paged, kv_append_paged

            # the positions of a step are the same for every layer: the contiguous copy and the lengths are made by
            # the first layer and reused by the others (two launches per step instead of two per layer)
            step = getattr(self, "_step_positions", None)
            if layer == 0 or step is None or step[0] is not positions:
                pos = positions[:, 0].to(torch.int32).contiguous()
                step = self._step_positions = (positions, pos, pos + 1)
            _, pos, lengths = step
            kv_append_paged(k[:, 0], v[:, 0], kp, vp, pos)
            lo = None if window is None else (pos - (window - 1)).clamp_min(0).to(torch.int32)
            return decode_attention_paged(q[:, 0], kp, vp, lengths, lo)[:, None]
        idx = positions.long()
        from_zero = T > 1 and bool((positions == torch.arange(T, device=q.device, dtype=positions.dtype)).all())
        if from_zero:
            # a prompt written from row 0: whole pages are strided block copies, no index arithmetic per element
            ps = self.page_size
            full = T // ps
            if full:
                kp[:, :full].copy_(k[:, :full * ps].reshape(B, full, ps, *k.shape[2:]).permute(0, 1, 3, 2, 4))
                vp[:, :full].copy_(v[:, :full * ps].reshape(B, full, ps, *v.shape[2:]).permute(0, 1, 3, 2, 4))
            rest = T - full * ps
            if rest:
                kp[:, full, :, :rest].copy_(k[:, full * ps:].permute(0, 2, 1, 3))
                vp[:, full, :, :rest].copy_(v[:, full * ps:].permute(0, 2, 1, 3))
        else:
            b_idx = torch.arange(B, device=q.device)[:, None].expand(B, T)
            kp[b_idx, idx // self.page_size, :, idx % self.page_size] = k.to(kp.dtype)
            vp[b_idx, idx // self.page_size, :, idx % self.page_size] = v.to(vp.dtype)
        if from_zero and native_ok:
            # prefill from position 0: the flash kernel over the rows just computed
            from research_b200.ops import native

            lo = None
            if window is not None:
                lo = (positions - (window - 1)).clamp_min(0).to(torch.int32).contiguous()
            o, _ = native.attn_fwd(q.contiguous(), k.contiguous(), v.contiguous(), causal=True, lo=lo)
            return o.reshape(B, T, -1)
        end = int(positions.max().item()) + 1
        keys, vals = self._rows(self.k, layer, end), self._rows(self.v, layer, end)
        kpos = torch.arange(end, device=q.device)
        allowed = kpos[None, None, :] <= idx[:, :, None]
        if window is not None:
            allowed = allowed & (kpos[None, None, :] > idx[:, :, None] - window)
        return _masked_attention(q, keys, vals, allowed)

    def advance(self, positions: torch.Tensor) -> None:
        self.lengths = torch.maximum(self.lengths, (positions.max(dim=1).values + 1).to(torch.int32))


def _masked_attention(q, k, v, allowed):
    B, T, Hq, D = q.shape
    g = Hq // k.shape[2]
    qf = q.permute(0, 2, 1, 3).float()
    kf = k.permute(0, 2, 1, 3).repeat_interleave(g, dim=1).float()
    vf = v.permute(0, 2, 1, 3).repeat_interleave(g, dim=1).float()
    s = torch.einsum("bhqd,bhkd->bhqk", qf, kf) * (D ** -0.5)
    s = s.masked_fill(~allowed[:, None], float("-inf"))
    p = torch.softmax(s, dim=-1).to(q.dtype).float()
    return torch.einsum("bhqk,bhkd->bhqd", p, vf).permute(0, 2, 1, 3).to(q.dtype).reshape(B, T, Hq * D)


def init_kv_cache(model, batch: int, max_len: int, *, page_size: int = 128) -> PagedKVCache:
    spec = model.spec
    p = next(model.parameters())
    attn = model.layers[0].attn
    return PagedKVCache(layers=spec.num_layers, batch=batch, max_len=max_len, kv_heads=attn.hkv,
                        head_dim=spec.head_dim, page_size=page_size, dtype=p.dtype, device=p.device)


def sample_next_token(logits: torch.Tensor, *, temperature: float, top_k: int | None, top_p: float | None,
                      generator: torch.Generator | None):
    """logits [B, V] -> (token [B] int64, logprob [B] fp32)."""

    if top_p is not None:
        raise ContractError("generation.top_p is not supported at runtime")
    if temperature <= 0:
        raise ContractError(f"generation.temperature must be positive, got {temperature}")
    if top_k is not None and top_k <= 0:
        raise ContractError(f"generation.top_k must be positive, got {top_k}")
    if logits.is_cuda and logits.dim() == 2 and logits.dtype in (torch.bfloat16, torch.float32):
        # one kernel: threshold select, softmax mass, inverse-CDF draw from a uniform number of ``generator``
        from research_b200.ops import native

        u = torch.rand(logits.shape[0], device=logits.device, generator=generator)
        return native.sample_topk(logits if logits.stride(1) == 1 else logits.contiguous(), u, float(temperature), top_k)
    scaled = logits.float() / float(temperature)
    if top_k is not None:
        k = min(int(top_k), scaled.shape[-1])
        threshold = torch.topk(scaled, k, dim=-1).values[:, -1:]
        scaled = torch.where(scaled >= threshold, scaled, torch.full_like(scaled, float("-inf")))
    logp = torch.log_softmax(scaled, dim=-1)
    if top_k == 1:
        token = torch.argmax(scaled, dim=-1)
    else:
        token = torch.multinomial(torch.exp(logp), 1, generator=generator)[:, 0]
    return token, logp.gather(1, token[:, None])[:, 0]


class GraphedDecodeStep:
    """One decode step (embedding -> layers -> logits of the new token) captured in a CUDA graph.

    A decode step of a small batch is a few hundred short kernels, so its cost is launch latency, not work; the
    captured graph replays them with one launch.  Token and position live in static device buffers that are
    overwritten before each replay; sampling stays outside the graph.  Shapes are fixed at capture (batch size,
    cache capacity)."""

    def __init__(self, model, cache: PagedKVCache, first_token: torch.Tensor, first_position: int):
        B = first_token.shape[0]
        dev = first_token.device
        self.token = first_token.reshape(B, 1).to(torch.int32).clone()
        self.position = torch.full((B, 1), int(first_position), device=dev, dtype=torch.int32)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(2):  # warm-up with the real inputs: the cache writes are idempotent
                model.run_with_cache(self.token, self.position, cache, last_only=True)
        torch.cuda.current_stream(dev).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.logits = model.run_with_cache(self.token, self.position, cache, last_only=True)[:, -1]

    def __call__(self, token: torch.Tensor, position: int) -> torch.Tensor:
        self.token.copy_(token.reshape(-1, 1))
        self.position.fill_(int(position))
        self.graph.replay()
        return self.logits


def _graph_ok(model, device: torch.device) -> bool:
    # collectives of a tensor-parallel step stay outside a captured graph
    return (device.type == "cuda" and getattr(model, "compute_dtype", None) == torch.bfloat16
            and getattr(getattr(model, "ex", None), "tp_size", 1) == 1)


KVCache = PagedKVCache


@torch.no_grad()
def prefill(model, prompt_ids: torch.Tensor, cache: PagedKVCache) -> torch.Tensor:
    """Run the prompt ``[B, P]`` through the model, fill ``cache`` and return the logits of the last position
    ``[B, V]`` (reference: src/jaxtitan/infer/core.py ``prefill``)."""

    B, P = prompt_ids.shape
    device = next(model.parameters()).device
    positions = torch.arange(P, device=device, dtype=torch.int32).expand(B, P).contiguous()
    logits = model.run_with_cache(prompt_ids.to(device=device, dtype=torch.int32), positions, cache, last_only=True)
    cache.advance(positions)
    return logits[:, -1]


@torch.no_grad()
def decode_one(model, token: torch.Tensor, position: int, cache: PagedKVCache) -> torch.Tensor:
    """One decode step: ``token`` ``[B]`` at ``position`` -> next-token logits ``[B, V]``; the cache grows by one."""

    B = token.shape[0]
    device = next(model.parameters()).device
    pos = torch.full((B, 1), int(position), device=device, dtype=torch.int32)
    logits = model.run_with_cache(token.to(device=device, dtype=torch.int32)[:, None], pos, cache, last_only=True)
    cache.advance(pos)
    return logits[:, -1]


@dataclass
class GenerationResult:
    prompt_ids: list[list[int]]
    generated_ids: list[list[int]]
    full_ids: list[list[int]]
    logprobs: list[list[float]]


@torch.no_grad()
def generate_tokens(model, prompt_ids: torch.Tensor, *, max_new_tokens: int, temperature: float = 1.0,
                    top_k: int | None = None, top_p: float | None = None, seed: int = 0,
                    page_size: int = 128) -> GenerationResult:
    """prompt_ids: [B, P] (all prompts the same length).  Prefill once, then one decode step per new token."""

    if max_new_tokens <= 0:
        raise ContractError(f"generation.max_new_tokens must be positive, got {max_new_tokens}")
    B, P = prompt_ids.shape
    total = P + max_new_tokens
    if total > model.spec.max_seq_len:
        raise ContractError(f"prompt + max_new_tokens = {total} exceeds model.max_seq_len = {model.spec.max_seq_len}")
    device = next(model.parameters()).device
    prompt_ids = prompt_ids.to(device)
    was_training = model.training
    model.eval()
    cache = init_kv_cache(model, B, total, page_size=page_size)
    gen = torch.Generator(device=device).manual_seed(int(seed))
    positions = torch.arange(P, device=device, dtype=torch.int32).expand(B, P).contiguous()
    logits = model.run_with_cache(prompt_ids.to(torch.int32), positions, cache, last_only=True)[:, -1]
    cache.advance(positions)
    tokens, logprobs = [], []
    step = None
    for t in range(max_new_tokens):
        tok, lp = sample_next_token(logits, temperature=temperature, top_k=top_k, top_p=top_p, generator=gen)
        tokens.append(tok)
        logprobs.append(lp)
        if t + 1 == max_new_tokens:
            break
        if _graph_ok(model, device):
            if step is None:
                step = GraphedDecodeStep(model, cache, tok, P + t)
            logits = step(tok, P + t)
            continue
        pos = torch.full((B, 1), P + t, device=device, dtype=torch.int32)
        logits = model.run_with_cache(tok[:, None].to(torch.int32), pos, cache, last_only=True)[:, -1]
        cache.advance(pos)
    model.train(was_training)
    out = torch.stack(tokens, dim=1).cpu()
    lps = torch.stack(logprobs, dim=1).cpu()
    prompts = prompt_ids.cpu().tolist()
    generated = out.tolist()
    return GenerationResult(prompts, generated, [p + g for p, g in zip(prompts, generated)], lps.tolist())
