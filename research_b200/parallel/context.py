"""Context-parallel attention: the sequence is split over the ``cp`` axis, zig-zag (rank ``r`` holds chunks ``r``
and ``2 cp - 1 - r`` of ``2 cp``) so that causal work is balanced, or contiguously when the length does not divide.

The reference shards activations on the sequence axis and lets XLA all-gather K/V around a plain global
einsum (src/jaxtitan/models/execution.py:227-240, mesh/sharding.py:165-167).  Here every rank normalises and
rotates its own q/k chunk (positions are global), K and V chunks are exchanged over the ``cp`` group, and the local
queries attend to the keys of their own and all earlier chunks with the flash-attention kernel's query-offset
form, so logits never materialise and only ``(r + 1) / cp`` of the keys are visited by rank ``r``.

Transport on GPUs: the exchange happens inside the attention kernels (:mod:`research_b200.parallel.ring_attention`:
transfer CTAs of the attention launch pull K/V blocks over NVLink while the other CTAs attend; dK/dV tiles are
reduce-added into their owners' buffers from the backward kernel).  Fallback, CPU path and test oracle:
``all_gather`` over the cp group (NCCL on GPUs, gloo on CPU) followed by the kernel, with a reduce-scatter of
dK/dV in backward.

``parallelism.context_attention = "ulysses"`` selects the other classic form (:func:`ulysses_attention`): an
all-to-all turns the sequence split into a head split, every rank runs ordinary causal flash attention over the
whole sequence for ``heads / cp`` heads, and a second all-to-all turns the result back.  It moves
``(hq + 2 hkv) / cp`` head-slices per token instead of gathering all K/V, and its attention call is the plain
single-device kernel.  (The reference ships this only as a vendored transport kernel:
third_party/ThunderKittens/kernels/parallel/ulysses_attn/ulysses_attn.cu.)
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from research_b200.models.execution import _reduce_scatter
from research_b200.ops import functional as Fn
from research_b200.ops import native


class _GatherKV(torch.autograd.Function):
    """[B, S_local, H, D] -> [B, cp * S_local, H, D]; backward reduce-scatters (sums) the gradient chunks."""

    @staticmethod
    def forward(ctx, x, group):
        n = dist.get_world_size(group)
        ctx.group, ctx.n = group, n
        xt = x.transpose(0, 1).contiguous()                       # [S_local, B, H, D]
        out = torch.empty((n * xt.shape[0],) + tuple(xt.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, xt, group=group)
        return out.transpose(0, 1)

    @staticmethod
    def backward(ctx, g):
        gt = g.transpose(0, 1).contiguous()
        out = torch.empty((gt.shape[0] // ctx.n,) + tuple(gt.shape[1:]), dtype=g.dtype, device=g.device)
        _reduce_scatter(out, gt, ctx.group)
        return out.transpose(0, 1), None


class _OffsetAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, lo, q_offset, scale):
        o, lse = native.attn_fwd(q, k, v, causal=True, lo=lo, scale=scale, q_offset=q_offset)
        hi = None if lo is None else native.kv_visibility_upper_bound(lo, k.shape[1], q_offset)
        ctx.save_for_backward(q, k, v, o, lse, lo, hi)
        ctx.cfg = (q_offset, scale)
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse, lo, hi = ctx.saved_tensors
        q_offset, scale = ctx.cfg
        dq, dk, dv = native.attn_bwd(q, k, v, o, d_o.contiguous(), lse, causal=True, lo=lo, hi=hi, scale=scale,
                                     q_offset=q_offset)
        return dq, dk, dv, None, None, None


def context_parallel_attention(ex, qkv: torch.Tensor, wq, wk, positions: torch.Tensor, *, B: int, S: int, hq: int,
                               hkv: int, D: int, eps: float, theta: float, rope: bool, lo: torch.Tensor | None,
                               chunks: tuple[tuple[int, int], ...] = ()) -> torch.Tensor:
    """qkv: this rank's ``[B*S_local, (hq + 2 hkv) D]`` projection; positions: *global* positions ``[B*S_local]``;
    ``lo``: per-row first visible global kv position or None; ``chunks``: the ``(first global position, length)``
    runs that make up the local rows (one run for a contiguous split, two for the zig-zag split).
    Returns ``[B, S_local, hq * D]``."""

    cp, rank, group = ex.cp_size, ex.cp_rank, ex.cp_group
    if not chunks:
        chunks = ((rank * S, S),)
    qk = Fn.qk_norm_rope(qkv, wq, wk, positions.to(torch.int32), hq, hkv, D, eps, theta, rope)
    q4 = qk[:, : hq * D].reshape(B, S, hq, D)
    k4 = qk[:, hq * D:].reshape(B, S, hkv, D)
    v4 = qkv[:, (hq + hkv) * D:].reshape(B, S, hkv, D)
    zigzag = S % 2 == 0   # the rule of steps.train.context_positions: an even local length means the zig-zag split
    from research_b200.parallel import ring_attention as ring

    if Fn.use_native(qkv) and ring.ring_available(ex, q4, S, hkv, D, chunks):
        ws = ring.workspace_for(group, B, S, hkv, D, zigzag, q4.device)
        if ws is not None:
            # the K/V exchange happens inside the attention launches (no all-gather, no reduce-scatter)
            return ring.ring_attention(q4, k4, v4, lo, ws, chunks, D ** -0.5).reshape(B, S, hq * D)
    k_all = _in_sequence_order(_GatherKV.apply(k4, group), cp, S, zigzag)
    v_all = _in_sequence_order(_GatherKV.apply(v4, group), cp, S, zigzag)
    scale = D ** -0.5
    outs = []
    row = 0
    for first, length in chunks:
        end = first + length                                   # this run sees the keys of positions [0, end)
        q_c = q4[:, row:row + length]
        lo_c = None if lo is None else lo[:, row:row + length].contiguous()
        k_c, v_c = k_all[:, :end], v_all[:, :end]
        if Fn.use_native(qkv) and D in (64, 128) and length % 128 == 0 and first % 128 == 0:
            outs.append(_OffsetAttentionFn.apply(q_c.contiguous(), k_c.contiguous(), v_c.contiguous(), lo_c, first,
                                                 scale))
        else:
            outs.append(Fn.attention_reference(q_c, k_c, v_c, causal=True, lo=lo_c, scale=scale))
        row += length
    o = outs[0] if len(outs) == 1 else torch.cat(outs, dim=1)
    return o.reshape(B, S, hq * D)


def _in_sequence_order(gathered: torch.Tensor, cp: int, s_local: int, zigzag: bool) -> torch.Tensor:
    """The all-gather returns rank-major rows; with the zig-zag split rank ``r`` holds chunks ``r`` and
    ``2 cp - 1 - r``, so the second halves come back in reverse rank order."""

    if not zigzag:
        return gathered
    B = gathered.shape[0]
    c = s_local // 2
    g = gathered.reshape(B, cp, 2, c, *gathered.shape[2:])
    first, second = g[:, :, 0], g[:, :, 1].flip(1)
    return torch.cat([first, second], dim=1).reshape(B, 2 * cp * c, *gathered.shape[2:])


def _order_index(cp: int, s_local: int, zigzag: bool, device) -> torch.Tensor | None:
    """Row index that turns rank-major gathered rows into sequence order (None when they already are)."""

    if not zigzag:
        return None
    c = s_local // 2
    idx = torch.arange(cp * s_local, device=device).view(cp, 2, c)
    return torch.cat([idx[:, 0], idx[:, 1].flip(0)], dim=0).reshape(-1)


class _SeqToHeads(torch.autograd.Function):
    """``[B, S_local, H, D]`` (all heads, my rows) -> ``[B, cp * S_local, H / cp, D]`` (my heads, all rows in
    sequence order); the backward is the opposite exchange."""

    @staticmethod
    def forward(ctx, x, group, order):
        cp = dist.get_world_size(group)
        B, S, H, D = x.shape
        ctx.group, ctx.order, ctx.cp = group, order, cp
        send = x.view(B, S, cp, H // cp, D).permute(2, 0, 1, 3, 4).contiguous()     # [dst, B, S, h, D]
        recv = torch.empty_like(send)                                                # [src, B, S, h, D]
        dist.all_to_all_single(recv, send, group=group)
        out = recv.permute(1, 0, 2, 3, 4).reshape(B, cp * S, H // cp, D)
        return out if order is None else out.index_select(1, order)

    @staticmethod
    def backward(ctx, g):
        return _heads_to_seq(g, ctx.group, ctx.order, ctx.cp), None, None


class _HeadsToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, order):
        cp = dist.get_world_size(group)
        ctx.group, ctx.order, ctx.cp = group, order, cp
        return _heads_to_seq(x, group, order, cp)

    @staticmethod
    def backward(ctx, g):
        return _SeqToHeads.forward(ctx, g.contiguous(), ctx.group, ctx.order), None, None


def _heads_to_seq(x: torch.Tensor, group, order, cp: int) -> torch.Tensor:
    """``[B, cp * S_local, h, D]`` in sequence order -> ``[B, S_local, cp * h, D]`` (my rows, all heads)."""

    B, S_full, h, D = x.shape
    S = S_full // cp
    if order is not None:
        x = torch.empty_like(x).index_copy_(1, order, x)         # back to rank-major rows
    send = x.reshape(B, cp, S, h, D).permute(1, 0, 2, 3, 4).contiguous()              # [dst, B, S, h, D]
    recv = torch.empty_like(send)                                                     # [head group, B, S, h, D]
    dist.all_to_all_single(recv, send, group=group)
    return recv.permute(1, 2, 0, 3, 4).reshape(B, S, cp * h, D)


def ulysses_attention(ex, qkv: torch.Tensor, wq, wk, positions: torch.Tensor, *, B: int, S: int, hq: int, hkv: int,
                      D: int, eps: float, theta: float, rope: bool, lo: torch.Tensor | None) -> torch.Tensor:
    """Same contract as :func:`context_parallel_attention`; ``lo`` holds global kv positions for the local rows."""

    cp, group = ex.cp_size, ex.cp_group
    if hq % cp or hkv % cp:
        raise ValueError(f"ulysses attention needs heads ({hq}) and kv heads ({hkv}) divisible by cp ({cp})")
    qk = Fn.qk_norm_rope(qkv, wq, wk, positions.to(torch.int32), hq, hkv, D, eps, theta, rope)
    q4 = qk[:, : hq * D].reshape(B, S, hq, D)
    k4 = qk[:, hq * D:].reshape(B, S, hkv, D)
    v4 = qkv[:, (hq + hkv) * D:].reshape(B, S, hkv, D)
    zigzag = S % 2 == 0
    order = _order_index(cp, S, zigzag, qkv.device)
    q_all = _SeqToHeads.apply(q4.contiguous(), group, order)
    k_all = _SeqToHeads.apply(k4.contiguous(), group, order)
    v_all = _SeqToHeads.apply(v4.contiguous(), group, order)
    lo_all = None
    if lo is not None:
        parts = torch.empty(cp * B, S, dtype=lo.dtype, device=lo.device)
        dist.all_gather_into_tensor(parts, lo.contiguous(), group=group)
        lo_all = parts.view(cp, B, S).permute(1, 0, 2).reshape(B, cp * S)
        if order is not None:
            lo_all = lo_all.index_select(1, order)
        lo_all = lo_all.contiguous()
    o = Fn.attention(q_all, k_all, v_all, causal=True, lo=lo_all, scale=D ** -0.5)
    return _HeadsToSeq.apply(o.contiguous(), group, order).reshape(B, S, hq * D)
