"""Context-parallel attention: the sequence is split over the ``cp`` axis, zig-zag (rank ``r`` holds chunks ``r``
and ``2 cp - 1 - r`` of ``2 cp``) so that causal work is balanced, or contiguously when the length does not divide.

The reference shards activations on the sequence axis and lets XLA all-gather K/V around a plain global
einsum (src/jaxtitan/models/execution.py:227-240, mesh/sharding.py:165-167).  Here every rank normalises and
rotates its own q/k chunk (positions are global), K and V chunks are exchanged over the ``cp`` group, and the local
queries attend to the keys of their own and all earlier chunks with the flash-attention kernel's query-offset
form, so logits never materialise and only ``(r + 1) / cp`` of the keys are visited by rank ``r``.

Transport: ``all_gather`` over the cp group (NCCL on GPUs, gloo on CPU).  Backward sends every rank's
contribution to dK/dV of the chunks it attended to back to their owners with a reduce-scatter.
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
