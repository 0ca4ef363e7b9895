"""Context-parallel attention: the sequence is split into contiguous chunks over the ``cp`` axis.

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
                               hkv: int, D: int, eps: float, theta: float, rope: bool,
                               lo: torch.Tensor | None) -> torch.Tensor:
    """qkv: this rank's ``[B*S_local, (hq + 2 hkv) D]`` projection; positions: local indices ``[B*S_local]``;
    ``lo``: per-row first visible *global* kv position or None.  Returns ``[B, S_local, hq * D]``."""

    cp, rank, group = ex.cp_size, ex.cp_rank, ex.cp_group
    q_offset = rank * S
    global_pos = (positions + q_offset).to(torch.int32)
    qk = Fn.qk_norm_rope(qkv, wq, wk, global_pos, hq, hkv, D, eps, theta, rope)
    q4 = qk[:, : hq * D].reshape(B, S, hq, D)
    k4 = qk[:, hq * D:].reshape(B, S, hkv, D)
    v4 = qkv[:, (hq + hkv) * D:].reshape(B, S, hkv, D)
    k_all = _GatherKV.apply(k4, group)[:, : (rank + 1) * S]
    v_all = _GatherKV.apply(v4, group)[:, : (rank + 1) * S]
    scale = D ** -0.5
    if Fn.use_native(qkv) and D in (64, 128) and S % 128 == 0:
        o = _OffsetAttentionFn.apply(q4.contiguous(), k_all.contiguous(), v_all.contiguous(), lo, q_offset, scale)
    else:
        o = Fn.attention_reference(q4, k_all, v_all, causal=True, lo=lo, scale=scale)
    return o.reshape(B, S, hq * D)
