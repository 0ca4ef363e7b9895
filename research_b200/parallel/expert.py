"""Routed-expert dispatch and combine: sort assignments expert-major, (optionally) exchange rows between
expert-parallel ranks, run the grouped expert FFN, send results back, un-sort, weight and sum over top-k.

Three dispatchers, as in the reference (src/jaxtitan/models/execution.py:79-86, components/moe.py:198-316, 482-791):
``all_to_all`` (default: ragged exchange of exactly the routed rows), ``rdep_static`` (the same exchange over
the data axis) and ``psum`` (every rank applies its local experts to all tokens and the partial outputs are
summed - the simple reference path).  The transport here is ``torch.distributed`` all-to-all (NCCL on GPUs,
gloo on CPU); the fused peer-memory dispatch kernel replaces it on CUDA when enabled.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from research_b200.models.execution import all_reduce_sum


class _AllToAllRows(torch.autograd.Function):
    """Variable-split all-to-all over dim 0; backward is the reverse exchange."""

    @staticmethod
    def forward(ctx, x, send_splits, recv_splits, group):
        ctx.group, ctx.send, ctx.recv = group, send_splits, recv_splits
        out = torch.empty((sum(recv_splits),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x.contiguous(), recv_splits, send_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = torch.empty((sum(ctx.send),) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_to_all_single(out, g.contiguous(), ctx.send, ctx.recv, group=ctx.group)
        return out, None, None, None


def _local_dispatch(experts, x, expert_ids, weights, num_experts):
    T, k = expert_ids.shape
    flat_e = expert_ids.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    token_of = order // k
    rows = x.index_select(0, token_of)
    counts = torch.bincount(flat_e, minlength=num_experts)
    out_rows = experts(rows, counts)
    w = weights.reshape(-1).index_select(0, order).to(out_rows.dtype)
    y = torch.zeros_like(x)
    return y.index_add(0, token_of, out_rows * w[:, None])


def dispatch_and_combine(experts, x: torch.Tensor, expert_ids: torch.Tensor, weights: torch.Tensor, *,
                         num_experts: int, ex, plan=None) -> torch.Tensor:
    """x: [T,H]; expert_ids, weights: [T,k] (global expert ids).  Returns sum_k w * expert(x) as [T,H].
    ``plan`` is the native routing plan of these assignments when the CUDA kernels are in use."""

    ep = ex.ep_size
    if ep > 1 and plan is not None:
        from research_b200.parallel.expert_fused import dispatch_and_combine_fused

        return dispatch_and_combine_fused(experts, x, weights, plan)
    if ep == 1:
        if plan is not None:
            from research_b200.ops.grouped import routed_expert_ffn

            return routed_expert_ffn(x, weights, plan, experts.w_gate_up, experts.w_down)
        return _local_dispatch(experts, x, expert_ids, weights, num_experts)
    if ex.ep_axis_sharing == "dedicated_ep" and not ex.extras.get("_ep_sliced"):
        # With a dedicated ``ep`` axis everything outside the routed experts is replicated over it: split the
        # tokens over the axis for the dispatch (the reference slices the sequence inside its shard_map,
        # components/moe.py:538-696) and gather the results back.
        from research_b200.models.execution import all_gather_replicated, slice_dim

        T = x.shape[0]
        pad = (-T) % ep
        if pad:
            x = torch.cat([x, x.new_zeros(pad, x.shape[1])])
            expert_ids = torch.cat([expert_ids, expert_ids.new_zeros(pad, expert_ids.shape[1])])
            weights = torch.cat([weights, weights.new_zeros(pad, weights.shape[1])])
        ex.extras["_ep_sliced"] = True
        try:
            y = dispatch_and_combine(experts, slice_dim(x, ex.ep_group, 0),
                                     expert_ids.chunk(ep, dim=0)[ex.ep_rank].contiguous(),
                                     slice_dim(weights, ex.ep_group, 0), num_experts=num_experts, ex=ex)
        finally:
            ex.extras["_ep_sliced"] = False
        y = all_gather_replicated(y, ex.ep_group, 0)
        return y[:T] if pad else y
    group = ex.ep_group
    rank = ex.ep_rank
    e_local = num_experts // ep
    T, k = expert_ids.shape
    if ex.ep_dispatcher == "psum":
        # apply local experts to every token that picked one of them, sum partial outputs over the axis
        local = (expert_ids // e_local) == rank
        w_local = weights * local.to(weights.dtype)
        ids_local = torch.where(local, expert_ids - rank * e_local, torch.zeros_like(expert_ids))
        flat_e = ids_local.reshape(-1)
        keep = local.reshape(-1)
        sel = torch.nonzero(keep, as_tuple=False)[:, 0]
        order = sel[torch.argsort(flat_e[sel], stable=True)]
        token_of = order // k
        rows = x.index_select(0, token_of)
        counts = torch.bincount(flat_e[order], minlength=e_local)
        out_rows = experts(rows, counts)
        w = w_local.reshape(-1).index_select(0, order).to(out_rows.dtype)
        y = torch.zeros_like(x).index_add(0, token_of, out_rows * w[:, None])
        return all_reduce_sum(y, group)
    # all_to_all / rdep_static: expert-major sort, ragged exchange, grouped FFN, reverse exchange
    flat_e = expert_ids.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    token_of = order // k
    rows = x.index_select(0, token_of)
    counts_global = torch.bincount(flat_e, minlength=num_experts)              # rows I send, per global expert
    recv_counts = torch.empty(ep * e_local, dtype=counts_global.dtype, device=x.device)
    dist.all_to_all_single(recv_counts, counts_global, group=group)            # [src_rank, local expert]
    send_splits = counts_global.view(ep, e_local).sum(dim=1).tolist()
    recv_matrix = recv_counts.view(ep, e_local)
    recv_splits = recv_matrix.sum(dim=1).tolist()
    recv_rows = _AllToAllRows.apply(rows, send_splits, recv_splits, group)     # grouped by source rank
    # regroup received rows expert-major: (src, expert) blocks -> (expert, src)
    blocks = recv_matrix.reshape(-1)
    block_expert = torch.arange(e_local, device=x.device).repeat(ep)
    row_expert = torch.repeat_interleave(block_expert, blocks)
    perm = torch.argsort(row_expert, stable=True)
    out_sorted = experts(recv_rows.index_select(0, perm), recv_matrix.sum(dim=0))
    out_rows = torch.zeros_like(out_sorted).index_copy(0, perm, out_sorted)
    back = _AllToAllRows.apply(out_rows, recv_splits, send_splits, group)
    w = weights.reshape(-1).index_select(0, order).to(back.dtype)
    return torch.zeros_like(x).index_add(0, token_of, back * w[:, None])
