"""Execution policy of a model replica: which process groups split activations and how.

One process drives one GPU; the named mesh axes are ``torch.distributed`` groups (see
:mod:`research_b200.parallel.mesh`).  This object carries the groups a model needs and implements the
activation-side collectives as differentiable functions:

* tensor parallel with Megatron-style sequence parallelism (reference: models/execution.py:183-250): the residual
  stream is ``[B, S/tp, H]`` between blocks, all-gathered along S before column-parallel projections and
  reduce-scattered after row-parallel ones; the lm_head is vocab-parallel;
* context parallel: the sequence is split across ``cp`` ranks for every per-token op and attention sees the
  keys/values of all earlier ranks (reference shards and lets XLA gather: models/execution.py:227-240);
* expert parallel: policy fields consumed by :mod:`research_b200.models.moe`.

The collectives here are the NCCL (or gloo, on CPU) baseline; fused compute+collective kernels replace them
where ``fused`` is enabled and the tensors are CUDA bf16.
"""

from __future__ import annotations

import os
from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.distributed as dist

from research_b200.ops import functional as Fn
from research_b200.ops import native

EP_DISPATCHERS = ("all_to_all", "rdep_static", "psum")


def _world(group) -> int:
    return 1 if group is None else dist.get_world_size(group)


def _rank(group) -> int:
    return 0 if group is None else dist.get_rank(group)


class _AllGatherDim(torch.autograd.Function):
    """Forward: all-gather along ``dim``; backward: reduce-scatter (sum) along ``dim``."""

    @staticmethod
    def forward(ctx, x, group, dim):
        n = dist.get_world_size(group)
        ctx.group, ctx.dim, ctx.n = group, dim, n
        xt = x.movedim(dim, 0).contiguous()
        out = torch.empty((n * xt.shape[0],) + tuple(xt.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, xt, group=group)
        return out.movedim(0, dim)

    @staticmethod
    def backward(ctx, g):
        gt = g.movedim(ctx.dim, 0).contiguous()
        out = torch.empty((gt.shape[0] // ctx.n,) + tuple(gt.shape[1:]), dtype=g.dtype, device=g.device)
        _reduce_scatter(out, gt, ctx.group)
        return out.movedim(0, ctx.dim), None, None


class _ReduceScatterDim(torch.autograd.Function):
    """Forward: reduce-scatter (sum) along ``dim``; backward: all-gather along ``dim``."""

    @staticmethod
    def forward(ctx, x, group, dim):
        n = dist.get_world_size(group)
        ctx.group, ctx.dim, ctx.n = group, dim, n
        xt = x.movedim(dim, 0).contiguous()
        out = torch.empty((xt.shape[0] // n,) + tuple(xt.shape[1:]), dtype=x.dtype, device=x.device)
        _reduce_scatter(out, xt, group)
        return out.movedim(0, dim)

    @staticmethod
    def backward(ctx, g):
        gt = g.movedim(ctx.dim, 0).contiguous()
        out = torch.empty((ctx.n * gt.shape[0],) + tuple(gt.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(out, gt, group=ctx.group)
        return out.movedim(0, ctx.dim), None, None


def _reduce_scatter(out: torch.Tensor, inp: torch.Tensor, group) -> None:
    if inp.is_cuda:
        dist.reduce_scatter_tensor(out, inp, group=group)
    else:  # gloo has no reduce_scatter: all-reduce then slice
        tmp = inp.clone()
        dist.all_reduce(tmp, group=group)
        n, r = dist.get_world_size(group), dist.get_rank(group)
        out.copy_(tmp.chunk(n, dim=0)[r])


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        out = x.clone()
        dist.all_reduce(out, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        return g, None


class _AllReduceSumSummedObjectives(torch.autograd.Function):
    """All-reduce forward and backward: for a group whose ranks each add an objective built on the sum to the total
    (context-parallel ranks - their gradients are added up), so a rank's input reaches every rank's objective."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        out = x.clone()
        dist.all_reduce(out, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _CopyToGroup(torch.autograd.Function):
    """Identity forward, all-reduce backward (input replicated, consumers hold partial gradients)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _SliceDim(torch.autograd.Function):
    """Forward: keep this rank's chunk along ``dim``; backward: all-gather the chunk gradients."""

    @staticmethod
    def forward(ctx, x, group, dim):
        n, r = dist.get_world_size(group), dist.get_rank(group)
        ctx.group, ctx.dim = group, dim
        return x.chunk(n, dim=dim)[r].contiguous()

    @staticmethod
    def backward(ctx, g):
        return _AllGatherDim.apply(g, ctx.group, ctx.dim), None, None


class _SliceDimLocal(torch.autograd.Function):
    """Forward: keep this rank's chunk along ``dim``; backward: that chunk's gradient, zeros elsewhere.

    For replicated inputs whose parameter gradients are summed over the group afterwards (the embedding in front
    of a sequence-parallel region): every rank contributes only the tokens it owns."""

    @staticmethod
    def forward(ctx, x, group, dim):
        n, r = dist.get_world_size(group), dist.get_rank(group)
        ctx.n, ctx.r, ctx.dim = n, r, dim
        return x.chunk(n, dim=dim)[r].contiguous()

    @staticmethod
    def backward(ctx, g):
        shape = list(g.shape)
        shape[ctx.dim] *= ctx.n
        full = g.new_zeros(shape)
        full.narrow(ctx.dim, ctx.r * g.shape[ctx.dim], g.shape[ctx.dim]).copy_(g)
        return full, None, None


class _AllGatherReplicated(torch.autograd.Function):
    """Forward: all-gather along ``dim``; backward: this rank's slice of the gradient, without a reduction.

    For results that feed a computation replicated over the group: every rank holds the same gradient of the
    gathered tensor, so summing it would count the downstream loss once per rank."""

    @staticmethod
    def forward(ctx, x, group, dim):
        n, r = dist.get_world_size(group), dist.get_rank(group)
        ctx.n, ctx.r, ctx.dim = n, r, dim
        xt = x.movedim(dim, 0).contiguous()
        out = torch.empty((n * xt.shape[0],) + tuple(xt.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, xt, group=group)
        return out.movedim(0, dim)

    @staticmethod
    def backward(ctx, g):
        return g.chunk(ctx.n, dim=ctx.dim)[ctx.r].contiguous(), None, None


def all_gather_replicated(x, group, dim):
    return x if _world(group) == 1 else _AllGatherReplicated.apply(x, group, dim)


def slice_dim_local(x, group, dim):
    return x if _world(group) == 1 else _SliceDimLocal.apply(x, group, dim)


def all_gather_dim(x, group, dim):
    return x if _world(group) == 1 else _AllGatherDim.apply(x, group, dim)


def reduce_scatter_dim(x, group, dim):
    return x if _world(group) == 1 else _ReduceScatterDim.apply(x, group, dim)


def all_reduce_sum(x, group):
    return x if _world(group) == 1 else _AllReduceSum.apply(x, group)


def all_reduce_sum_summed_objectives(x, group):
    return x if _world(group) == 1 else _AllReduceSumSummedObjectives.apply(x, group)


def copy_to_group(x, group):
    return x if _world(group) == 1 else _CopyToGroup.apply(x, group)


def slice_dim(x, group, dim):
    return x if _world(group) == 1 else _SliceDim.apply(x, group, dim)


@dataclass
class ExecutionContext:
    """Groups and switches a model forward needs.  The default is a single device with nothing split."""

    tp_group: Any = None
    cp_group: Any = None
    ep_group: Any = None
    expert_fsdp_group: Any = None
    sequence_parallel: bool = True
    ep_dispatcher: str = "all_to_all"
    ep_axis_name: str | None = None
    ep_axis_sharing: str | None = None
    cp_attention: str = "gather"            # context-parallel attention: K/V all-gather or Ulysses all-to-all
    fused: bool = True                      # use fused compute+collective kernels where available
    vocab_parallel: bool = False            # lm_head split over the vocabulary across the tensor-parallel group
    extras: dict[str, Any] = field(default_factory=dict)

    # ---- sizes -----------------------------------------------------------------------------------
    @property
    def tp_size(self) -> int:
        return _world(self.tp_group)

    @property
    def tp_rank(self) -> int:
        return _rank(self.tp_group)

    @property
    def cp_size(self) -> int:
        return _world(self.cp_group)

    @property
    def cp_rank(self) -> int:
        return _rank(self.cp_group)

    @property
    def ep_size(self) -> int:
        return _world(self.ep_group)

    @property
    def ep_rank(self) -> int:
        return _rank(self.ep_group)

    @property
    def efsdp_size(self) -> int:
        """Ranks that split the routed experts' intermediate dimension (the ``expert_fsdp`` axis)."""

        return _world(self.expert_fsdp_group)

    @property
    def efsdp_rank(self) -> int:
        return _rank(self.expert_fsdp_group)

    @property
    def sp(self) -> bool:
        return self.tp_size > 1 and self.sequence_parallel and self.cp_size == 1

    @contextmanager
    def replicated_activations(self):
        """Inside: every tensor-parallel rank holds the whole activations (no sequence-parallel shards), so a
        column-parallel projection reads its input as it is and a row-parallel one all-reduces its output.  This
        is how a few tokens at a time are run with a KV cache: a decode step has one row, nothing to split."""

        before = self.sequence_parallel
        self.sequence_parallel = False
        try:
            yield self
        finally:
            self.sequence_parallel = before

    # ---- tensor / sequence parallel activations ------------------------------------------------------
    def scatter_sequence(self, x: torch.Tensor) -> torch.Tensor:
        """Replicated ``[B,S,H]`` -> this rank's ``[B,S/tp,H]`` (start of the sequence-parallel region)."""

        return slice_dim_local(x, self.tp_group, 1) if self.sp else x

    def gather_sequence(self, x: torch.Tensor) -> torch.Tensor:
        """Before a column-parallel projection: SP shard -> full sequence (or mark the replicated input)."""

        if self.tp_size == 1:
            return x
        if self.sp:
            return all_gather_dim(x, self.tp_group, 1)
        return copy_to_group(x, self.tp_group)

    def reduce_scatter_sequence(self, x: torch.Tensor) -> torch.Tensor:
        """After a row-parallel projection: sum the partial outputs (and go back to the SP shard)."""

        if self.tp_size == 1:
            return x
        if self.sp:
            return reduce_scatter_dim(x, self.tp_group, 1)
        return all_reduce_sum(x, self.tp_group)

    # ---- fused tensor-parallel linears ----------------------------------------------------------------
    def _fusion_for(self, x: torch.Tensor, rows_local: int, width: int):
        """The fused-GEMM workspace of the tp group, or None when the NCCL formulation must run.

        Fused kernels need CUDA bf16 activations, sequence parallelism, shards in whole 128-row blocks and
        64-column multiples; the workspace is (re)built collectively the first time a larger shard shows up."""

        if not (self.fused and self.sp and x.is_cuda and x.dtype == torch.bfloat16 and Fn.use_native(x)):
            return None
        if os.environ.get("RESEARCH_B200_PEER_COLLECTIVES", "1") == "0" or self.tp_size > 8:
            return None
        if native.deterministic():      # the scatter epilogue reduce-adds into the owner in arrival order
            return None
        if rows_local % 128 or width % 64:
            return None
        need = x.shape[0] * rows_local * width
        if self.extras.get("tp_fusion_failed"):
            return None
        ws = self.extras.get("tp_fusion")
        if ws is None or ws.stage.numel() < need:
            from research_b200.parallel.symmetric import build_collectively
            from research_b200.parallel.tensor_fused import TensorParallelFusion

            ws = build_collectively(
                self.tp_group,
                lambda: TensorParallelFusion(self.tp_group, max_shard_elems=need, max_out_elems=need, device=x.device),
                "fused tensor-parallel workspace")
            self.extras["tp_fusion"] = ws
            if ws is None:
                self.extras["tp_fusion_failed"] = True
        return ws

    def column_linear(self, x: torch.Tensor, p: torch.Tensor) -> torch.Tensor:
        """Column-parallel ``y = gather_seq(x) W^T`` for a sequence-parallel shard ``[B, S/tp, H]``."""

        if self.tp_size > 1 and x.dim() == 3 and p.shape[0] % 64 == 0:
            ws = self._fusion_for(x, x.shape[1], max(x.shape[2], 64))
            if ws is not None:
                from research_b200.parallel.tensor_fused import column_linear

                return column_linear(x.contiguous(), p, ws)
        return Fn.linear(self.gather_sequence(x), p)

    def row_linear(self, h: torch.Tensor, p: torch.Tensor) -> torch.Tensor:
        """Row-parallel ``y = reduce_scatter_seq(h W^T)`` for ``h`` ``[B, S, K/tp]``."""

        if self.tp_size > 1 and h.dim() == 3 and h.shape[1] % self.tp_size == 0 and h.shape[2] % 64 == 0:
            ws = self._fusion_for(h, h.shape[1] // self.tp_size, p.shape[0])
            if ws is not None:
                from research_b200.parallel.tensor_fused import row_linear

                return row_linear(h, p, ws)
        return self.reduce_scatter_sequence(Fn.linear(h, p))

    def gather_vocab(self, logits: torch.Tensor) -> torch.Tensor:
        return all_gather_dim(logits, self.tp_group, logits.dim() - 1) if self.tp_size > 1 else logits

    # ---- attention (local, or context parallel) ------------------------------------------------------
    def attention(self, qkv, wq, wk, positions, *, B, S, hq, hkv, D, eps, theta, rope, lo, hi, chunks=()):
        if self.cp_size == 1:
            return Fn.attention_block(qkv, wq, wk, positions, B=B, S=S, hq=hq, hkv=hkv, D=D, eps=eps, theta=theta,
                                      rope=rope, causal=True, lo=lo, hi=hi)
        from research_b200.parallel.context import context_parallel_attention, ulysses_attention

        if self.cp_attention == "ulysses":
            return ulysses_attention(self, qkv, wq, wk, positions, B=B, S=S, hq=hq, hkv=hkv, D=D, eps=eps,
                                     theta=theta, rope=rope, lo=lo)
        return context_parallel_attention(self, qkv, wq, wk, positions, B=B, S=S, hq=hq, hkv=hkv, D=D, eps=eps,
                                          theta=theta, rope=rope, lo=lo, chunks=chunks)
