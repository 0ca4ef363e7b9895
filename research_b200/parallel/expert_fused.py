"""Expert-parallel dispatch and combine over peer memory (no sort, no NCCL all-to-all of rows).

Per MoE layer, with the routed experts split over the ``ep`` ranks of one node:

1. every rank ranks its own (token, choice) assignments per global expert (``ops/csrc/moe.cu``) and the per-expert
   counts are all-gathered (a ``[ranks, experts]`` int32 table, the only NCCL call);
2. from that table every rank derives, identically, where each sender's rows of each expert start inside the
   owner's expert-major, 128-row padded buffer;
3. **dispatch**: the sender's kernel stores each kept row straight into the owner's arena buffer over NVLink;
4. the owner runs the grouped tcgen05 expert FFN on its buffer;
5. **combine**: the sender's kernel loads its rows of the expert outputs from the owners' arena buffers, weights
   and sums them per token.

Backward mirrors it (push of weighted output gradients, pull of input gradients).  Stream-ordered peer barriers
(bounded waits) separate the phases.  The path needs a capacity factor, which bounds the owner's buffer.
The NCCL formulation in :mod:`research_b200.parallel.expert` is the fallback and the test oracle.

Reference: src/jaxtitan/models/components/moe.py:538-696 (ragged all-to-all dispatcher), 606-662 (metadata and
payload exchanges).
"""

from __future__ import annotations

import ctypes
from types import SimpleNamespace

import torch
import torch.distributed as dist

from research_b200.errors import KernelError
from research_b200.ops import functional as Fn
from research_b200.ops import native
from research_b200.ops.grouped import TILE, _GroupedLinearFn, _moe_lib
from research_b200.parallel.symmetric import SymmetricArena

BARRIER_CHANNEL = 5


class ExpertParallelWorkspace:
    """Two row buffers per rank in a symmetric arena: one that peers write (dispatch, backward of combine) and one
    that peers read (combine, backward of dispatch)."""

    def __init__(self, group, rows: int, hidden: int, device: torch.device):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.rows, self.hidden = rows, hidden
        self.arena = SymmetricArena(group, 2 * rows * hidden * 2 + 8192, device=device, tag="ep")
        self.inbox, self.inbox_off = self.arena.carve(rows * hidden, torch.bfloat16)
        self.outbox, self.outbox_off = self.arena.carve(rows * hidden, torch.bfloat16)
        self.inbox = self.inbox.view(rows, hidden)
        self.outbox = self.outbox.view(rows, hidden)

    def ptrs(self, offset: int):
        arr = (ctypes.c_void_p * self.world)()
        for r in range(self.world):
            arr[r] = self.arena.peer_ptr(r, offset)
        return arr

    def barrier(self) -> None:
        self.arena.barrier(BARRIER_CHANNEL)


def workspace_for(ex, rows: int, hidden: int, device: torch.device) -> ExpertParallelWorkspace | None:
    """The arena workspace of the ep group, built (collectively) on first use; None when peer memory is refused."""

    if ex.extras.get("ep_workspace_failed"):
        return None
    ws = ex.extras.get("ep_workspace")
    if ws is None or ws.rows < rows or ws.hidden != hidden:
        from research_b200.parallel.symmetric import build_collectively

        ws = build_collectively(ex.ep_group, lambda: ExpertParallelWorkspace(ex.ep_group, rows, hidden, device),
                                "expert-parallel workspace")
        ex.extras["ep_workspace"] = ws
        if ws is None:
            ex.extras["ep_workspace_failed"] = True
    return ws


class ExpertParallelPlan:
    """Routing plan of one layer under expert parallelism (device tensors only, no host synchronisation)."""

    def __init__(self, expert_ids: torch.Tensor, num_experts: int, capacity: int, ex, hidden: int):
        lib = _moe_lib()
        dev = expert_ids.device
        R, rank = ex.ep_size, ex.ep_rank
        E = num_experts
        el = E // R
        self.T, self.k = expert_ids.shape
        A = self.T * self.k
        ids = expert_ids.reshape(-1).to(torch.int32).contiguous()
        i32 = dict(dtype=torch.int32, device=dev)
        st = native._stream()
        hist = torch.empty(lib.b200_moe_chunks(A) * E, **i32)
        self.pos = torch.empty(A, **i32)
        counts = torch.empty(E, **i32)
        native._check(lib.b200_moe_rank(ids.data_ptr(), A, E, hist.data_ptr(), self.pos.data_ptr(), counts.data_ptr(),
                                        st), "b200_moe_rank")
        counts_all = torch.empty(R, E, **i32)
        dist.all_gather_into_tensor(counts_all, counts, group=ex.ep_group)
        kept = counts_all.clamp(max=capacity)                                   # [src, expert]
        total = kept.sum(dim=0)                                                 # rows of every expert at its owner
        padded = (total + (TILE - 1)) // TILE * TILE
        per_owner = padded.view(R, el)
        pad_start = (per_owner.cumsum(dim=1) - per_owner).reshape(E)            # inside the owner's buffer
        before = kept.cumsum(dim=0) - kept                                      # rows of earlier senders
        self.starts = (pad_start + before[rank]).to(torch.int32).contiguous()   # my first row per global expert
        # static bound of an owner's buffer: every sender may fill every local expert up to the capacity
        self.rows_per_rank = (el * ((R * capacity + TILE - 1) // TILE * TILE) + TILE - 1) // TILE * TILE
        self.dest = torch.empty(A, **i32)
        native._check(lib.b200_moe_dest(ids.data_ptr(), self.pos.data_ptr(), self.starts.data_ptr(), A, E, capacity, el,
                                        self.rows_per_rank, self.dest.data_ptr(), None, st), "b200_moe_dest")
        # owner side: layout of my local experts (tile table and contraction ranges for the grouped GEMMs)
        tiles = self.rows_per_rank // TILE
        mine = total[rank * el:(rank + 1) * el].to(torch.int32).contiguous()
        starts_local = torch.empty(el, **i32)
        k_range = torch.empty(2 * el, **i32)
        tile_group = torch.empty(tiles, **i32)
        native._check(lib.b200_moe_layout(mine.data_ptr(), el, 0, TILE, tiles, starts_local.data_ptr(),
                                          k_range.data_ptr(), tile_group.data_ptr(), None, st), "b200_moe_layout")
        self.owner = SimpleNamespace(tile_group=tile_group, k_range=k_range.view(el, 2))
        self.ex = ex
        self.ws = workspace_for(ex, self.rows_per_rank, hidden, dev)   # None: peer memory refused, use NCCL

    @property
    def kept_mask(self) -> torch.Tensor:
        return (self.dest >= 0).view(self.T, self.k)


def _push_rows(x, scale, plan: ExpertParallelPlan, ws: ExpertParallelWorkspace, *, keep: bool) -> torch.Tensor:
    """Zero my inbox, barrier, store my rows into the owners' inboxes, barrier.  Returns my inbox: a private copy
    when the rows must outlive the next use of the inbox (``keep``: forward activations saved for backward), else
    the arena view itself (gradients, which the next autograd node consumes before anything is pushed again)."""

    lib = _moe_lib()
    used = ws.inbox[:plan.rows_per_rank]
    used.zero_()
    ws.barrier()
    rc = lib.b200_moe_gather(x.data_ptr(), None if scale is None else scale.data_ptr(), None, plan.dest.data_ptr(),
                             ws.ptrs(ws.inbox_off), ws.world, plan.T * plan.k, x.shape[1], plan.k, plan.rows_per_rank,
                             native._stream())
    native._check(rc, "b200_moe_gather")
    ws.barrier()
    return used.clone() if keep else used


def _pull_rows(local_rows, w, plan: ExpertParallelPlan, ws: ExpertParallelWorkspace, rows_out=None) -> torch.Tensor:
    """Publish my outbox, barrier, gather-and-sum my tokens' rows from the owners' outboxes (optionally keeping the
    unweighted rows in ``rows_out``).  The caller issues the closing barrier."""

    lib = _moe_lib()
    mine = ws.outbox[:plan.rows_per_rank]
    if local_rows.data_ptr() != mine.data_ptr():   # the grouped GEMM normally writes straight into the outbox
        mine.copy_(local_rows)
    ws.barrier()
    H = local_rows.shape[1]
    y = torch.empty(plan.T, H, dtype=torch.bfloat16, device=local_rows.device)
    rc = lib.b200_moe_combine(ws.ptrs(ws.outbox_off), ws.world, None if w is None else w.data_ptr(),
                              plan.dest.data_ptr(), y.data_ptr(), None if rows_out is None else rows_out.data_ptr(),
                              plan.T, H, plan.k, plan.rows_per_rank, native._stream())
    native._check(rc, "b200_moe_combine")
    return y


class _EpDispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, plan, ws):
        ctx.plan, ctx.ws = plan, ws
        return _push_rows(x.contiguous(), None, plan, ws, keep=True)

    @staticmethod
    def backward(ctx, d_rows):
        plan, ws = ctx.plan, ctx.ws
        dx = _pull_rows(d_rows.contiguous(), None, plan, ws)
        ws.barrier()  # everybody has read my outbox
        return dx, None, None


class _EpCombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rows, w, plan, ws):
        lib = _moe_lib()
        w32 = w.reshape(-1).to(torch.float32).contiguous()
        # keep my unweighted rows for the gradient of the routing weights: the same pass that sums them stores them
        mine = torch.empty(plan.T * plan.k, rows.shape[1], dtype=torch.bfloat16, device=rows.device)
        y = _pull_rows(rows.contiguous(), w32, plan, ws, rows_out=mine)
        ws.barrier()  # everybody has read my outbox
        ctx.save_for_backward(mine, w32)
        ctx.plan, ctx.ws, ctx.w_dtype, ctx.w_shape = plan, ws, w.dtype, w.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        mine, w32 = ctx.saved_tensors
        plan, ws = ctx.plan, ctx.ws
        dy = dy.contiguous()
        d_rows = _push_rows(dy, w32, plan, ws, keep=False) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            # dw[a] = <row a of my unweighted expert outputs, dy[token of a]>: one warp per assignment
            lib = _moe_lib()
            A = plan.T * plan.k
            ident = plan.__dict__.get("_ident")
            if ident is None:
                ident = plan._ident = torch.arange(A, device=dy.device, dtype=torch.int32)
            dw32 = torch.empty(A, dtype=torch.float32, device=dy.device)
            one = (ctypes.c_void_p * 1)()
            one[0] = mine.data_ptr()
            rc = lib.b200_moe_combine_dw(one, 1, dy.data_ptr(), ident.data_ptr(), dw32.data_ptr(), A, mine.shape[1],
                                         plan.k, 0, native._stream())
            native._check(rc, "b200_moe_combine_dw")
            dw = dw32.view(ctx.w_shape).to(ctx.w_dtype)
        return d_rows, dw, None, None


def fused_available(ex, x: torch.Tensor, capacity) -> bool:
    import os

    return (capacity is not None and ex.ep_size > 1 and ex.ep_size <= 8 and x.is_cuda and x.dtype == torch.bfloat16
            and Fn.use_native(x) and ex.ep_dispatcher in ("all_to_all", "rdep_static")
            and os.environ.get("RESEARCH_B200_PEER_COLLECTIVES", "1") != "0")


def dispatch_and_combine_fused(experts, x: torch.Tensor, weights: torch.Tensor, plan: ExpertParallelPlan) -> torch.Tensor:
    """x [T,H] bf16 local tokens, weights [T,k] (already masked by the capacity) -> sum_k w * expert(x)."""

    ex = plan.ex
    if x.shape[1] % 8:
        raise KernelError("expert-parallel dispatch needs a hidden size that is a multiple of 8")
    ws = plan.ws
    rows = _EpDispatchFn.apply(x, plan, ws)
    outbox = ws.outbox[:plan.rows_per_rank]
    # the input gradient of the first product and the output of the second are what peers read: write them
    # straight into the outbox
    h = Fn.swiglu(_GroupedLinearFn.apply(rows, experts.w_gate_up, plan.owner, None, outbox))
    out = _GroupedLinearFn.apply(h, experts.w_down, plan.owner, outbox, None)
    return _EpCombineFn.apply(out, weights, plan, ws)
