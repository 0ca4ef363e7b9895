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
Every MoE layer has an inbox of its own for the forward rows (they are what the backward pass of the grouped GEMMs
reads, so nothing is copied out of the arena), a shared inbox takes the gradient rows, and only the padding rows
behind each expert's block are zeroed before a push.

With a per-layer inbox the forward dispatch and the first expert GEMM are one kernel (``ops/csrc/moe_comm_gemm.cu``):
the senders only post 8 bytes per row (which token of which rank the row is), the owner's kernel pulls the rows
from the senders' token buffers with its transfer CTAs and its tensor-core CTAs start on every 128-row tile as soon
as that tile has landed.  ``RESEARCH_B200_MOE_FUSED=0`` keeps the push + barrier + GEMM sequence.
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


FORWARD_SLOT_BUDGET_BYTES = 48 << 30     # per-layer forward inboxes are used while they fit in this much memory


class ExpertParallelWorkspace:
    """Row buffers per rank in a symmetric arena: inboxes that peers write (one per MoE layer for the forward rows
    when that fits the budget, one shared for gradient rows) and an outbox that peers read (combine, backward of
    dispatch)."""

    def __init__(self, group, rows: int, hidden: int, device: torch.device, layers: int = 0, tokens: int = 0):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.rows, self.hidden, self.tokens = rows, hidden, tokens
        per = rows * hidden * 2
        self.forward_slots = layers if 0 < layers and layers * per <= FORWARD_SLOT_BUDGET_BYTES else 0
        n_in = 1 + self.forward_slots
        fused_bytes = (tokens * hidden * 2 + rows * 8 + 1024) if (tokens and self.forward_slots) else 0
        self.arena = SymmetricArena(group, (n_in + 1) * (per + 512) + fused_bytes + 8192, device=device, tag="ep")
        self.inboxes, self.inbox_offs = [], []
        for _ in range(n_in):
            t, off = self.arena.carve(rows * hidden, torch.bfloat16)
            self.inboxes.append(t.view(rows, hidden))
            self.inbox_offs.append(off)
        self.inbox, self.inbox_off = self.inboxes[0], self.inbox_offs[0]      # the shared (gradient) inbox
        self.outbox, self.outbox_off = self.arena.carve(rows * hidden, torch.bfloat16)
        self.outbox = self.outbox.view(rows, hidden)
        # fused dispatch + GEMM: my tokens where peers can read them, the source list that peers write, and the
        # local per-tile flags (epochs only grow, so the arrays are shared by all layers and never cleared)
        self.xbox = None
        if fused_bytes:
            self.xbox, self.xbox_off = self.arena.carve(tokens * hidden, torch.bfloat16)
            self.xbox = self.xbox.view(tokens, hidden)
            self.sources, self.sources_off = self.arena.carve(rows, torch.int64)
            self.sources.zero_()
            self.row_flags = torch.zeros(rows // TILE, dtype=torch.int32, device=device)
            self.tile_parts = torch.zeros(rows // TILE, dtype=torch.int32, device=device)
            self.dispatch_epoch = 0

    def inbox_for(self, layer_slot: int | None) -> tuple[torch.Tensor, int, bool]:
        """``(buffer, arena offset, private)`` of the inbox for a forward push of MoE layer ``layer_slot`` (private:
        nothing else is pushed into it during the step) or, with None, of the shared gradient inbox."""

        if layer_slot is not None and layer_slot < self.forward_slots:
            return self.inboxes[1 + layer_slot], self.inbox_offs[1 + layer_slot], True
        return self.inbox, self.inbox_off, False

    def ptrs(self, offset: int):
        arr = (ctypes.c_void_p * self.world)()
        for r in range(self.world):
            arr[r] = self.arena.peer_ptr(r, offset)
        return arr

    def barrier(self) -> None:
        self.arena.barrier(BARRIER_CHANNEL)


def workspace_for(ex, rows: int, hidden: int, device: torch.device, tokens: int = 0) -> ExpertParallelWorkspace | None:
    """The arena workspace of the ep group, built (collectively) on first use; None when peer memory is refused."""

    if ex.extras.get("ep_workspace_failed"):
        return None
    ws = ex.extras.get("ep_workspace")
    if ws is None or ws.rows < rows or ws.hidden != hidden or ws.tokens < tokens:
        from research_b200.parallel.symmetric import build_collectively

        layers = int(ex.extras.get("moe_layer_count", 0))
        if ws is not None:
            rows, tokens = max(rows, ws.rows), max(tokens, ws.tokens)
            ws.arena.close()
        ws = build_collectively(ex.ep_group,
                                lambda: ExpertParallelWorkspace(ex.ep_group, rows, hidden, device, layers, tokens),
                                "expert-parallel workspace")
        ex.extras["ep_workspace"] = ws
        if ws is None:
            ex.extras["ep_workspace_failed"] = True
    return ws


class ExpertParallelPlan:
    """Routing plan of one layer under expert parallelism (device tensors only, no host synchronisation)."""

    def __init__(self, expert_ids: torch.Tensor, num_experts: int, capacity: int, ex, hidden: int,
                 layer_slot: int | None = None):
        lib = _moe_lib()
        self.layer_slot = layer_slot          # index of the MoE layer among the model's MoE layers (or None)
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
        self.local_starts, self.local_counts, self.local_experts = starts_local, mine, el
        self.ex = ex
        # None: peer memory refused, use NCCL
        self.ws = workspace_for(ex, self.rows_per_rank, hidden, dev, self.T if fused_gemm_requested() else 0)

    @property
    def kept_mask(self) -> torch.Tensor:
        return (self.dest >= 0).view(self.T, self.k)


def _push_rows(x, scale, plan: ExpertParallelPlan, ws: ExpertParallelWorkspace, *, forward: bool) -> torch.Tensor:
    """Store my rows into the owners' inboxes and return my inbox (an arena view, no copy).

    ``forward``: the rows are activations that the backward pass reads again.  They go into the inbox of this MoE
    layer, which nothing else writes during the step, so no barrier has to protect a previous reader.  Without a
    per-layer inbox (or for gradient rows) the shared inbox is used: a barrier first makes sure every owner has
    finished reading what the previous push left there, and forward rows are copied out afterwards.  Only the
    padding rows behind each expert's block are zeroed: the real rows are overwritten by the senders."""

    lib = _moe_lib()
    inbox, offset, private = ws.inbox_for(plan.layer_slot if forward else None)
    used = inbox[:plan.rows_per_rank]
    rc = lib.b200_moe_zero_pad(used.data_ptr(), plan.local_starts.data_ptr(), plan.local_counts.data_ptr(),
                               plan.local_experts, x.shape[1], native._stream())
    native._check(rc, "b200_moe_zero_pad")
    if not private:
        ws.barrier()
    rc = lib.b200_moe_gather(x.data_ptr(), None if scale is None else scale.data_ptr(), None, plan.dest.data_ptr(),
                             ws.ptrs(offset), ws.world, plan.T * plan.k, x.shape[1], plan.k, plan.rows_per_rank,
                             native._stream())
    native._check(rc, "b200_moe_gather")
    ws.barrier()
    return used.clone() if (forward and not private) else used


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
        return _push_rows(x.contiguous(), None, plan, ws, forward=True)

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
        d_rows = _push_rows(dy, w32, plan, ws, forward=False) if ctx.needs_input_grad[0] else None
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


def fused_gemm_requested() -> bool:
    import os

    return os.environ.get("RESEARCH_B200_MOE_FUSED", "1") != "0" and not native.deterministic()


class _EpDispatchLinearFn(torch.autograd.Function):
    """Forward dispatch and the gate|up product of the routed experts as one kernel: ``x`` [T, H] local tokens ->
    [rows, N] for my experts' rows.  The pulled rows stay in this layer's inbox for the weight gradient."""

    @staticmethod
    def forward(ctx, x, p, plan, ws):
        import os

        lib = _moe_lib()
        w = Fn.compute_weight(p, x)                                   # [local experts, N, K]
        inbox, _, private = ws.inbox_for(plan.layer_slot)
        if not private or ws.xbox is None:
            raise KernelError("the fused dispatch needs a per-layer inbox and a token buffer in the arena")
        rows, (T, H) = plan.rows_per_rank, x.shape
        used = inbox[:rows]
        ws.xbox[:T].copy_(x)
        ws.dispatch_epoch += 1
        epoch = ws.dispatch_epoch & 0x7FFFFFFF
        st = native._stream()
        rc = lib.b200_moe_post_sources(plan.dest.data_ptr(), plan.T * plan.k, plan.k, rows, ws.world, ws.rank, epoch,
                                       ws.ptrs(ws.sources_off), st)
        native._check(rc, "b200_moe_post_sources")
        ws.barrier()                                                  # token buffers and source lists are in place
        out = torch.empty(rows, w.shape[1], dtype=torch.bfloat16, device=x.device)
        rc = lib.b200_moe_dispatch_gemm(ws.ptrs(ws.xbox_off), ws.tokens, ws.sources.data_ptr(), used.data_ptr(),
                                        w.data_ptr(), out.data_ptr(), rows, w.shape[1], H, w.shape[0], w.stride(1),
                                        w.stride(0), plan.owner.tile_group.data_ptr(), ws.world, ws.rank,
                                        int(os.environ.get("RESEARCH_B200_MOE_XFER_CTAS", "32")),
                                        ws.row_flags.data_ptr(), ws.tile_parts.data_ptr(), epoch,
                                        native.status_word(x.device).data_ptr(), st)
        native._check(rc, "b200_moe_dispatch_gemm")
        ws.barrier()                                                  # peers have finished reading my tokens
        # kept as a plain attribute: every buffer of the arena is a view of one byte tensor, so a later copy into the
        # token buffer would trip the version check of a saved tensor although this layer's inbox is untouched
        ctx.rows_in = used
        ctx.p, ctx.plan, ctx.ws = p, plan, ws
        return out

    @staticmethod
    def backward(ctx, dy):
        from research_b200.ops.grouped import _grouped_k, _grouped_rows

        rows_in, p, plan, ws = ctx.rows_in, ctx.p, ctx.plan, ctx.ws
        w = Fn.compute_weight(p, rows_in)
        dy = dy.contiguous()
        # the input gradient of my rows goes straight into the outbox, from where their senders pull it
        d_rows = _grouped_rows(dy, w, plan.owner, b_mn=True, out_n=w.shape[2], out=ws.outbox[:plan.rows_per_rank])
        if p.requires_grad:
            _grouped_k(dy, rows_in, Fn._main_grad(p), plan.owner)
        dx = _pull_rows(d_rows, None, plan, ws)
        ws.barrier()  # everybody has read my outbox
        return dx, None, None, None


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
    outbox = ws.outbox[:plan.rows_per_rank]
    if (fused_gemm_requested() and ws.xbox is not None and ws.inbox_for(plan.layer_slot)[2] and x.shape[1] % 64 == 0
            and x.shape[0] <= ws.tokens and experts.w_gate_up.shape[1] % 64 == 0):
        # dispatch and the gate|up product in one kernel: the GEMM starts on row tiles as they arrive
        h = Fn.swiglu(_EpDispatchLinearFn.apply(x.contiguous(), experts.w_gate_up, plan, ws))
        out = _GroupedLinearFn.apply(h, experts.w_down, plan.owner, outbox, None)
        return _EpCombineFn.apply(out, weights, plan, ws)
    rows = _EpDispatchFn.apply(x, plan, ws)
    # the input gradient of the first product and the output of the second are what peers read: write them
    # straight into the outbox
    h = Fn.swiglu(_GroupedLinearFn.apply(rows, experts.w_gate_up, plan.owner, None, outbox))
    out = _GroupedLinearFn.apply(h, experts.w_down, plan.owner, outbox, None)
    return _EpCombineFn.apply(out, weights, plan, ws)
