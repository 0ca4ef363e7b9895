"""Grouped expert feed-forward: every local expert's SwiGLU applied to its own contiguous block of rows.

Native path: rows are laid out expert-major with every expert's block padded to a multiple of 128 rows, so a
single persistent tcgen05 GEMM launch covers all experts - the B operand (the expert's weight) is selected per
128-row tile from a small device-side table, and weight gradients are one launch with a per-expert contraction
range.  All bookkeeping stays on the device: no host synchronisation on the routing counts.
Reference path: a loop over experts in plain PyTorch (what the reference's ``ragged_dot`` computes,
src/jaxtitan/models/components/moe.py:636-641).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from research_b200.ops import functional as Fn
from research_b200.ops import native

TILE = 128


class PaddedLayout:
    """Expert-major padded row layout derived from per-expert counts (device tensors only)."""

    def __init__(self, counts: torch.Tensor, total_rows: int):
        E = counts.numel()
        counts = counts.to(torch.int64)
        padded = (counts + (TILE - 1)) // TILE * TILE
        ends = torch.cumsum(padded, 0)
        starts = ends - padded
        self.rows_pad = (total_rows + E * (TILE - 1) + TILE - 1) // TILE * TILE   # static upper bound
        self.starts = starts
        src_starts = torch.cumsum(counts, 0) - counts
        # destination row of every sorted assignment
        idx = torch.arange(total_rows, device=counts.device)
        expert_of = torch.searchsorted(torch.cumsum(counts, 0), idx, right=True).clamp_max(E - 1)
        self.dest = (starts[expert_of] + (idx - src_starts[expert_of])).contiguous()
        tiles = self.rows_pad // TILE
        tile_start = torch.arange(tiles, device=counts.device) * TILE
        tg = torch.searchsorted(ends, tile_start, right=True)
        self.tile_group = torch.where(tile_start < ends[-1], tg, torch.full_like(tg, -1)).to(torch.int32).contiguous()
        self.k_range = torch.stack([starts, ends], dim=1).to(torch.int32).contiguous()


def _grouped_rows(a: torch.Tensor, w3: torch.Tensor, layout: PaddedLayout, *, b_mn: bool, out_n: int,
                  out: torch.Tensor | None = None) -> torch.Tensor:
    lib = native.load()
    if out is None:
        out = torch.empty(a.shape[0], out_n, dtype=torch.bfloat16, device=a.device)
    E = w3.shape[0]
    K = a.shape[1]
    rc = lib.b200_gemm_bf16_grouped_rows(a.data_ptr(), w3.data_ptr(), out.data_ptr(), a.shape[0], out_n, K, E,
                                         a.stride(0), w3.stride(1), out.stride(0), w3.stride(0), int(b_mn), 0, 0,
                                         layout.tile_group.data_ptr(), native.status_word(a.device).data_ptr(),
                                         native._stream())
    native._check(rc, "b200_gemm_bf16_grouped_rows")
    return out


def _grouped_k(a: torch.Tensor, b: torch.Tensor, out3: torch.Tensor, layout: PaddedLayout) -> None:
    lib = native.load()
    E, M, N = out3.shape
    rc = lib.b200_gemm_bf16_grouped_k(a.data_ptr(), b.data_ptr(), out3.data_ptr(), M, N, a.shape[0], E, a.stride(0),
                                      b.stride(0), out3.stride(1), out3.stride(0), int(out3.dtype == torch.float32), 1,
                                      layout.k_range.data_ptr(), native.status_word(a.device).data_ptr(),
                                      native._stream())
    native._check(rc, "b200_gemm_bf16_grouped_k")


class _GroupedLinearFn(torch.autograd.Function):
    """y[rows of expert e] = x[rows of e] @ W[e]^T for an expert-major padded x."""

    @staticmethod
    def forward(ctx, x_pad, p, layout, out=None, dx_out=None):
        """``out`` / ``dx_out``: optional preallocated buffers for the product and for the input gradient (the
        expert-parallel path points them at its outbox in the symmetric arena, which saves a copy each way)."""

        w = Fn.compute_weight(p, x_pad)
        ctx.save_for_backward(x_pad)
        ctx.p, ctx.layout, ctx.dx_out = p, layout, dx_out
        return _grouped_rows(x_pad, w, layout, b_mn=False, out_n=w.shape[1], out=out)

    @staticmethod
    def backward(ctx, dy):
        (x_pad,) = ctx.saved_tensors
        p, layout = ctx.p, ctx.layout
        w = Fn.compute_weight(p, x_pad)
        dy = dy.contiguous()
        dx = _grouped_rows(dy, w, layout, b_mn=True, out_n=w.shape[2], out=ctx.dx_out)
        if p.requires_grad:
            _grouped_k(dy, x_pad, Fn._main_grad(p), layout)
        return dx, None, None, None, None


def grouped_expert_ffn(rows: torch.Tensor, counts: torch.Tensor, w_gate_up: torch.Tensor,
                       w_down: torch.Tensor) -> torch.Tensor:
    """rows: ``[R, H]`` sorted by local expert; counts: ``[E]`` rows per expert.  Returns ``[R, H]``."""

    R = rows.shape[0]
    if Fn.use_native(rows) and R > 0:
        layout = PaddedLayout(counts, R)
        x_pad = torch.zeros(layout.rows_pad, rows.shape[1], dtype=rows.dtype, device=rows.device)
        x_pad = x_pad.index_copy(0, layout.dest, rows)
        h = Fn.swiglu(_GroupedLinearFn.apply(x_pad, w_gate_up, layout))
        y_pad = _GroupedLinearFn.apply(h, w_down, layout)
        return y_pad.index_select(0, layout.dest)
    out = torch.zeros_like(rows)
    offsets = [0] + torch.cumsum(counts.to(torch.int64), 0).tolist()
    pieces = []
    for e in range(w_gate_up.shape[0]):
        seg = rows[offsets[e]:offsets[e + 1]]
        if seg.shape[0] == 0:
            continue
        h = Fn.swiglu(F.linear(seg, w_gate_up[e].to(seg.dtype)))
        pieces.append(F.linear(h, w_down[e].to(seg.dtype)))
    if pieces:
        return torch.cat(pieces, dim=0)
    # No row reached these experts.  The result must still be a function of ``rows``: under expert parallelism the
    # exchanges before and after this call run in the backward pass of every rank or of none, and a result cut off
    # from its input would take them out of this rank's backward while its peers wait in theirs.
    return out + rows * 0


# --------------------------------------------------------------------------------------------------
# Native routing plan: ranks, capacity, padded layout, dispatch and combine without sorts or one-hots
# --------------------------------------------------------------------------------------------------
import ctypes as _ct


def _moe_lib():
    lib = native.load()
    if not getattr(lib, "_moe_declared", False):
        vp, ci, ll = _ct.c_void_p, _ct.c_int, _ct.c_longlong
        pvp = _ct.POINTER(vp)
        lib.b200_moe_chunks.argtypes = [ci]
        lib.b200_moe_rank.argtypes = [vp, ci, ci, vp, vp, vp, vp]
        lib.b200_moe_layout.argtypes = [vp, ci, ci, ci, ci, vp, vp, vp, vp, vp]
        lib.b200_moe_dest.argtypes = [vp, vp, vp, ci, ci, ci, ci, ll, vp, vp, vp]
        lib.b200_moe_zero_pad.argtypes = [vp, vp, vp, ci, ci, vp]
        lib.b200_moe_zero_pad.restype = ci
        lib.b200_moe_gather.argtypes = [vp, vp, vp, vp, pvp, ci, ll, ci, ci, ll, vp]
        lib.b200_moe_combine.argtypes = [pvp, ci, vp, vp, vp, vp, ll, ci, ci, ll, vp]
        lib.b200_moe_combine_dw.argtypes = [pvp, ci, vp, vp, vp, ll, ci, ci, ll, vp]
        lib.b200_moe_post_sources.argtypes = [vp, ll, ci, ll, ci, ci, _ct.c_uint, pvp, vp]
        lib.b200_moe_post_sources.restype = ci
        lib.b200_moe_dispatch_gemm.argtypes = [pvp, ci, vp, vp, vp, vp, ci, ci, ci, ci, ll, ll, vp, ci, ci, ci, vp, vp,
                                               _ct.c_uint, vp, vp]
        lib.b200_moe_dispatch_gemm.restype = ci
        for fn in (lib.b200_moe_chunks, lib.b200_moe_rank, lib.b200_moe_layout, lib.b200_moe_dest, lib.b200_moe_gather,
                   lib.b200_moe_combine, lib.b200_moe_combine_dw):
            fn.restype = ci
        lib._moe_declared = True
    return lib


def _one_ptr(t: torch.Tensor):
    arr = (_ct.c_void_p * 1)()
    arr[0] = t.data_ptr()
    return arr


class RoutingPlan:
    """Device-side plan of one MoE layer: where every (token, choice) assignment goes in the expert-major buffer
    whose expert blocks are padded to 128 rows.  ``capacity`` (rows per expert, token-order priority) is optional.
    Carries ``tile_group`` / ``k_range`` for the grouped GEMMs (the attributes :class:`PaddedLayout` has)."""

    def __init__(self, expert_ids: torch.Tensor, num_experts: int, capacity: int | None = None):
        lib = _moe_lib()
        dev = expert_ids.device
        self.T, self.k = expert_ids.shape
        A = self.T * self.k
        E = num_experts
        ids = expert_ids.reshape(-1).to(torch.int32).contiguous()
        cap = int(capacity) if capacity else 0
        per_expert = min(A, cap) if cap else A
        bound = min(A + E * (TILE - 1), E * ((per_expert + TILE - 1) // TILE * TILE))
        self.rows_pad = (bound + TILE - 1) // TILE * TILE
        tiles = self.rows_pad // TILE
        i32 = dict(dtype=torch.int32, device=dev)
        hist = torch.empty(lib.b200_moe_chunks(A) * E, **i32)
        self.pos = torch.empty(A, **i32)
        self.counts = torch.empty(E, **i32)
        self.starts = torch.empty(E, **i32)
        self.k_range = torch.empty(2 * E, **i32)
        self.tile_group = torch.empty(tiles, **i32)
        self.kept = torch.empty(E, **i32)
        self.dest = torch.empty(A, **i32)
        self.src = torch.full((self.rows_pad,), -1, **i32)
        st = native._stream()
        native._check(lib.b200_moe_rank(ids.data_ptr(), A, E, hist.data_ptr(), self.pos.data_ptr(),
                                        self.counts.data_ptr(), st), "b200_moe_rank")
        native._check(lib.b200_moe_layout(self.counts.data_ptr(), E, cap, TILE, tiles, self.starts.data_ptr(),
                                          self.k_range.data_ptr(), self.tile_group.data_ptr(), self.kept.data_ptr(),
                                          st), "b200_moe_layout")
        native._check(lib.b200_moe_dest(ids.data_ptr(), self.pos.data_ptr(), self.starts.data_ptr(), A, E, cap, 0, 0,
                                        self.dest.data_ptr(), self.src.data_ptr(), st), "b200_moe_dest")
        native.LAUNCHES += 1
        self.k_range = self.k_range.view(E, 2)

    @property
    def kept_mask(self) -> torch.Tensor:
        """[T, k] bool: assignments that were not dropped by the capacity."""

        return (self.dest >= 0).view(self.T, self.k)


def _gather_rows(x, scale, plan: RoutingPlan) -> torch.Tensor:
    lib = _moe_lib()
    H = x.shape[1]
    out = torch.empty(plan.rows_pad, H, dtype=torch.bfloat16, device=x.device)
    rc = lib.b200_moe_gather(x.data_ptr(), None if scale is None else scale.data_ptr(), plan.src.data_ptr(),
                             plan.dest.data_ptr(), _one_ptr(out), 1, plan.rows_pad, H, plan.k, 0, native._stream())
    native._check(rc, "b200_moe_gather")
    return out


def _combine_rows(pad, w, plan: RoutingPlan) -> torch.Tensor:
    lib = _moe_lib()
    H = pad.shape[1]
    y = torch.empty(plan.T, H, dtype=torch.bfloat16, device=pad.device)
    rc = lib.b200_moe_combine(_one_ptr(pad), 1, None if w is None else w.data_ptr(), plan.dest.data_ptr(), y.data_ptr(),
                              None, plan.T, H, plan.k, 0, native._stream())
    native._check(rc, "b200_moe_combine")
    return y


class _DispatchFn(torch.autograd.Function):
    """x [T,H] -> expert-major padded rows; backward sums the k row gradients of every token."""

    @staticmethod
    def forward(ctx, x, plan):
        ctx.plan = plan
        return _gather_rows(x.contiguous(), None, plan)

    @staticmethod
    def backward(ctx, d_pad):
        return _combine_rows(d_pad.contiguous(), None, ctx.plan), None


class _CombineFn(torch.autograd.Function):
    """y[t] = sum_j w[t,j] * pad[dest[t,j]]; gradients for the rows and for the routing weights."""

    @staticmethod
    def forward(ctx, pad, w, plan):
        w32 = w.reshape(-1).to(torch.float32).contiguous()
        ctx.save_for_backward(pad, w32)
        ctx.plan, ctx.w_dtype, ctx.w_shape = plan, w.dtype, w.shape
        return _combine_rows(pad.contiguous(), w32, plan)

    @staticmethod
    def backward(ctx, dy):
        pad, w32 = ctx.saved_tensors
        plan = ctx.plan
        dy = dy.contiguous()
        d_pad = _gather_rows(dy, w32, plan) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            lib = _moe_lib()
            dw32 = torch.empty(plan.T * plan.k, dtype=torch.float32, device=dy.device)
            rc = lib.b200_moe_combine_dw(_one_ptr(pad), 1, dy.data_ptr(), plan.dest.data_ptr(), dw32.data_ptr(),
                                         plan.T * plan.k, pad.shape[1], plan.k, 0, native._stream())
            native._check(rc, "b200_moe_combine_dw")
            dw = dw32.view(ctx.w_shape).to(ctx.w_dtype)
        return d_pad, dw, None


def routed_expert_ffn(x: torch.Tensor, weights: torch.Tensor, plan: RoutingPlan, w_gate_up: torch.Tensor,
                      w_down: torch.Tensor) -> torch.Tensor:
    """Local routed experts on the native path: dispatch -> grouped SwiGLU FFN -> weighted combine.
    ``x`` [T,H] bf16, ``weights`` [T,k] (dropped assignments contribute nothing whatever their weight)."""

    x_pad = _DispatchFn.apply(x, plan)
    h = Fn.swiglu(_GroupedLinearFn.apply(x_pad, w_gate_up, plan))
    y_pad = _GroupedLinearFn.apply(h, w_down, plan)
    return _CombineFn.apply(y_pad, weights, plan)
