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


def _grouped_rows(a: torch.Tensor, w3: torch.Tensor, layout: PaddedLayout, *, b_mn: bool, out_n: int) -> torch.Tensor:
    lib = native.load()
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
    def forward(ctx, x_pad, p, layout):
        w = Fn.compute_weight(p, x_pad)
        ctx.save_for_backward(x_pad)
        ctx.p, ctx.layout = p, layout
        return _grouped_rows(x_pad, w, layout, b_mn=False, out_n=w.shape[1])

    @staticmethod
    def backward(ctx, dy):
        (x_pad,) = ctx.saved_tensors
        p, layout = ctx.p, ctx.layout
        w = Fn.compute_weight(p, x_pad)
        dy = dy.contiguous()
        dx = _grouped_rows(dy, w, layout, b_mn=True, out_n=w.shape[2])
        if p.requires_grad:
            _grouped_k(dy, x_pad, Fn._main_grad(p), layout)
        return dx, None, None


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
    return torch.cat(pieces, dim=0) if pieces else out
