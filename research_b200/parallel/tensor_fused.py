"""Tensor-parallel linears whose collective runs inside the GEMM kernel (``csrc/comm_gemm.cu``).

``column_linear``: sequence-parallel shard ``[B, S/tp, K]`` -> ``[B, S, N_local]``; the all-gather of the rows is
done by transfer CTAs of the GEMM kernel itself.  ``row_linear``: ``[B, S, K_local]`` -> sequence-parallel shard
``[B, S/tp, N]``; the GEMM epilogue reduce-adds each tile into the owner's buffer over NVLink.  The backward of
one is the other (plus an ordinary weight-gradient GEMM on the gathered operand), so a Megatron-style block runs
four fused kernels forward and four backward and no separate collective.

The NCCL formulation of the same ops (all_gather / reduce_scatter around plain GEMMs) is
:class:`research_b200.models.execution.ExecutionContext`'s default and the oracle in the tests.  Reference:
models/execution.py:183-250 (XLA inserts the collectives), kernels named in ``csrc/comm_gemm.cu``.
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from research_b200.errors import KernelError
from research_b200.ops import functional as Fn
from research_b200.ops import native
from research_b200.parallel.symmetric import SymmetricArena

GATHER_CHANNEL = 2
SCATTER_CHANNEL = 3


def _declare(lib) -> None:
    if getattr(lib, "_comm_gemm_declared", False):
        return
    vp, ci, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    pvp = ctypes.POINTER(vp)
    lib.b200_gemm_allgather.argtypes = [pvp, vp, vp, vp, ci, ci, ci, ll, ci, ci, ci, ci, ci, ci, vp, vp, pvp,
                                        ctypes.c_uint, vp, vp]
    lib.b200_gemm_allgather.restype = ci
    lib.b200_gemm_reducescatter.argtypes = [vp, vp, pvp, ci, ci, ci, ll, ll, ci, ci, ci, ci, vp, pvp, ctypes.c_uint,
                                            vp, vp]
    lib.b200_gemm_reducescatter.restype = ci
    lib._comm_gemm_declared = True


class TensorParallelFusion:
    """Workspace of one tensor-parallel group: a symmetric arena with a staging shard and an output shard."""

    def __init__(self, group, *, max_shard_elems: int, max_out_elems: int, device: torch.device | None = None,
                 transfer_ctas: int = 16):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.lib = native.load()
        if not hasattr(self.lib, "b200_gemm_allgather"):
            raise KernelError("the kernel library was built without the fused tensor-parallel GEMMs")
        _declare(self.lib)
        self.arena = SymmetricArena(group, 2 * (max_shard_elems + max_out_elems) + 4096, device=device, tag="tp")
        self.stage, self.stage_off = self.arena.carve(max_shard_elems, torch.bfloat16)
        self.out, self.out_off = self.arena.carve(max_out_elems, torch.bfloat16)
        self.device = self.arena.device
        self.row_flags = torch.zeros(1 << 16, dtype=torch.int32, device=self.device)
        self.counter = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.transfer_ctas = transfer_ctas

    def _ptrs(self, values):
        arr = (ctypes.c_void_p * self.world)()
        for i, v in enumerate(values):
            arr[i] = v
        return arr

    # ---- all-gather -> GEMM --------------------------------------------------------------------------
    def gather_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, *, b_mn: bool, chunk_rows: int):
        """x_shard ``[M/world, K]`` bf16, ``w`` ``[N, K]`` (``b_mn=False``) or ``[K, N]`` (``b_mn=True``).
        Returns ``(y [M, N], x_full [M, K])``; rows are interleaved in stretches of ``chunk_rows`` per rank."""

        m_local, K = x_shard.shape
        N = w.shape[1] if b_mn else w.shape[0]
        M = m_local * self.world
        if m_local % 128 or chunk_rows % 128 or m_local % chunk_rows or K % 64 or N % 64:
            raise KernelError(f"fused all-gather GEMM needs 128-row blocks and 64-column multiples, got "
                              f"rows {m_local}, stretch {chunk_rows}, K {K}, N {N}")
        if x_shard.numel() > self.stage.numel() or M // 128 > self.row_flags.numel():
            raise KernelError("fused all-gather GEMM: shard larger than the staging buffer")
        stage = self.stage[:x_shard.numel()].view(m_local, K)
        stage.copy_(x_shard)
        x_full = torch.empty((M, K), dtype=torch.bfloat16, device=self.device)
        # own rows go into the gathered operand here (one strided local copy); the kernel moves only remote rows
        x_full.view(-1, self.world, chunk_rows, K)[:, self.rank].copy_(x_shard.view(-1, chunk_rows, K))
        y = torch.empty((M, N), dtype=torch.bfloat16, device=self.device)
        shards = self._ptrs([self.arena.peer_ptr(r, self.stage_off) for r in range(self.world)])
        flags = self._ptrs(self.arena.flag_ptrs(GATHER_CHANNEL))
        rc = self.lib.b200_gemm_allgather(shards, x_full.data_ptr(), w.data_ptr(), y.data_ptr(), M, N, K, w.stride(0),
                                          int(b_mn), self.world, self.rank, chunk_rows // 128, self.transfer_ctas, 0,
                                          self.row_flags.data_ptr(), self.counter.data_ptr(), flags,
                                          self.arena.next_epoch(GATHER_CHANNEL),
                                          native.status_word(self.device).data_ptr(), native._stream())
        native._check(rc, "b200_gemm_allgather")
        return y, x_full

    # ---- GEMM -> reduce-scatter ----------------------------------------------------------------------
    def gemm_scatter(self, a: torch.Tensor, w: torch.Tensor, *, b_mn: bool, chunk_rows: int) -> torch.Tensor:
        """``a`` ``[M, K]`` bf16 (this rank's partial operand), ``w`` as above.  Returns this rank's ``[M/world, N]``
        rows of the sum over ranks."""

        M, K = a.shape
        N = w.shape[1] if b_mn else w.shape[0]
        m_local = M // self.world
        if M % (128 * self.world) or chunk_rows % 128 or m_local % chunk_rows or K % 64 or N % 64:
            raise KernelError(f"fused GEMM reduce-scatter needs 128-row blocks and 64-column multiples, got "
                              f"M {M}, stretch {chunk_rows}, K {K}, N {N}")
        if m_local * N > self.out.numel():
            raise KernelError("fused GEMM reduce-scatter: output larger than the arena buffer")
        out = self.out[:m_local * N].view(m_local, N)
        out.zero_()
        shards = self._ptrs([self.arena.peer_ptr(r, self.out_off) for r in range(self.world)])
        flags = self._ptrs(self.arena.flag_ptrs(SCATTER_CHANNEL))
        rc = self.lib.b200_gemm_reducescatter(a.data_ptr(), w.data_ptr(), shards, M, N, K, a.stride(0), w.stride(0),
                                              int(b_mn), self.world, self.rank, chunk_rows // 128,
                                              self.counter[1:].data_ptr(), flags,
                                              self.arena.next_epoch(SCATTER_CHANNEL),
                                              native.status_word(self.device).data_ptr(), native._stream())
        native._check(rc, "b200_gemm_reducescatter")
        return out.clone()


class _ColumnLinearFn(torch.autograd.Function):
    """y = gather_seq(x) @ W^T, backward dx = reduce_scatter_seq(dy @ W)."""

    @staticmethod
    def forward(ctx, x, p, fusion):
        w = Fn.compute_weight(p, x)
        B, s_local, K = x.shape
        y, x_full = fusion.gather_gemm(x.reshape(B * s_local, K), w, b_mn=False, chunk_rows=s_local)
        ctx.save_for_backward(x_full)
        ctx.p, ctx.fusion, ctx.shape = p, fusion, (B, s_local, K)
        return y.view(B, s_local * fusion.world, w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        (x_full,) = ctx.saved_tensors
        p, fusion = ctx.p, ctx.fusion
        B, s_local, K = ctx.shape
        w = Fn.compute_weight(p, x_full)
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = fusion.gemm_scatter(dy2, w, b_mn=True, chunk_rows=s_local).view(B, s_local, K)
        if p.requires_grad:
            native.gemm_wgrad(dy2, x_full, Fn._main_grad(p))
        return dx, None, None


class _RowLinearFn(torch.autograd.Function):
    """y_shard = reduce_scatter_seq(h @ W^T), backward dh = gather_seq(dy) @ W."""

    @staticmethod
    def forward(ctx, h, p, fusion):
        w = Fn.compute_weight(p, h)
        B, S, K = h.shape
        s_local = S // fusion.world
        h2 = h.reshape(B * S, K)
        if not h2.is_contiguous():
            h2 = h2.contiguous()
        y = fusion.gemm_scatter(h2, w, b_mn=False, chunk_rows=s_local)
        ctx.save_for_backward(h2)
        ctx.p, ctx.fusion, ctx.shape = p, fusion, (B, S, K)
        return y.view(B, s_local, w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        (h2,) = ctx.saved_tensors
        p, fusion = ctx.p, ctx.fusion
        B, S, K = ctx.shape
        s_local = S // fusion.world
        w = Fn.compute_weight(p, h2)
        dy2 = dy.reshape(B * s_local, -1)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dh, dy_full = fusion.gather_gemm(dy2, w, b_mn=True, chunk_rows=s_local)
        if p.requires_grad:
            native.gemm_wgrad(dy_full, h2, Fn._main_grad(p))
        return (dh.view(B, S, K) if ctx.needs_input_grad[0] else None), None, None


def column_linear(x_shard: torch.Tensor, p: torch.Tensor, fusion: TensorParallelFusion) -> torch.Tensor:
    return _ColumnLinearFn.apply(x_shard, p, fusion)


def row_linear(h: torch.Tensor, p: torch.Tensor, fusion: TensorParallelFusion) -> torch.Tensor:
    return _RowLinearFn.apply(h, p, fusion)
