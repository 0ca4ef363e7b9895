"""Context-parallel attention with the K/V exchange inside the attention kernels.

Every rank of the context group copies its K and V rows into a buffer of a symmetric arena.  The first CTAs of the
attention launch pull the rows this rank's queries can see from their owners over NVLink into ONE staging buffer in
sequence order, block by block, while the remaining CTAs of the same launch attend to the blocks that have landed
(``ops/csrc/ring.cuh``, ``attention_fwd.cu``, ``attention_bwd.cu``).  The backward pass stages K/V the same way from
inside the dQ kernel, and the dK/dV kernel adds its tiles straight into the gradient buffers of the ranks that own
the kv rows (TMA reduce-adds over NVLink), so no all-gather precedes the kernels, no reduce-scatter follows them, and
a layer saves only its local K/V for backward.

The all-gather formulation of :mod:`research_b200.parallel.context` stays as the CPU path, the fallback and the test
oracle.  Reference structure: third_party/ThunderKittens/kernels/parallel/ring_attn/ring_attn_h100.cu:77-294.
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from research_b200.errors import KernelError
from research_b200.ops import native

RING_CHANNEL = 8
MAX_PEERS = 8
MAX_SEGMENTS = 16
c_void_p, c_int, c_ll, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


class RingHostArgs(ctypes.Structure):
    """Mirror of ``b200ring::RingHostArgs`` (ops/csrc/ring.cuh)."""

    _fields_ = [
        ("world", c_int), ("rank", c_int), ("n_transfer", c_int), ("n_units", c_int), ("seq_len", c_int),
        ("local_rows", c_int), ("epoch", ctypes.c_uint), ("seg_rows", c_int),
        ("seg_owner", c_int * MAX_SEGMENTS), ("seg_first_row", c_int * MAX_SEGMENTS),
        ("units", c_void_p), ("peer_k", c_void_p * MAX_PEERS), ("peer_v", c_void_p * MAX_PEERS),
        ("block_flags", c_void_p), ("flags", c_void_p * MAX_PEERS), ("counter", c_void_p),
        ("peer_dk", c_void_p * MAX_PEERS), ("peer_dv", c_void_p * MAX_PEERS),
    ]


def _declare(lib: ctypes.CDLL) -> None:
    if getattr(lib, "_ring_declared", False):
        return
    lib.b200_attn_fwd_ring.argtypes = [c_void_p] * 6 + [c_int] * 5 + [c_ll] * 8 + [c_float, c_int, c_ll, c_void_p,
                                                                                   c_void_p, c_void_p]
    lib.b200_attn_fwd_ring.restype = c_int
    lib.b200_attn_bwd_ring.argtypes = [c_void_p] * 10 + [c_int] * 5 + [c_ll] * 10 + [c_float, c_int, c_ll, c_void_p,
                                                                                    c_void_p, c_void_p]
    lib.b200_attn_bwd_ring.restype = c_int
    lib._ring_declared = True


def segment_layout(cp: int, s_local: int, zigzag: bool) -> tuple[int, list[int], list[int]]:
    """``(rows per segment, owner of every segment, first row of the segment in its owner's buffer)``.

    Zig-zag: the sequence is ``2 cp`` segments and rank ``r`` holds segments ``r`` and ``2 cp - 1 - r`` one after the
    other; contiguous: ``cp`` segments, rank ``r`` holds segment ``r``."""

    if not zigzag:
        return s_local, list(range(cp)), [0] * cp
    c = s_local // 2
    owners = [s if s < cp else 2 * cp - 1 - s for s in range(2 * cp)]
    first = [0 if s < cp else c for s in range(2 * cp)]
    return c, owners, first


def build_units(cp: int, rank: int, B: int, s_local: int, zigzag: bool) -> list[tuple[int, int, int, int]]:
    """``(owner, first row in the owner's buffer, block index in the sequence, batch)`` for every 128-row block that
    the queries of ``rank`` can see under a causal mask (everything up to the end of its last segment), in the order
    in which the attention CTAs walk the sequence."""

    seg_rows, owners, first = segment_layout(cp, s_local, zigzag)
    last_seg = max(s for s, o in enumerate(owners) if o == rank)
    blocks_per_seg = seg_rows // 128
    rows = []
    for gb in range((last_seg + 1) * blocks_per_seg):
        seg, inner = divmod(gb, blocks_per_seg)
        for b in range(B):
            rows.append((owners[seg], first[seg] + inner * 128, gb, b))
    return rows


def emulate_staging(local: torch.Tensor, group, zigzag: bool) -> torch.Tensor:
    """What the transfer CTAs build, with ``torch.distributed`` instead of peer loads: the staging buffer
    ``[B, cp * S_local, ...]`` of this rank, filled block by block from the unit table (rows that the rank never
    needs stay zero).  CPU tests compare it with the all-gather formulation."""

    cp, rank = dist.get_world_size(group), dist.get_rank(group)
    B, s_local = local.shape[0], local.shape[1]
    everyone = [torch.empty_like(local) for _ in range(cp)]
    dist.all_gather(everyone, local.contiguous(), group=group)
    stage = torch.zeros((B, cp * s_local) + tuple(local.shape[2:]), dtype=local.dtype, device=local.device)
    for owner, row, gb, b in build_units(cp, rank, B, s_local, zigzag):
        stage[b, gb * 128:(gb + 1) * 128] = everyone[owner][b, row:row + 128]
    return stage


class RingWorkspace:
    """Buffers of one context group for one K/V shape ``[B, S_local, Hkv, D]``."""

    def __init__(self, group, B: int, s_local: int, hkv: int, D: int, zigzag: bool, device: torch.device,
                 transfer_ctas: int | None = None):
        from research_b200.parallel.symmetric import SymmetricArena

        self.group = group
        self.cp, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.B, self.s_local, self.hkv, self.D, self.zigzag = B, s_local, hkv, D, zigzag
        self.seq_len = self.cp * s_local
        self.seg_rows, self.seg_owner, self.seg_first = segment_layout(self.cp, s_local, zigzag)
        self.transfer_ctas = int(transfer_ctas or os.environ.get("RESEARCH_B200_RING_CTAS", "16"))
        n = B * s_local * hkv * D
        self.arena = SymmetricArena(group, 4 * n * 2 + 4 * 4096, device=device, tag="ring-attn", multicast=False)
        shape = (B, s_local, hkv, D)
        (k, self.k_off), (v, self.v_off) = self.arena.carve(n, torch.bfloat16), self.arena.carve(n, torch.bfloat16)
        (dk, self.dk_off), (dv, self.dv_off) = self.arena.carve(n, torch.bfloat16), self.arena.carve(n, torch.bfloat16)
        self.k_slot, self.v_slot, self.dk_acc, self.dv_acc = (t.view(shape) for t in (k, v, dk, dv))
        self.stage_k = torch.empty(B, self.seq_len, hkv, D, dtype=torch.bfloat16, device=device)
        self.stage_v = torch.empty_like(self.stage_k)
        self.block_flags = torch.zeros(B * self.seq_len // 128, dtype=torch.int32, device=device)
        self.counter = torch.zeros(4, dtype=torch.int32, device=device)
        rows = build_units(self.cp, self.rank, B, s_local, zigzag)
        self.n_units = len(rows)
        self.units = torch.tensor(rows, dtype=torch.int32, device=device).contiguous()
        self.bytes_over_nvlink = sum(1 for r in rows if r[0] != self.rank) * 2 * 128 * hkv * D * 2

    def args(self, *, stage: bool, epoch: int) -> RingHostArgs:
        a = RingHostArgs()
        a.world, a.rank = self.cp, self.rank
        a.n_transfer, a.n_units = (self.transfer_ctas, self.n_units) if stage else (0, 0)
        a.seq_len, a.local_rows, a.epoch, a.seg_rows = self.seq_len, self.s_local, epoch, self.seg_rows
        for s, (owner, first) in enumerate(zip(self.seg_owner, self.seg_first)):
            a.seg_owner[s], a.seg_first_row[s] = owner, first
        a.units = self.units.data_ptr()
        flags = self.arena.flag_ptrs(RING_CHANNEL)
        for r in range(self.cp):
            a.peer_k[r] = self.arena.peer_ptr(r, self.k_off)
            a.peer_v[r] = self.arena.peer_ptr(r, self.v_off)
            a.peer_dk[r] = self.arena.peer_ptr(r, self.dk_off)
            a.peer_dv[r] = self.arena.peer_ptr(r, self.dv_off)
            a.flags[r] = flags[r]
        a.block_flags = self.block_flags.data_ptr()
        a.counter = self.counter.data_ptr()
        return a


_WORKSPACES: dict[tuple, RingWorkspace | None] = {}


def workspace_for(group, B: int, s_local: int, hkv: int, D: int, zigzag: bool, device: torch.device):
    """The workspace of this group and shape, built collectively on first use; ``None`` when symmetric memory is
    unavailable on some rank (the caller then takes the all-gather formulation)."""

    from research_b200.parallel.symmetric import build_collectively

    key = (id(group), B, s_local, hkv, D, zigzag, device.index)
    if key not in _WORKSPACES:
        _WORKSPACES[key] = build_collectively(group, lambda: RingWorkspace(group, B, s_local, hkv, D, zigzag, device),
                                              "symmetric arena for ring attention")
    return _WORKSPACES[key]


def ring_available(ex, q: torch.Tensor, s_local: int, hkv: int, D: int, chunks) -> bool:
    """Shapes and switches under which the in-kernel exchange runs (else: all-gather + flash attention)."""

    if os.environ.get("RESEARCH_B200_PEER_COLLECTIVES", "1") == "0" or os.environ.get("RESEARCH_B200_RING", "1") == "0":
        return False
    if native.deterministic():          # dK / dV partial sums are reduce-added into their owner in arrival order
        return False
    if not (q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128) and 2 <= ex.cp_size <= MAX_PEERS):
        return False
    if (128 * hkv * D * 2) % 16384:
        return False
    return all(first % 128 == 0 and length % 128 == 0 for first, length in chunks) and s_local % 128 == 0


class _RingAttentionFn(torch.autograd.Function):
    """q [B, S_local, Hq, D], k / v [B, S_local, Hkv, D] (local rows), ``lo`` [B, S_local] first visible GLOBAL kv
    position per row or None; ``chunks``: ``(first global position, length)`` runs of the local rows."""

    @staticmethod
    def forward(ctx, q, k, v, lo, ws: RingWorkspace, chunks, scale):
        lib = native.load()
        _declare(lib)
        B, S, Hq, D = q.shape
        Hkv = k.shape[2]
        ws.k_slot.copy_(k)
        ws.v_slot.copy_(v)
        epoch = ws.arena.next_epoch(RING_CHANNEL)
        o = torch.empty((B, S, Hq, D), dtype=q.dtype, device=q.device)
        order = sorted(range(len(chunks)), key=lambda i: -chunks[i][0])          # the chunk that sees most keys first
        starts = [sum(c[1] for c in chunks[:i]) for i in range(len(chunks))]
        lses, los = [None] * len(chunks), [None] * len(chunks)
        for n, i in enumerate(order):
            first, length = chunks[i]
            row = starts[i]
            q_c, o_c = q[:, row:row + length], o[:, row:row + length]
            lo_c = None if lo is None else lo[:, row:row + length].contiguous()
            lse = torch.empty((B, Hq, length), dtype=torch.float32, device=q.device)
            args = ws.args(stage=n == 0, epoch=epoch)
            rc = lib.b200_attn_fwd_ring(
                q_c.data_ptr(), ws.stage_k.data_ptr(), ws.stage_v.data_ptr(), o_c.data_ptr(), lse.data_ptr(),
                native._ptr(lo_c), B, length, Hq, Hkv, D, q_c.stride(1), q_c.stride(0), ws.stage_k.stride(1),
                ws.stage_k.stride(0), ws.stage_v.stride(1), ws.stage_v.stride(0), o_c.stride(1), o_c.stride(0), scale, 1,
                (first + length) | (int(first) << 32), ctypes.addressof(args),
                native.status_word(q.device).data_ptr(), native._stream())
            native._check(rc, "b200_attn_fwd_ring")
            lses[i], los[i] = lse, lo_c
        ctx.save_for_backward(q, k, v, o, *lses, *[t for t in los if t is not None])
        ctx.cfg = (ws, chunks, scale, starts, order, lo is not None)
        return o

    @staticmethod
    def backward(ctx, d_o):
        ws, chunks, scale, starts, order, has_lo = ctx.cfg
        saved = ctx.saved_tensors
        q, k, v, o = saved[:4]
        lses = saved[4:4 + len(chunks)]
        los = list(saved[4 + len(chunks):]) if has_lo else [None] * len(chunks)
        lib = native.load()
        B, S, Hq, D = q.shape
        Hkv = k.shape[2]
        d_o = d_o.reshape(B, S, Hq, D)
        if not d_o.is_contiguous():
            d_o = d_o.contiguous()
        ws.dk_acc.zero_()          # before this rank's announcement inside the dQ launch: no peer adds earlier
        ws.dv_acc.zero_()
        ws.k_slot.copy_(k)
        ws.v_slot.copy_(v)
        epoch = ws.arena.next_epoch(RING_CHANNEL)
        dq = torch.empty_like(q)
        for n, i in enumerate(order):
            first, length = chunks[i]
            row = starts[i]
            q_c, o_c, do_c, dq_c = (t[:, row:row + length] for t in (q, o, d_o, dq))
            lo_c = los[i]
            hi_c = None if lo_c is None else native.kv_visibility_upper_bound(lo_c, first + length, first)
            delta = torch.empty((B, Hq, length), dtype=torch.float32, device=q.device)
            args = ws.args(stage=n == 0, epoch=epoch)
            rc = lib.b200_attn_bwd_ring(
                q_c.data_ptr(), ws.stage_k.data_ptr(), ws.stage_v.data_ptr(), o_c.data_ptr(), do_c.data_ptr(),
                lses[i].data_ptr(), delta.data_ptr(), dq_c.data_ptr(), native._ptr(lo_c), native._ptr(hi_c), B, length,
                Hq, Hkv, D, q_c.stride(1), q_c.stride(0), ws.stage_k.stride(1), ws.stage_k.stride(0), o_c.stride(1),
                o_c.stride(0), do_c.stride(1), do_c.stride(0), dq_c.stride(1), dq_c.stride(0), scale, 1,
                (first + length) | (int(first) << 32), ctypes.addressof(args),
                native.status_word(q.device).data_ptr(), native._stream())
            native._check(rc, "b200_attn_bwd_ring")
            native.LAUNCHES += 2
        ws.arena.barrier(channel=RING_CHANNEL + 1)      # every rank's adds into this rank's buffers have landed
        return dq, ws.dk_acc.clone(), ws.dv_acc.clone(), None, None, None, None


def ring_attention(q, k, v, lo, ws: RingWorkspace, chunks, scale: float) -> torch.Tensor:
    if ws.cp < 2:
        raise KernelError("ring attention needs a context group of at least two ranks")
    return _RingAttentionFn.apply(q.contiguous(), k.contiguous(), v.contiguous(), lo, ws, tuple(chunks), scale)
