"""Distributed Newton-Schulz for matrices that are split over the tensor-parallel group: execution plans, Gram
buckets, and the bucketed iteration itself.

What the reference does (src/jaxtitan/optim/muon.py:354-463, plans in src/jaxtitan/optim/build.py:766-892): every
tensor-parallel-sharded Muon matrix is brought to its canonical orientation (rows <= columns).  If the long side is
the split one ("direct"), the left Gram ``X X^T`` contracts over the split side, so it is the sum of the ranks'
local Grams.  If the short side is split, either the shards are exchanged first so that the long side becomes the
split one ("exchange": an all-to-all before and after the iteration), or the right Gram ``X^T X`` is used, which
contracts over the split short side ("large_gram": no exchange, a larger Gram).  The global Frobenius norm is an
fp32 reduction.  Leaves that share an execution are packed into buckets of at most 32 MiB of bf16 Gram payload and
each bucket does ONE reduction per Newton-Schulz step for all its Grams.

How it runs here: the local Grams of a bucket are written by the tcgen05 GEMM as fp32 straight into one packed
buffer inside a symmetric arena of the tensor-parallel group; one kernel per step sums the ranks' copies of that
buffer (NVLink peer loads in a fixed rank order, or ``multimem.ld_reduce`` through the switch) into a local buffer;
the polynomial and the apply products are batched tcgen05 GEMMs over the leaves of equal shape.  The norm reduction
rides in the first step's packed buffer: the first Gram is formed from the unnormalised shards and divided by the
squared norm afterwards.  On CPU (gloo) and for fp32 the same schedule runs on ``torch.distributed`` collectives and
plain matrix products, which is also the test oracle's transport.
"""

from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Callable

import torch
import torch.distributed as dist

from research_b200.errors import ContractError
from research_b200.optim import orthogonalize as orth

GRAM_BUCKET_MAX_BYTES = 32 * 1024 * 1024
EXECUTIONS = ("duplicated", "distributed_direct", "distributed_exchange", "distributed_large_gram")


@dataclass(frozen=True)
class MuonLeafPlan:
    """Static plan of one tensor-parallel-sharded Muon matrix."""

    name: str
    logical_shape: tuple[int, int]      # global [in, out] shape of the reference layout
    tp_partition_dim: int               # logical axis that the tensor-parallel group splits
    transpose_for_shape: bool           # canonical orientation = logical transposed (rows > columns)
    canonical_tp_dim: int               # split axis in canonical orientation: 1 = long side, 0 = short side
    requested_mode: str
    execution: str
    fallback_reason: str | None
    bucket_id: int
    weight_decay: bool

    @property
    def gram_dimension(self) -> int:
        short, long = min(self.logical_shape), max(self.logical_shape)
        return long if self.execution == "distributed_large_gram" else short

    def to_dict(self) -> dict[str, Any]:
        return {"path": self.name, "logical_shape": list(self.logical_shape),
                "tp_partition_dim": self.tp_partition_dim, "transpose_for_shape": self.transpose_for_shape,
                "canonical_tp_dim": self.canonical_tp_dim, "requested_mode": self.requested_mode,
                "execution": self.execution, "fallback_reason": self.fallback_reason, "bucket_id": self.bucket_id,
                "gram_dimension": self.gram_dimension, "weight_decay": self.weight_decay}


def resolve_execution(requested_mode: str, canonical_tp_dim: int, logical_shape: tuple[int, int],
                      tp_size: int) -> tuple[str, str | None]:
    """Execution for one leaf (reference rule: optim/build.py:866-882; ``large_gram`` is requested explicitly)."""

    if requested_mode == "duplicated":
        return "duplicated", None
    if requested_mode not in ("distributed", "distributed_large_gram"):
        raise ContractError(f"unsupported Muon TP mode {requested_mode!r}")
    if canonical_tp_dim == 1:
        return "distributed_direct", None
    if requested_mode == "distributed_large_gram":
        return "distributed_large_gram", None
    if max(logical_shape) % tp_size:
        return "duplicated", "exchange_long_dimension_not_divisible_by_tp"
    return "distributed_exchange", None


def assign_bucket_ids(plans: tuple[MuonLeafPlan, ...]) -> tuple[MuonLeafPlan, ...]:
    """Greedy, deterministic buckets of compatible leaves with at most 32 MiB of bf16 Gram payload each."""

    states: dict[tuple, tuple[int, int]] = {}
    next_id = 0
    assigned: dict[str, MuonLeafPlan] = {}
    for plan in sorted(plans, key=lambda p: p.name):
        if plan.execution == "duplicated":
            assigned[plan.name] = plan
            continue
        key = (plan.execution, plan.transpose_for_shape, plan.canonical_tp_dim)
        payload = plan.gram_dimension * plan.gram_dimension * 2
        bucket, used = states.get(key, (-1, 0))
        if bucket < 0 or used + payload > GRAM_BUCKET_MAX_BYTES:
            bucket, used = next_id, 0
            next_id += 1
        states[key] = (bucket, used + payload)
        assigned[plan.name] = replace(plan, bucket_id=bucket)
    return tuple(assigned[p.name] for p in plans)


def build_muon_execution_plans(assignments, metadata, *, tp_size: int,
                               requested_mode: str) -> tuple[MuonLeafPlan, ...]:
    """Plans for every ``dist_muon`` route (rank-2 leaves whose ``matrix_axis`` is the tensor-parallel axis)."""

    shapes = {m.name: tuple(m.shape) for m in metadata}
    plans = []
    for a in assignments:
        if a.backend != "dist_muon":
            continue
        shape = shapes.get(a.name)
        if shape is None or len(shape) != 2:
            raise ContractError(f"distributed Muon execution plan for {a.name!r} requires a rank-2 logical shape")
        rows, cols = int(shape[0]), int(shape[1])
        axis = int(a.matrix_axis)
        transpose = rows > cols
        canonical = 1 - axis if transpose else axis
        execution, reason = resolve_execution(requested_mode, canonical, (rows, cols), tp_size)
        plans.append(MuonLeafPlan(a.name, (rows, cols), axis, transpose, canonical, requested_mode, execution, reason,
                                  -1, bool(a.weight_decay)))
    return assign_bucket_ids(tuple(plans))


def summarize_plans(plans: tuple[MuonLeafPlan, ...]) -> dict[str, Any]:
    """Counts per execution and per bucket for ``diagnostics/runtime.json`` and the resume fingerprint."""

    by_exec: dict[str, int] = {}
    buckets: dict[int, dict[str, Any]] = {}
    for p in plans:
        by_exec[p.execution] = by_exec.get(p.execution, 0) + 1
        if p.bucket_id >= 0:
            b = buckets.setdefault(p.bucket_id, {"bucket_id": p.bucket_id, "execution": p.execution, "leaves": 0,
                                                 "gram_payload_bytes": 0})
            b["leaves"] += 1
            b["gram_payload_bytes"] += p.gram_dimension * p.gram_dimension * 2
    return {"leaf_count": len(plans), "execution_counts": dict(sorted(by_exec.items())),
            "gram_bucket_max_bytes": GRAM_BUCKET_MAX_BYTES, "buckets": [buckets[k] for k in sorted(buckets)],
            "leaves": [p.to_dict() for p in plans]}


# ---------------------------------------------------------------------------------------------------
# transport of the packed reductions
# ---------------------------------------------------------------------------------------------------
class TorchReducer:
    """Packed fp32 sums over the group with ``torch.distributed`` (CPU / gloo, and the fallback on CUDA)."""

    def __init__(self, group):
        self.group = group
        self.reductions = 0

    def buffer(self, numel: int, device: torch.device) -> torch.Tensor:
        return torch.empty(numel, dtype=torch.float32, device=device)

    def all_reduce(self, packed: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(packed, group=self.group)
        self.reductions += 1
        return packed

    def all_to_all(self, out: torch.Tensor, inp: torch.Tensor) -> None:
        """``inp[r]`` goes to rank ``r``; ``out[r]`` comes from rank ``r`` (bf16 travels as raw bytes)."""

        inp = inp.contiguous()
        if inp.dtype == torch.bfloat16:                      # bytes travel unchanged; gloo has no bf16 all-to-all
            out, inp = out.view(torch.uint8), inp.view(torch.uint8)
        dist.all_to_all_single(out, inp, group=self.group)


class ArenaReducer(TorchReducer):
    """The same sums as one peer-memory kernel per call: the packed buffer lives in a symmetric arena of the group,
    every rank reads all ranks' copies (NVLink peer loads in rank order, or ``multimem.ld_reduce``) and writes the
    total into a local buffer.  Two input slots alternate, so the next step's Grams can be written while a slow peer
    still reads the previous ones."""

    CHANNEL = 7

    def __init__(self, group, capacity: int, device: torch.device):
        super().__init__(group)
        from research_b200.parallel.symmetric import SymmetricArena

        self.capacity = int(capacity)
        self.arena = SymmetricArena(group, 2 * self.capacity * 4 + 8192, device=device, tag="muon-gram")
        self.slots = [self.arena.carve(self.capacity, torch.float32) for _ in range(2)]
        self.out = torch.empty(self.capacity, dtype=torch.float32, device=device)
        self.turn = 0

    def buffer(self, numel: int, device: torch.device) -> torch.Tensor:
        if numel > self.capacity:
            # a single Gram larger than a slot (a bucket never holds more than one such matrix): the library
            # all-reduce takes it, in its own buffer
            self._oversize = super().buffer(numel, device)
            return self._oversize
        self.turn ^= 1
        return self.slots[self.turn][0][:numel]

    def all_reduce(self, packed: torch.Tensor) -> torch.Tensor:
        oversize = getattr(self, "_oversize", None)
        if oversize is not None and packed.data_ptr() == oversize.data_ptr():
            self._oversize = None
            return super().all_reduce(packed)
        n = packed.numel()
        pad = (-n) % 4
        tensor, offset = self.slots[self.turn]
        if packed.data_ptr() != tensor.data_ptr():
            raise ContractError("ArenaReducer.all_reduce expects the buffer handed out by buffer()")
        if pad:
            tensor[n:n + pad].zero_()
        self.arena.reduce_scatter(offset, n + pad, out=self.out[:n + pad], channel=self.CHANNEL)
        self.reductions += 1
        return self.out[:n]


# ---------------------------------------------------------------------------------------------------
# the iteration
# ---------------------------------------------------------------------------------------------------
def _native(x: torch.Tensor) -> bool:
    return orth._native_ok(x)


def _gram(x: torch.Tensor, right: bool, out: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 Gram of a bf16 / fp32 stack ``[n, r, c]``: ``X X^T`` (left) or ``X^T X`` (right)."""

    if _native(x):
        from research_b200.ops import native

        if right:
            return native.gemm(x, x, trans_a=True, trans_b=False, out=out, out_dtype=torch.float32)
        return native.gemm(x, x, trans_b=True, out=out, out_dtype=torch.float32)
    xf = x.float()
    g = xf.transpose(-1, -2) @ xf if right else xf @ xf.transpose(-1, -2)
    if out is not None:
        out.copy_(g)
        return out
    return g


def _step(x: torch.Tensor, gram: torch.Tensor, right: bool, coeff) -> torch.Tensor:
    """``X <- a X + (b G + c G^2) X`` (left) or ``a X + X (b G + c G^2)`` (right); ``gram`` in the dtype of ``x``."""

    a, b, c = coeff
    if _native(x):
        from research_b200.ops import native

        lhs = native.affine_identity(gram, b, c)                         # b I + c G
        q = native.gemm(lhs, gram, trans_b=True)                         # G symmetric: (b I + c G) G = b G + c G^2
        native.affine_identity(q, a, 1.0, out=q)                         # + a I
        return native.gemm(x, q, trans_b=True) if right else native.gemm(q, x, trans_b=False)
    poly = b * gram + c * (gram @ gram)
    return a * x + (x @ poly if right else poly @ x)


def bucketed_distributed_zeropower(values: list[torch.Tensor], plans: list[MuonLeafPlan], storage_axes: list[int],
                                   group, reducer: TorchReducer | None = None,
                                   compute_dtype: torch.dtype = torch.bfloat16) -> list[torch.Tensor]:
    """Newton-Schulz on the local shards of one bucket; one packed reduction per step for the whole bucket.

    ``values[i]``: this rank's shard of leaf ``i`` in STORAGE orientation (``[out, in]`` = logical transposed),
    split along ``storage_axes[i]``.  Orthogonalisation commutes with transposition, so the iteration works on
    whichever orientation makes the split side the contraction: the result has the shape of the input shard."""

    if not values or len(values) != len(plans) or len(values) != len(storage_axes):
        raise ContractError("distributed Muon bucket requires equally sized non-empty values, plans and axes")
    execution = plans[0].execution
    if execution not in EXECUTIONS[1:] or any(p.execution != execution for p in plans):
        raise ContractError(f"distributed Muon bucket contains incompatible executions: {[p.execution for p in plans]}")
    reducer = reducer or TorchReducer(group)
    world = dist.get_world_size(group)
    dev = values[0].device
    # orientation in which the iteration runs: rows = the side that stays whole, columns = contraction side
    # direct / exchange: left Gram over the long side; large_gram: right Gram over the (short) split side
    work: list[torch.Tensor] = []
    flips: list[bool] = []
    for v, axis in zip(values, storage_axes):
        x = v.to(compute_dtype)
        if execution == "distributed_large_gram":
            flip = axis == 1                 # bring the split side to dim 0 (rows): Gram X^T X contracts over it
        elif execution == "distributed_direct":
            flip = axis == 0                 # bring the split (long) side to dim 1: Gram X X^T contracts over it
        else:                                # exchange: the split side is the short one; put it on dim 0 first
            flip = axis == 1
        work.append(x.transpose(0, 1).contiguous() if flip else x.contiguous())
        flips.append(flip)
    right = execution == "distributed_large_gram"
    # ---- norms: local sums of squares ride in the first packed reduction ------------------------------------
    sq_local = torch.stack([w.float().pow(2).sum() for w in work])
    if execution == "distributed_exchange":
        # [rows/world, cols] -> [rows, cols/world]: every rank sends column block r of its rows to rank r
        exchanged = []
        for w in work:
            r_loc, cols = w.shape
            if cols % world:
                raise ContractError("distributed_exchange needs the long side divisible by the group size")
            send = w.view(r_loc, world, cols // world).transpose(0, 1).contiguous()       # [world, r_loc, cols/world]
            recv = torch.empty_like(send)
            reducer.all_to_all(recv, send)
            exchanged.append(recv.reshape(world * r_loc, cols // world))
        work = exchanged
    # ---- leaves of equal working shape are stacked: batched GEMMs ---------------------------------------------
    groups: dict[tuple[int, int], list[int]] = {}
    for i, w in enumerate(work):
        groups.setdefault(tuple(w.shape), []).append(i)
    stacks = {shape: torch.stack([work[i] for i in idx]) for shape, idx in groups.items()}
    gram_dim = {shape: (shape[1] if right else shape[0]) for shape in stacks}
    sizes = {shape: len(idx) * gram_dim[shape] ** 2 for shape, idx in groups.items()}
    total = sum(sizes.values())
    coeffs = (orth.MUON_NS_COEFFICIENTS,) * orth.MUON_NS_STEPS
    inv_norm = None
    for step, coeff in enumerate(coeffs):
        extra = len(work) if step == 0 else 0
        packed = reducer.buffer(total + extra, dev)
        at = 0
        for shape, stack in stacks.items():
            n, d = stack.shape[0], gram_dim[shape]
            _gram(stack, right, out=packed[at:at + sizes[shape]].view(n, d, d))
            at += sizes[shape]
        if step == 0:
            packed[total:total + extra].copy_(sq_local)
        summed = reducer.all_reduce(packed)
        if step == 0:
            norms = summed[total:total + extra].sqrt().clamp_min(orth.MUON_NS_EPS)
            inv_norm = (1.0 / norms)
        at = 0
        for shape, idx in groups.items():
            n, d = len(idx), gram_dim[shape]
            gram = summed[at:at + sizes[shape]].view(n, d, d)
            at += sizes[shape]
            stack = stacks[shape]
            if step == 0:                                   # normalise now: X / |X|, G / |X|^2
                s = inv_norm[idx].view(n, 1, 1)
                gram = gram * (s * s)
                stack = (stack.float() * s).to(compute_dtype)
            stacks[shape] = _step(stack, gram.to(compute_dtype).contiguous(), right, coeff)
    # ---- back to the input layout -----------------------------------------------------------------------------
    out: list[torch.Tensor | None] = [None] * len(values)
    for shape, idx in groups.items():
        for k, i in enumerate(idx):
            out[i] = stacks[shape][k]
    if execution == "distributed_exchange":
        for i, x in enumerate(out):
            rows, c_loc = x.shape
            send = x.view(world, rows // world, c_loc).contiguous()                         # row block r -> rank r
            recv = torch.empty_like(send)
            reducer.all_to_all(recv, send)
            out[i] = recv.transpose(0, 1).reshape(rows // world, world * c_loc)
    results = []
    for x, flip, v in zip(out, flips, values):
        x = x.transpose(0, 1) if flip else x
        results.append(x.contiguous().to(v.dtype))
    return results
