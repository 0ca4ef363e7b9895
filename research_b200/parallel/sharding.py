"""Parameter / gradient / optimizer-state placement for one rank.

The reference expresses placement as per-leaf ``NamedSharding`` s that XLA turns into collectives
(src/jaxtitan/mesh/sharding.py:140-340).  Here placement is explicit and laid out for 180 GB of HBM per GPU:

* **compute arena** - one flat tensor in the compute dtype holding every local parameter; the model's
  ``nn.Parameter`` s are views into it.  It stays resident for the whole step (no per-layer re-gather).
* **gradient arena** - one flat fp32 tensor; every parameter's ``main_grad`` is a view.  Backward kernels add into
  it; the data-parallel reduction is one collective per section.
* **master / optimizer state** - fp32.  In ``ddp`` mode every rank keeps all of it; in ``zero2`` and ``fsdp``
  modes each section is split over the ``fsdp`` axis: element ranges for AdamW sections, whole matrices (balanced
  by FLOPs) for Muon / Dion sections, so each rank updates only what it owns and the updated compute weights are
  all-gathered back into the arena.

Sections group parameters that share an optimizer backend and the same set of gradient-reduction groups.
"""

from __future__ import annotations

import math
import os
import re
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.distributed as dist

from research_b200.errors import ContractError
from research_b200.models.build import NORM_TAGS, ROUTED_EXPERT_TAGS, ModelBuildResult, ParamMeta
from research_b200.parallel.mesh import MeshContext

ALIGN = 256  # elements; keeps every parameter 512-byte (bf16) / 1 KiB (fp32) aligned inside the arenas
BUCKET_CHANNEL = 6          # flag channel of the bucketed gradient reduction that overlaps the backward pass
_LAYER_RE = re.compile(r"(?:^|\.)layers\.(\d+)\.")


def layer_of(name: str) -> int:
    """Index of the transformer block a parameter belongs to, or -1 (embedding, final norm, lm_head)."""

    m = _LAYER_RE.search(name)
    return int(m.group(1)) if m else -1


def _ceil_to(n: int, m: int) -> int:
    return (n + m - 1) // m * m


@dataclass
class StorageEntry:
    """One physical ``nn.Parameter`` (possibly holding several logical parameters)."""

    name: str
    param: torch.nn.Parameter
    metas: list[ParamMeta]
    backend: str                    # "adamw" | "muon" | "dion2" | "frozen"
    reduce_axes: tuple[str, ...]    # mesh axes over which gradients are summed
    shard_axis: str | None          # mesh axis over which optimizer state is split (None = replicated)
    offset: int = 0                 # element offset inside the arenas
    numel: int = 0
    owner: int = 0                  # owning rank along shard_axis (matrix sections)
    decay: bool = True              # AdamW entries: decoupled weight decay applies (the route's ``weight_decay`` flag)

    @property
    def is_expert(self) -> bool:
        return any(m.tag in ROUTED_EXPERT_TAGS for m in self.metas)


@dataclass
class Section:
    key: tuple
    backend: str
    reduce_axes: tuple[str, ...]
    shard_axis: str | None
    entries: list[StorageEntry] = field(default_factory=list)
    start: int = 0
    length: int = 0                 # padded so that it splits evenly over the shard axis
    owner_block: int = 0            # matrix sections: elements per owner block
    decay: bool = True              # AdamW sections: whether weight decay applies to every element of the section
    # matrix sections split over owners: layer -> element range of that layer's matrices inside THIS rank's owner
    # block (entries of a block are laid out in backward order, so every layer is one contiguous range)
    bucket_ranges: dict = field(default_factory=dict)
    bucket_layers: tuple = ()       # all layers that have matrices in this section, in backward order (every rank)

    def local_range(self, shard_rank: int, shard_size: int) -> tuple[int, int]:
        if self.shard_axis is None or shard_size == 1:
            return self.start, self.start + self.length
        per = self.length // shard_size
        return self.start + shard_rank * per, self.start + (shard_rank + 1) * per


class ParamStore:
    def __init__(self, result: ModelBuildResult, mesh: MeshContext, *, mode: str, compute_dtype: torch.dtype,
                 backend_of: dict[str, str], ep_axis: str | None = None, decay_of: dict[str, bool] | None = None):
        self.result = result
        self.mesh = mesh
        self.mode = mode
        self.compute_dtype = compute_dtype
        self.device = next(result.model.parameters()).device
        self.ep_axis = ep_axis
        by_storage: dict[str, list[ParamMeta]] = {}
        for meta in result.metadata:
            by_storage.setdefault(meta.storage, []).append(meta)
        named = dict(result.model.named_parameters())
        self.entries: list[StorageEntry] = []
        tp_active = result.execution.tp_size > 1
        for name, metas in by_storage.items():
            param = named[name]
            backends = {backend_of.get(m.name, "adamw") for m in metas}
            if not param.requires_grad:
                backend = "frozen"
            elif len(backends) != 1:
                raise ContractError(f"logical parameters fused in {name} route to different optimizers: {backends}")
            else:
                backend = backends.pop()
            is_expert = any(m.tag in ROUTED_EXPERT_TAGS for m in metas)
            axes = []
            for axis in ("data", "fsdp", "cp"):
                if mesh.size(axis) > 1 and not (is_expert and axis == ep_axis):
                    axes.append(axis)
            replicated_over_tp = all(m.tp_axis is None for m in metas) and not is_expert
            if tp_active and replicated_over_tp and result.execution.sp:
                axes.append("tp")  # sequence-parallel regions see only a slice of the tokens
            shard_axis = None
            if mode in ("zero2", "fsdp") and mesh.size("fsdp") > 1 and not (is_expert and ep_axis == "fsdp"):
                shard_axis = "fsdp"
            decays = {bool((decay_of or {}).get(m.name, True)) for m in metas}
            if backend == "adamw" and len(decays) != 1:
                raise ContractError(f"logical parameters fused in {name} disagree on weight decay")
            self.entries.append(StorageEntry(name, param, metas, backend, tuple(axes), shard_axis,
                                             numel=param.numel(), decay=decays.pop() if backend == "adamw" else True))
        self._layout()
        self._materialise()

    # ---- layout ----------------------------------------------------------------------------------
    def _layout(self) -> None:
        sections: dict[tuple, Section] = {}
        order = {"adamw": 0, "muon": 1, "dion2": 2, "frozen": 3}
        tp_sharded = lambda e: any(m.tp_axis is not None for m in e.metas)  # noqa: E731
        for e in sorted(self.entries, key=lambda e: (order[e.backend], e.reduce_axes, str(e.shard_axis),
                                                     e.is_expert, tp_sharded(e), not e.decay)):
            # expert and tensor-parallel-sharded parameters are disjoint across their axis, the rest is replicated:
            # they must not share a section because norms are summed per section; AdamW parameters with and without
            # weight decay get sections of their own because the kernel takes one decay per launch
            key = (e.backend, e.reduce_axes, e.shard_axis, e.is_expert, tp_sharded(e), e.decay)
            sections.setdefault(key, Section(key, e.backend, e.reduce_axes, e.shard_axis,
                                             decay=e.decay)).entries.append(e)
        cursor = 0
        self.sections: list[Section] = []
        for sec in sections.values():
            n_shard = self.mesh.size(sec.shard_axis) if sec.shard_axis else 1
            sec.start = cursor
            if sec.backend in ("muon", "dion2") and n_shard > 1:
                # whole matrices per owner, balanced by orthogonalisation cost; one equal-size block per owner
                loads = [0.0] * n_shard
                blocks: list[list[StorageEntry]] = [[] for _ in range(n_shard)]
                for e in sorted(sec.entries, key=lambda e: -_ns_cost(e.param.shape)):
                    owner = min(range(n_shard), key=lambda r: loads[r])
                    loads[owner] += _ns_cost(e.param.shape)
                    blocks[owner].append(e)
                    e.owner = owner
                sizes = [sum(_ceil_to(e.numel, ALIGN) for e in b) for b in blocks]
                sec.owner_block = _ceil_to(max(sizes) if sizes else 0, ALIGN)
                me = self.mesh.coord(sec.shard_axis)
                for owner, b in enumerate(blocks):
                    off = sec.start + owner * sec.owner_block
                    # backward order inside a block: the gradients of a layer become final together, and the
                    # reduction of that contiguous range can start while earlier layers are still in backward
                    for e in sorted(b, key=lambda e: (-layer_of(e.name), e.name)):
                        e.offset = off
                        if owner == me:
                            lo_hi = sec.bucket_ranges.get(layer_of(e.name))
                            end = off + _ceil_to(e.numel, ALIGN)
                            sec.bucket_ranges[layer_of(e.name)] = (off, end) if lo_hi is None else (lo_hi[0], end)
                        off += _ceil_to(e.numel, ALIGN)
                sec.bucket_layers = tuple(sorted({layer_of(e.name) for e in sec.entries}, reverse=True))
                sec.length = sec.owner_block * n_shard
            else:
                off = sec.start
                for e in sec.entries:
                    e.offset = off
                    off += _ceil_to(e.numel, ALIGN)
                sec.length = _ceil_to(off - sec.start, ALIGN * n_shard)
            cursor = sec.start + sec.length
            self.sections.append(sec)
        self.total = cursor

    def _symmetric_group(self):
        """The process group whose ranks exchange shards through peer memory, or None (NCCL / gloo path).

        Used when the tensors live on CUDA, exactly one mesh axis shards the store, and the environment does not
        switch it off (``RESEARCH_B200_PEER_COLLECTIVES=0``)."""

        if self.device.type != "cuda" or os.environ.get("RESEARCH_B200_PEER_COLLECTIVES", "1") == "0":
            return None
        axes = {sec.shard_axis for sec in self.sections if sec.shard_axis is not None and sec.backend != "frozen"}
        if len(axes) != 1:
            return None
        axis = axes.pop()
        group = self.mesh.group(axis)
        if group is None or self.mesh.size(axis) < 2 or self.mesh.size(axis) > 8:
            return None
        return group

    def _materialise(self) -> None:
        dev = self.device
        self.arena = None
        group = self._symmetric_group()
        if group is not None:
            from research_b200.parallel.symmetric import SymmetricArena, build_collectively

            esize = torch.empty((), dtype=self.compute_dtype).element_size()
            self.arena = build_collectively(
                group, lambda: SymmetricArena(group, self.total * (4 + esize) + 8192, device=dev, tag="params"),
                "symmetric parameter arena")
        if self.arena is not None:
            self.grad_arena, self._grad_off = self.arena.carve(self.total, torch.float32)
            self.compute_arena, self._compute_off = self.arena.carve(self.total, self.compute_dtype)
        else:
            self.compute_arena = torch.zeros(self.total, dtype=self.compute_dtype, device=dev)
            self.grad_arena = torch.zeros(self.total, dtype=torch.float32, device=dev)
        # bucketed reduction on a side stream (see begin_backward_overlap)
        self._overlap = (self.arena is not None and os.environ.get("RESEARCH_B200_OVERLAP_REDUCE", "1") != "0")
        self._comm_stream = torch.cuda.Stream(dev, priority=-1) if self._overlap else None
        self._bucket_ctas = int(os.environ.get("RESEARCH_B200_REDUCE_CTAS", "48"))
        self._pending: list[tuple[Section, int]] = []
        self._armed = False
        separate_master = self.compute_dtype != torch.float32
        for sec in self.sections:
            lo, hi = self.local_master_range(sec)
            sec.master = torch.zeros(hi - lo, dtype=torch.float32, device=dev) if separate_master else None
        for e in self.entries:
            sec = self.section_of(e)
            fp32 = e.param.data.detach().to(torch.float32).reshape(-1)
            view = self.compute_arena[e.offset:e.offset + e.numel]
            view.copy_(fp32)
            if separate_master:
                lo, hi = self.local_master_range(sec)
                a, b = max(e.offset, lo), min(e.offset + e.numel, hi)
                if b > a:
                    sec.master[a - lo:b - lo].copy_(fp32[a - e.offset:b - e.offset])
            e.param.data = view.view(e.param.shape)
            e.param.main_grad = self.grad_arena[e.offset:e.offset + e.numel].view(e.param.shape)
        if not separate_master:
            for sec in self.sections:
                lo, hi = self.local_master_range(sec)
                sec.master = self.compute_arena[lo:hi]
        self.result.model.compute_dtype = self.compute_dtype

    # ---- queries ---------------------------------------------------------------------------------
    def section_of(self, e: StorageEntry) -> Section:
        for sec in self.sections:
            if e in sec.entries:
                return sec
        raise ContractError(f"storage entry {e.name} is not in any section")

    def shard_coords(self, sec: Section) -> tuple[int, int]:
        if sec.shard_axis is None:
            return 0, 1
        return self.mesh.coord(sec.shard_axis), self.mesh.size(sec.shard_axis)

    def local_master_range(self, sec: Section) -> tuple[int, int]:
        r, n = self.shard_coords(sec)
        return sec.local_range(r, n)

    def owns(self, sec: Section, e: StorageEntry) -> bool:
        r, n = self.shard_coords(sec)
        return n == 1 or sec.backend not in ("muon", "dion2") or e.owner == r

    def master_view(self, sec: Section, e: StorageEntry) -> torch.Tensor | None:
        """fp32 master values of a whole storage entry, if this rank holds all of it."""

        lo, hi = self.local_master_range(sec)
        if e.offset < lo or e.offset + e.numel > hi:
            return None
        return sec.master[e.offset - lo:e.offset - lo + e.numel].view(e.param.shape)

    # ---- gradient plumbing -------------------------------------------------------------------------
    def zero_grads(self) -> None:
        self.grad_arena.zero_()

    def collect_autograd_grads(self) -> None:
        """Reference path: fold ``.grad`` (filled by ordinary autograd) into the gradient arena."""

        for e in self.entries:
            g = e.param.grad
            if g is not None:
                e.param.main_grad.add_(g.to(torch.float32))
                e.param.grad = None

    # ---- bucketed reduction that overlaps the backward pass ----------------------------------------------
    def _bucketed(self, sec: Section) -> bool:
        return (self._overlap and sec.backend in ("muon", "dion2") and sec.shard_axis is not None and
                sec.shard_axis in sec.reduce_axes and self.mesh.size(sec.shard_axis) > 1 and bool(sec.bucket_layers))

    def begin_backward_overlap(self) -> None:
        """Arm the per-layer reduction for the backward pass that follows (the last microbatch of a step).

        Matrix sections that are split over owners keep each layer's matrices contiguous inside an owner's block.
        When the model reports that the backward pass of layer ``i`` has been issued (``on_layer_backward``), the
        reduce-scatter of that layer's ranges is launched on a high-priority side stream behind an event of the
        compute stream, with a capped grid, so that it runs over NVLink while earlier layers are still in backward.
        ``reduce_gradients`` launches what is left and joins the streams."""

        self._pending = [(sec, layer) for sec in self.sections if self._bucketed(sec) for layer in sec.bucket_layers]
        self._pending.sort(key=lambda item: -item[1])           # backward order, the same on every rank
        self._armed = bool(self._pending)

    def on_layer_backward(self, layer: int) -> None:
        """Autograd hook of the model: every kernel of layer ``layer``'s backward pass is on the compute stream."""

        if not self._armed:
            return
        ready = [item for item in self._pending if item[1] >= layer]
        if ready:
            self._launch_buckets(ready)
            self._pending = [item for item in self._pending if item[1] < layer]

    def _launch_buckets(self, items: list[tuple[Section, int]]) -> None:
        comm = self._comm_stream
        comm.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(comm):
            for sec, layer in items:
                a, b = sec.bucket_ranges.get(layer, (sec.start, sec.start))       # this rank may own nothing here
                self.arena.reduce_scatter(self._grad_off + 4 * a, b - a, channel=BUCKET_CHANNEL,
                                          max_ctas=self._bucket_ctas)
                for axis in sec.reduce_axes:
                    group = self.mesh.group(axis)
                    if axis != sec.shard_axis and group is not None and b > a:
                        dist.all_reduce(self.grad_arena[a:b], group=group)

    def reduce_gradients(self) -> None:
        """Sum gradients over every replica axis; sharded sections end with only the local range valid."""

        bucketed = set()
        if self._armed:
            if self._pending:
                self._launch_buckets(self._pending)
                self._pending = []
            bucketed = {id(sec) for sec in self.sections if self._bucketed(sec)}
        for sec in self.sections:
            if sec.backend == "frozen" or sec.length == 0 or id(sec) in bucketed:
                continue
            buf = self.grad_arena[sec.start:sec.start + sec.length]
            for axis in sec.reduce_axes:
                group = self.mesh.group(axis)
                if group is None:
                    continue
                if axis == sec.shard_axis:
                    n, r = self.mesh.size(axis), self.mesh.coord(axis)
                    per = sec.length // n
                    out = buf[r * per:(r + 1) * per]
                    if self.arena is not None:
                        # one kernel: pull the peers' copies of the local slice over NVLink and sum in rank order
                        self.arena.reduce_scatter(self._grad_off + 4 * (sec.start + r * per), per, channel=0)
                    elif buf.is_cuda:
                        dist.reduce_scatter_tensor(out, buf, group=group)
                    else:
                        dist.all_reduce(buf, group=group)
                else:
                    dist.all_reduce(buf, group=group)
        if self._armed:
            torch.cuda.current_stream(self.device).wait_stream(self._comm_stream)
            self._armed = False

    def gather_compute_weights(self) -> None:
        """After the optimizer step: every rank gets the updated compute weights of sharded sections."""

        for sec in self.sections:
            if sec.shard_axis is None or sec.backend == "frozen":
                continue
            group = self.mesh.group(sec.shard_axis)
            if group is None:
                continue
            n, r = self.shard_coords(sec)[1], self.shard_coords(sec)[0]
            buf = self.compute_arena[sec.start:sec.start + sec.length]
            per = sec.length // n
            if self.arena is not None:
                esize = buf.element_size()
                self.arena.all_gather(self._compute_off + esize * sec.start, per * esize, channel=1)
            else:
                dist.all_gather_into_tensor(buf, buf[r * per:(r + 1) * per].clone(), group=group)

    def describe(self) -> dict[str, Any]:
        return {
            "mode": self.mode,
            "compute_dtype": str(self.compute_dtype).replace("torch.", ""),
            "arena_elements": self.total,
            "sections": [
                {"backend": s.backend, "reduce_axes": list(s.reduce_axes), "shard_axis": s.shard_axis,
                 "elements": s.length, "parameters": len(s.entries)}
                for s in self.sections
            ],
        }


def _ns_cost(shape) -> float:
    """Relative Newton-Schulz cost of a (stack of) matrices: ~ batch * (2 m^2 n + m^3), m <= n."""

    dims = list(shape)
    batch = 1
    if len(dims) == 3:
        batch, dims = dims[0], dims[1:]
    if len(dims) != 2:
        return float(math.prod(shape))
    m, n = min(dims), max(dims)
    return float(batch) * (2.0 * m * m * n + float(m) ** 3)
