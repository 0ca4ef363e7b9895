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

``parallelism.fsdp_resident = false`` (ZeRO-3): the compute copy of a sharded section is kept only where it is owned
(each rank its element range or its owner block, 1/N of the section).  The weights of one transformer layer are
brought from their owners into one of two layer buffers right before the layer runs, forward and backward, over
NVLink peer loads on a side stream while the previous layer computes (NCCL / gloo collectives off CUDA); embeddings,
the final norm and the lm_head are gathered once per step.  The reference shards every tagged parameter along its
``fsdp_axis`` and lets XLA gather it at use (src/jaxtitan/mesh/sharding.py:445-501).
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
    rest_start: int = 0             # weights sharded at rest: where this rank's part of the section starts

    def local_range(self, shard_rank: int, shard_size: int) -> tuple[int, int]:
        if self.shard_axis is None or shard_size == 1:
            return self.start, self.start + self.length
        per = self.length // shard_size
        return self.start + shard_rank * per, self.start + (shard_rank + 1) * per


class ParamStore:
    def __init__(self, result: ModelBuildResult, mesh: MeshContext, *, mode: str, compute_dtype: torch.dtype,
                 backend_of: dict[str, str], ep_axis: str | None = None, decay_of: dict[str, bool] | None = None,
                 resident: bool = True):
        self.result = result
        self.mesh = mesh
        self.mode = mode
        self.compute_dtype = compute_dtype
        self.device = next(result.model.parameters()).device
        self.ep_axis = ep_axis
        self.resident = bool(resident)
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
            head_local = any(m.tag in ("attention_q_norm", "attention_k_norm") for m in metas)
            if tp_active and replicated_over_tp and (result.execution.sp or head_local):
                # sequence-parallel regions see only a slice of the tokens; the per-head q/k norm scales see only
                # this rank's heads whether or not the sequence is split
                axes.append("tp")
            if tp_active and is_expert and result.execution.sp and "tp" not in axes:
                # routed experts are not split over tp: every tensor-parallel rank routes its own slice of the tokens
                # through the same expert weights, so their gradients are partial sums over that axis
                axes.append("tp")
            shard_axis = None
            # parameters that no optimizer moves (the routers' balance bias) keep their whole fp32 value on every
            # rank: whatever updates them does so identically everywhere and needs no gather to read them
            if mode in ("zero2", "fsdp") and mesh.size("fsdp") > 1 and not (is_expert and ep_axis == "fsdp") \
                    and backend != "frozen":
                shard_axis = "fsdp"
            decays = {bool((decay_of or {}).get(m.name, True)) for m in metas}
            if backend == "adamw" and len(decays) != 1:
                raise ContractError(f"logical parameters fused in {name} disagree on weight decay")
            self.entries.append(StorageEntry(name, param, metas, backend, tuple(axes), shard_axis,
                                             numel=param.numel(), decay=decays.pop() if backend == "adamw" else True))
        self._layout()
        if not self.resident and not any(self._sharded(sec) for sec in self.sections):
            self.resident = True            # nothing is split over a shard axis: there is nothing to keep away
        if self.resident:
            self._materialise()
        else:
            self._materialise_sharded()

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
        self._overlap = (self.arena is not None and os.environ.get("RESEARCH_B200_OVERLAP_REDUCE", "0") == "1")
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

    # ---- compute copy: where the optimizer writes it -----------------------------------------------------
    def _sharded(self, sec: Section) -> bool:
        return sec.shard_axis is not None and self.mesh.size(sec.shard_axis) > 1 and sec.backend != "frozen"

    def _section_at(self, offset: int) -> Section:
        for sec in self.sections:
            if sec.start <= offset < sec.start + max(sec.length, 1):
                return sec
        raise ContractError(f"arena offset {offset} is outside every section")

    def shadow(self, a: int, b: int | None = None) -> torch.Tensor:
        """Compute-dtype storage of the arena elements ``[a, b)`` (``b`` omitted: up to the end of what this rank
        holds of that section).  With resident weights that is a slice of the compute arena; with weights sharded
        at rest the range must lie inside what this rank owns."""

        if self.resident:
            return self.compute_arena[a:] if b is None else self.compute_arena[a:b]
        sec = self._section_at(a)
        lo, hi = self.local_master_range(sec) if self._sharded(sec) else (sec.start, sec.start + sec.length)
        end = hi if b is None else b
        if a < lo or end > hi:
            raise ContractError(f"arena range [{a}, {end}) is not held by this rank (it holds [{lo}, {hi}))")
        base = sec.rest_start - lo
        return self.rest[base + a:base + end]

    def write_entry_shadow(self, e: StorageEntry, master: torch.Tensor) -> None:
        """Refresh the compute copy of a whole storage entry from its fp32 master (owner of the entry only)."""

        if self.resident:
            e.param.data.copy_(master)
        else:
            self.shadow(e.offset, e.offset + e.numel).copy_(master.reshape(-1))

    def load_shadow(self, e: StorageEntry, flat: torch.Tensor) -> None:
        """Checkpoint restore: ``flat`` holds the whole entry; keep what this rank stores of it."""

        if self.resident:
            self.compute_arena[e.offset:e.offset + e.numel].copy_(flat)
            return
        sec = self.section_of(e)
        lo, hi = self.local_master_range(sec) if self._sharded(sec) else (sec.start, sec.start + sec.length)
        a, b = max(e.offset, lo), min(e.offset + e.numel, hi)
        if b > a:
            self.shadow(a, b).copy_(flat[a - e.offset:b - e.offset])

    # ---- weights sharded at rest (ZeRO-3) -------------------------------------------------------------------
    def _materialise_sharded(self) -> None:
        dev = self.device
        dtype = self.compute_dtype
        esize = torch.empty((), dtype=dtype).element_size()
        # what every rank keeps: its 1/N of sharded sections, all of the others
        cursor = 0
        for sec in self.sections:
            n = self.mesh.size(sec.shard_axis) if self._sharded(sec) else 1
            sec.rest_start = cursor
            cursor += _ceil_to(sec.length // n, ALIGN)
        rest_total = cursor
        self.arena = None
        group = self._symmetric_group()
        if group is not None:
            from research_b200.parallel.symmetric import SymmetricArena, build_collectively

            self.arena = build_collectively(
                group, lambda: SymmetricArena(group, self.total * 4 + rest_total * esize + 8192, device=dev,
                                              tag="params"), "symmetric parameter arena")
        if self.arena is not None:
            self.grad_arena, self._grad_off = self.arena.carve(self.total, torch.float32)
            self.rest, self._rest_off = self.arena.carve(rest_total, dtype)
        else:
            self.grad_arena = torch.zeros(self.total, dtype=torch.float32, device=dev)
            self.rest = torch.zeros(rest_total, dtype=dtype, device=dev)
        self.compute_arena = None
        # gathered entries: per layer into a layer buffer, the rest (embedding, final norm, lm_head) once per step
        gathered = [e for e in self.entries if self._sharded(self.section_of(e))]
        self._layers = sorted({layer_of(e.name) for e in gathered if layer_of(e.name) >= 0})
        self._layer_entries = {l: sorted((e for e in gathered if layer_of(e.name) == l), key=lambda e: e.offset)
                               for l in self._layers}
        self._extra_entries = sorted((e for e in gathered if layer_of(e.name) < 0), key=lambda e: e.offset)
        self._dst_off: dict[str, int] = {}
        slot_size = 0
        for l, entries in self._layer_entries.items():
            off = 0
            for e in entries:
                self._dst_off[e.name] = off
                off += _ceil_to(e.numel, ALIGN)
            slot_size = max(slot_size, off)
        off = 0
        for e in self._extra_entries:
            self._dst_off[e.name] = off
            off += _ceil_to(e.numel, ALIGN)
        native_path = dev.type == "cuda" and dtype == torch.bfloat16
        # plain autograd keeps references to the weights it saw in forward, so off the native path every layer keeps
        # a buffer of its own for the whole step; the native kernels read the parameter at launch time and two
        # buffers (the layer in use, the layer being fetched) are enough
        self._n_slots = 2 if native_path else max(len(self._layers), 1)
        self._slots = [torch.zeros(max(slot_size, 1), dtype=dtype, device=dev) for _ in range(self._n_slots)]
        self._extras = torch.zeros(max(off, 1), dtype=dtype, device=dev)
        self._slot_layer: list[int | None] = [None] * self._n_slots
        self._gather_stream = torch.cuda.Stream(dev) if dev.type == "cuda" else None
        self._slot_ready = [None] * self._n_slots          # event: the gather into the slot has finished
        self._slot_free = [None] * self._n_slots           # event: the compute that read the slot has been issued
        self._tables: dict[tuple, tuple[torch.Tensor, int]] = {}
        self._overlap = (self.arena is not None and os.environ.get("RESEARCH_B200_OVERLAP_REDUCE", "0") == "1")
        self._comm_stream = torch.cuda.Stream(dev, priority=-1) if self._overlap else None
        self._bucket_ctas = int(os.environ.get("RESEARCH_B200_REDUCE_CTAS", "48"))
        self._pending = []
        self._armed = False
        separate_master = dtype != torch.float32
        for sec in self.sections:
            lo, hi = self.local_master_range(sec)
            sec.master = torch.zeros(hi - lo, dtype=torch.float32, device=dev) if separate_master else None
        for e in self.entries:
            sec = self.section_of(e)
            fp32 = e.param.data.detach().to(torch.float32).reshape(-1)
            lo, hi = self.local_master_range(sec) if self._sharded(sec) else (sec.start, sec.start + sec.length)
            a, b = max(e.offset, lo), min(e.offset + e.numel, hi)
            if b > a:
                self.shadow(a, b).copy_(fp32[a - e.offset:b - e.offset])
                if separate_master:
                    mlo, _ = self.local_master_range(sec)
                    ma, mb = max(e.offset, mlo), min(e.offset + e.numel, self.local_master_range(sec)[1])
                    if mb > ma:
                        sec.master[ma - mlo:mb - mlo].copy_(fp32[ma - e.offset:mb - e.offset])
            if self._sharded(sec):
                # a view of the buffer the values will be fetched into: the shape is right from the start, the
                # contents only while the layer is acquired (or, outside the layers, after the per-step gather)
                layer = layer_of(e.name)
                buf = self._extras if layer < 0 else self._slots[self._slot_for(layer)]
                off = self._dst_off[e.name]
                e.param.data = buf[off:off + e.numel].view(e.param.shape)
            else:
                e.param.data = self.shadow(e.offset, e.offset + e.numel).view(e.param.shape)
            e.param.main_grad = self.grad_arena[e.offset:e.offset + e.numel].view(e.param.shape)
        if not separate_master:
            for sec in self.sections:
                lo, hi = self.local_master_range(sec)
                sec.master = self.shadow(lo, hi)
        self.result.model.compute_dtype = dtype
        self.refresh_resident_extras()

    def _pieces(self, entries: list[StorageEntry]) -> list[tuple[int, int, int, int]]:
        """``(owning rank, offset in the owner's rest buffer, offset in the destination buffer, elements)`` for every
        stretch of ``entries`` that one rank holds."""

        out = []
        for e in entries:
            sec = self.section_of(e)
            n = self.mesh.size(sec.shard_axis)
            per = sec.length // n
            for r in range(n):
                lo = sec.start + r * per
                a, b = max(e.offset, lo), min(e.offset + e.numel, lo + per)
                if b > a:
                    out.append((r, sec.rest_start + a - lo, self._dst_off[e.name] + a - e.offset, b - a))
        return out

    def _gather(self, entries: list[StorageEntry], dst: torch.Tensor, key: tuple) -> None:
        """Fill ``dst`` with the compute copy of ``entries`` from the ranks that hold them."""

        if not entries:
            return
        pieces = self._pieces(entries)
        sec = self.section_of(entries[0])
        me = self.mesh.coord(sec.shard_axis)
        esize = dst.element_size()
        if self.arena is not None:
            from research_b200.parallel.symmetric import copy_pieces

            if key not in self._tables:
                rows = [(self.arena.peer_ptr(r, self._rest_off) + src * esize, dst.data_ptr() + off * esize, n * esize)
                        for r, src, off, n in pieces]
                self._tables[key] = (torch.tensor(rows, dtype=torch.int64, device=self.device), len(rows))
            table, n = self._tables[key]
            copy_pieces(table, n)
            return
        # collectives: every rank contributes what it holds, zeros elsewhere (adding zeros is exact)
        dst.zero_()
        for r, src, off, n in pieces:
            if r == me:
                dst[off:off + n].copy_(self.rest[src:src + n])
        group = self.mesh.group(sec.shard_axis)
        if group is not None:
            dist.all_reduce(dst, group=group)

    def refresh_resident_extras(self) -> None:
        """Once per step, after the optimizer: every rank gets the parameters that are used outside the transformer
        layers (embedding, final norm, lm_head); the layer buffers are stale from here on."""

        if self.resident:
            return
        if self.arena is not None:
            self.arena.barrier()            # every rank's rest buffer holds the updated weights
        self._gather(self._extra_entries, self._extras, ("extras",))
        for e in self._extra_entries:
            off = self._dst_off[e.name]
            e.param.data = self._extras[off:off + e.numel].view(e.param.shape)
        self._slot_layer = [None] * self._n_slots

    def _fetch(self, layer: int, slot: int) -> None:
        dev_cuda = self._gather_stream is not None
        if dev_cuda:
            if self._slot_free[slot] is not None:
                self._gather_stream.wait_event(self._slot_free[slot])      # the slot's previous reader is done
            self._gather_stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self._gather_stream):
                self._gather(self._layer_entries[layer], self._slots[slot], ("layer", layer, slot))
                ev = torch.cuda.Event()
                ev.record(self._gather_stream)
            self._slot_ready[slot] = ev
        else:
            self._gather(self._layer_entries[layer], self._slots[slot], ("layer", layer, slot))
        self._slot_layer[slot] = layer

    def _slot_for(self, layer: int) -> int:
        return self._layers.index(layer) % self._n_slots

    def acquire_layer(self, layer: int, direction: int = 1) -> None:
        """Make the weights of ``layer`` usable (its parameters point into a layer buffer that holds them) and start
        fetching the next layer in ``direction`` (+1 forward, -1 backward).  No-op with resident weights."""

        if self.resident or layer not in self._layer_entries:
            return
        slot = self._slot_for(layer)
        if self._slot_layer[slot] != layer:
            self._fetch(layer, slot)
        if self._slot_ready[slot] is not None:
            torch.cuda.current_stream(self.device).wait_event(self._slot_ready[slot])
        buf = self._slots[slot]
        for e in self._layer_entries[layer]:
            off = self._dst_off[e.name]
            e.param.data = buf[off:off + e.numel].view(e.param.shape)
        nxt = layer + direction
        if nxt in self._layer_entries:
            nslot = self._slot_for(nxt)
            if nslot != slot and self._slot_layer[nslot] != nxt:
                if self._gather_stream is not None and self._slot_layer[nslot] is not None:
                    # the kernels that read the other slot (the previous layer) are all on the stream by now
                    ev = torch.cuda.Event()
                    ev.record(torch.cuda.current_stream(self.device))
                    self._slot_free[nslot] = ev
                self._fetch(nxt, nslot)

    def memory_report(self) -> dict[str, Any]:
        """Bytes of the compute copy this rank holds, by kind (for the resident / sharded comparison)."""

        esize = torch.empty((), dtype=self.compute_dtype).element_size()
        if self.resident:
            return {"mode": "resident", "compute_bytes": self.total * esize, "layer_buffer_bytes": 0,
                    "extras_bytes": 0}
        return {"mode": "sharded", "compute_bytes": self.rest.numel() * esize,
                "layer_buffer_bytes": sum(s.numel() for s in self._slots) * esize,
                "extras_bytes": self._extras.numel() * esize, "layer_buffers": self._n_slots}

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

        if not self.resident:
            self.refresh_resident_extras()
            return
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
            "weights_resident": self.resident,
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
