"""The optimizer step over a :class:`ParamStore`: global-norm clip, AdamW, Muon, distributed Muon, Dion2.

Update rules restate the reference transforms: AdamW with decoupled decay ``-lr * wd * p`` and bias correction
(optax semantics, src/jaxtitan/optim/build.py:29-31); Muon ``m <- 0.95 m + 0.05 g``, Nesterov input
``0.05 g + 0.95 m``, five Newton-Schulz steps in bf16, step ``-lr * 0.2 sqrt(max(rows, cols)) * O - lr * wd * p``
(optim/muon.py:65-167, 482-526); Dion2 ``m <- m + g``, top quarter of rows/columns by L1 norm, Polar Express,
scatter with ``sqrt(rows/cols)``, selected momentum scaled by 0.95 (optim/dion2.py:34-125).  The learning rate
is the schedule at the *old* count (steps/train.py:227).

Where the work happens: AdamW is one flat-arena kernel launch per section (fp32 master, moments and the compute
copy updated in one pass); matrix optimizers run per logical matrix on the rank that owns it, with every
product on the tcgen05 GEMM.  Tensor-parallel shards either gather the logical matrix (``duplicated``) or
all-reduce the Gram matrices of their shards (``distributed``; optim/muon.py:354-463).
"""

from __future__ import annotations

import math
from typing import Any

import torch
import torch.distributed as dist

from research_b200.errors import ContractError
from research_b200.models.build import ROUTED_EXPERT_TAGS
from research_b200.ops import functional as Fn
from research_b200.ops import native
from research_b200.optim import orthogonalize as orth
from research_b200.optim.build import ADAMW_B1, ADAMW_B2, ADAMW_EPS, OptimizerBuildResult
from research_b200.parallel.sharding import ParamStore, Section, StorageEntry


def _sumsq(x: torch.Tensor, out: torch.Tensor, index: int) -> None:
    if x.numel() == 0:
        return
    if x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and x.is_contiguous() and Fn.native_enabled():
        native.sumsq(x.reshape(-1), out[index:index + 1], accumulate=True)
    else:
        out[index] += x.float().pow(2).sum()


class Optimizer:
    def __init__(self, build: OptimizerBuildResult, store: ParamStore):
        self.build = build
        self.store = store
        self.spec = build.spec
        self.count = 0
        self.mesh = store.mesh
        self.routes = {a.name: a for a in build.route_assignments}
        dev = store.device
        self.state: dict[int, dict[str, torch.Tensor]] = {}
        for i, sec in enumerate(store.sections):
            lo, hi = store.local_master_range(sec)
            n = hi - lo
            if sec.backend == "adamw":
                self.state[i] = {"mu": torch.zeros(n, dtype=torch.float32, device=dev),
                                 "nu": torch.zeros(n, dtype=torch.float32, device=dev)}
            elif sec.backend in ("muon", "dion2"):
                self.state[i] = {"momentum": torch.zeros(n, dtype=torch.float32, device=dev)}
            else:
                self.state[i] = {}
        self._norm_buf = torch.zeros(len(store.sections), dtype=torch.float32, device=dev)
        self._clip = torch.ones(1, dtype=torch.float32, device=dev)
        self.tp_group = store.result.execution.tp_group
        self.tp_size = store.result.execution.tp_size
        self.muon_plans = {p.name: p for p in getattr(build, "muon_execution_plans", ())}
        self._gram_reducer = None
        from research_b200.optim.diagnostics import group_templates

        self.group_templates, self.group_index = group_templates(build.route_assignments, store.result.metadata)

    # ---- norms -----------------------------------------------------------------------------------
    def _sum_axes(self, sec: Section) -> list[str]:
        axes = []
        if sec.shard_axis is not None and self.mesh.size(sec.shard_axis) > 1:
            axes.append(sec.shard_axis)
        if self.tp_size > 1 and sec.entries and any(m.tp_axis is not None for m in sec.entries[0].metas):
            axes.append("tp")
        ep_axis = self.store.ep_axis
        if ep_axis and self.mesh.size(ep_axis) > 1 and any(e.is_expert for e in sec.entries) and ep_axis not in axes:
            axes.append(ep_axis)
        if self.mesh.size("expert_fsdp") > 1 and any(e.is_expert for e in sec.entries):
            axes.append("expert_fsdp")   # every rank of the axis holds a distinct slice of the intermediate dimension
        return axes

    def _global_sumsq(self, arena: torch.Tensor | None, use_master: bool = False) -> torch.Tensor:
        """Sum of squares over all distinct parameters' values in ``arena`` (or the fp32 masters)."""

        buf = self._norm_buf
        buf.zero_()
        for i, sec in enumerate(self.store.sections):
            if sec.backend == "frozen" or sec.length == 0:
                continue
            lo, hi = self.store.local_master_range(sec)
            src = sec.master if use_master else arena[lo:hi]
            _sumsq(src, buf, i)
        axes_needed: dict[str, list[int]] = {}
        for i, sec in enumerate(self.store.sections):
            for axis in self._sum_axes(sec):
                axes_needed.setdefault(axis, []).append(i)
        for axis, idx in axes_needed.items():
            group = self.mesh.group(axis)
            if group is None:
                continue
            part = buf[idx].clone()
            dist.all_reduce(part, group=group)
            buf[idx] = part
        return buf.sum()

    # ---- the step ----------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, *, diagnostics: bool = False) -> dict[str, Any]:
        store, spec = self.store, self.spec
        lr = float(self.build.schedule(self.count))
        fb = self.build.adamw_fallback_schedule
        adamw_lr = lr if (fb is None or spec.name == "adamw") else float(fb(self.count))
        grad_sq = self._global_sumsq(store.grad_arena)
        grad_norm = grad_sq.sqrt()
        if spec.grad_clip_norm is not None:
            clip = float(spec.grad_clip_norm)
            self._clip.copy_((clip / torch.clamp(grad_norm, min=clip)).reshape(1))
        else:
            self._clip.fill_(1.0)
        before = None
        if diagnostics:
            before = [sec.master.clone() if sec.backend != "frozen" else None for sec in store.sections]
        for i, sec in enumerate(store.sections):
            if sec.backend == "adamw":
                self._adamw(i, sec, adamw_lr)
            elif sec.backend in ("muon", "dion2"):
                slow = [e for e in sec.entries if store.owns(sec, e)]
                if sec.backend == "muon" and self.tp_size > 1 and self.muon_plans:
                    slow = self._dist_muon_bucketed(i, sec, slow, lr)
                if sec.backend == "muon" and self._fast_muon_ok():
                    slow = self._muon_section_fast(i, sec, slow, lr)
                elif sec.backend == "dion2" and self._fast_muon_ok():
                    slow = [e for e in slow if not self._dion2_entry_fast(i, sec, e, lr)]
                for e in slow:
                    self._matrix_entry(i, sec, e, lr)
        store.gather_compute_weights()
        self.count += 1
        out: dict[str, Any] = {"lr": lr, "adamw_lr": adamw_lr, "grad_norm": grad_norm, "clip_scale": self._clip[0]}
        if diagnostics:
            out["param_norm"] = self._global_sumsq(None, use_master=True).sqrt().clone()
            upd = torch.zeros(1, dtype=torch.float32, device=store.device)
            buf = self._norm_buf
            buf.zero_()
            for i, sec in enumerate(store.sections):
                if before[i] is not None:
                    _sumsq((sec.master - before[i]).contiguous(), buf, i)
            # one reduction per axis, in an order that is the same in every process: iterating a set of strings
            # follows the per-process hash seed, and ranks that reduce over two axes in opposite orders wait on one
            # another for ever
            sum_axes: dict[str, list[int]] = {}
            for i, sec in enumerate(store.sections):
                for axis in self._sum_axes(sec):
                    sum_axes.setdefault(axis, []).append(i)
            for axis, idx in sum_axes.items():
                group = self.mesh.group(axis)
                if group is not None and idx:
                    part = buf[idx].clone()
                    dist.all_reduce(part, group=group)
                    buf[idx] = part
            out["update_norm"] = buf.sum().sqrt().clone()
            del upd
            from research_b200.optim.diagnostics import group_square_sums

            out["group_squares"] = group_square_sums(self, before, _sumsq)      # [groups, 3], still on the device
        return out

    # ---- AdamW -------------------------------------------------------------------------------------
    def _adamw(self, i: int, sec: Section, lr: float) -> None:
        store = self.store
        lo, hi = store.local_master_range(sec)
        if hi <= lo:
            return
        st = self.state[i]
        g = store.grad_arena[lo:hi]
        p = sec.master
        wd = float(self.spec.weight_decay) if sec.decay else 0.0      # the route's weight_decay flag
        step = self.count + 1
        separate = store.compute_dtype != torch.float32
        if p.is_cuda and Fn.native_enabled():
            shadow = store.shadow(lo, hi) if separate else None
            native.adamw(p, st["mu"], st["nu"], g, shadow, self._clip, lr, ADAMW_B1, ADAMW_B2, ADAMW_EPS, wd, step)
            return
        gs = g * self._clip
        st["mu"].mul_(ADAMW_B1).add_(gs, alpha=1 - ADAMW_B1)
        st["nu"].mul_(ADAMW_B2).addcmul_(gs, gs, value=1 - ADAMW_B2)
        mhat = st["mu"] / (1 - ADAMW_B1 ** step)
        vhat = st["nu"] / (1 - ADAMW_B2 ** step)
        p.sub_(lr * (mhat / (vhat.sqrt() + ADAMW_EPS) + wd * p))
        if separate:
            store.shadow(lo, hi).copy_(p)

    # ---- matrix optimizers -------------------------------------------------------------------------
    def _fast_muon_ok(self) -> bool:
        return (self.store.device.type == "cuda" and self.store.compute_dtype == torch.bfloat16 and
                Fn.native_enabled())

    def _muon_section_fast(self, i: int, sec: Section, entries: list[StorageEntry], lr: float) -> list[StorageEntry]:
        """Batched Muon: logical matrices of equal shape are stacked so that each Newton-Schulz step is three
        batched GEMMs.  Covers plain 2-D parameters (and row slices of fused ones) and rank-3 expert stacks, whose
        per-expert matrices are addressed with a stride; returns the entries this path does not handle."""

        store = self.store
        lo, _ = store.local_master_range(sec)
        leftovers: list[StorageEntry] = []
        # (rows, cols) -> [(entry, meta, offset of the first matrix inside the entry, matrices, stride)]
        groups: dict[tuple[int, int], list[tuple[StorageEntry, Any, int, int, int]]] = {}
        for e in entries:
            master = store.master_view(sec, e)
            simple = master is not None and master.dim() in (2, 3) and e.numel % 4 == 0 and all(
                self.routes[m.name].backend == "muon" for m in e.metas)
            if not simple:
                leftovers.append(e)
                continue
            full_rows, cols = e.param.shape[-2], e.param.shape[-1]
            batch = e.param.shape[0] if master.dim() == 3 else 1
            spans = [meta.rows if meta.rows is not None else (0, full_rows) for meta in e.metas]
            if any((b - a) % 8 for a, b in spans) or cols % 8:
                leftovers.append(e)
                continue
            for meta, (a, b) in zip(e.metas, spans):
                groups.setdefault((b - a, cols), []).append((e, meta, a * cols, batch, full_rows * cols))
        wd = float(self.spec.weight_decay)
        mom_all = self.state[i]["momentum"]
        max_stack = 1 << 29  # elements per Newton-Schulz batch (1 GiB of bf16)
        for (rows, cols), items in groups.items():
            per = rows * cols
            chunk: list[tuple[StorageEntry, Any, int, int, int]] = []
            count = 0
            for item in items + [None]:
                if item is not None and (not chunk or (count + item[3]) * per <= max_stack):
                    chunk.append(item)
                    count += item[3]
                    continue
                self._muon_stack(sec, chunk, count, rows, cols, lo, mom_all, lr, wd)
                chunk, count = ([item], item[3]) if item is not None else ([], 0)
        return leftovers

    def _muon_stack(self, sec: Section, items, n: int, rows: int, cols: int, lo: int, mom_all, lr: float,
                    wd: float) -> None:
        store = self.store
        per = rows * cols
        stack = native.scratch("muon_stack", n * per, torch.bfloat16, store.device)[: n * per].view(n, rows, cols)
        sq = torch.zeros(n, dtype=torch.float32, device=store.device)
        at = 0
        for e, meta, first, batch, stride in items:
            native.muon_momentum_batched(store.grad_arena[e.offset + first:], mom_all[e.offset - lo + first:],
                                         stack[at:], sq[at:], self._clip, per, stride, batch, orth.MUON_MOMENTUM,
                                         orth.MUON_NESTEROV)
            at += batch
        if native.deterministic():        # the kernel adds per-CTA partial sums in arrival order
            sq = stack.float().pow(2).sum(dim=(1, 2))
        native.scale_by_inv_norm(stack, sq, orth.MUON_NS_EPS)
        out = orth.newton_schulz_stack_(stack)
        step = lr * orth.rms_match_scale((rows, cols))
        at = 0
        for e, meta, first, batch, stride in items:
            decay = 1.0 - lr * wd if self.routes[meta.name].weight_decay else 1.0
            native.muon_apply_batched(sec.master[e.offset - lo + first:], out[at:],
                                      store.shadow(e.offset + first), per, stride, batch, decay, step)
            at += batch

    # ---- distributed Muon over the tensor-parallel group ---------------------------------------------
    def _reducer(self):
        """Transport of the packed Gram reductions: a symmetric arena of the tensor-parallel group on CUDA (one
        peer-memory kernel per reduction), ``torch.distributed`` otherwise."""

        if self._gram_reducer is None:
            import os

            from research_b200.optim import distributed_ns as dns

            reducer = None
            use_arena = (self.store.device.type == "cuda" and Fn.native_enabled() and self.tp_size <= 8 and
                         os.environ.get("RESEARCH_B200_PEER_COLLECTIVES", "1") != "0")
            if use_arena:
                from research_b200.parallel.symmetric import build_collectively

                # bf16 payload limit of a bucket, held as fp32, plus one norm slot per leaf
                capacity = dns.GRAM_BUCKET_MAX_BYTES // 2 + 4096
                largest = max((p.gram_dimension ** 2 for p in self.muon_plans.values()), default=0)
                capacity = max(capacity, largest + 4096)
                reducer = build_collectively(self.tp_group,
                                             lambda: dns.ArenaReducer(self.tp_group, capacity, self.store.device),
                                             "symmetric arena for distributed Muon")
            self._gram_reducer = reducer or dns.TorchReducer(self.tp_group)
        return self._gram_reducer

    def _dist_muon_bucketed(self, i: int, sec: Section, entries: list[StorageEntry], lr: float) -> list[StorageEntry]:
        """Muon for the tensor-parallel-sharded matrices of a section whose plan is a distributed execution: momentum
        update per leaf, then one bucketed Newton-Schulz per Gram bucket (one packed reduction per step for all
        leaves of the bucket), then the parameter update.  Returns the entries that take another path."""

        from research_b200.optim.distributed_ns import bucketed_distributed_zeropower

        store = self.store
        lo, _ = store.local_master_range(sec)
        wd = float(self.spec.weight_decay)
        leftovers: list[StorageEntry] = []
        buckets: dict[int, list[tuple]] = {}
        touched: list[StorageEntry] = []
        for e in entries:
            plans = [self.muon_plans.get(m.name) for m in e.metas]
            master = store.master_view(sec, e)
            if (master is None or master.dim() != 2 or
                    any(p is None or p.execution == "duplicated" for p in plans)):
                leftovers.append(e)
                continue
            mom = self.state[i]["momentum"][e.offset - lo:e.offset - lo + e.numel].view(e.param.shape)
            grad = e.param.main_grad
            touched.append(e)
            for meta, plan in zip(e.metas, plans):
                route = self.routes[meta.name]
                sl = slice(None) if meta.rows is None else slice(*meta.rows)
                g = grad[sl] * self._clip
                m = mom[sl]
                m.mul_(orth.MUON_MOMENTUM).add_(g, alpha=1.0 - orth.MUON_MOMENTUM)
                u = (1.0 - orth.MUON_MOMENTUM) * g + orth.MUON_MOMENTUM * m if orth.MUON_NESTEROV else m
                axis = (len(meta.shape) - 1 - route.matrix_axis) if meta.transposed else route.matrix_axis
                buckets.setdefault(plan.bucket_id, []).append((meta, route, plan, u.to(torch.bfloat16), master[sl], axis))
        dtype = torch.bfloat16 if orth.MUON_NS_PRECISION == "bfloat16" else torch.float32
        for bucket_id in sorted(buckets):
            items = buckets[bucket_id]
            outs = bucketed_distributed_zeropower([it[3] for it in items], [it[2] for it in items],
                                                  [it[5] for it in items], self.tp_group, self._reducer(), dtype)
            for (meta, route, plan, _, w, _), o in zip(items, outs):
                if wd != 0.0 and route.weight_decay:
                    w.mul_(1.0 - lr * wd)
                w.add_(o.to(w.dtype), alpha=-lr * orth.rms_match_scale(meta.shape))
        if store.compute_dtype != torch.float32:
            for e in touched:
                store.write_entry_shadow(e, store.master_view(sec, e))
        return leftovers

    def _matrix_entry(self, i: int, sec: Section, e: StorageEntry, lr: float) -> None:
        store = self.store
        master = store.master_view(sec, e)
        if master is None:
            raise ContractError(f"matrix parameter {e.name} is not fully resident on its owner")
        lo, _ = store.local_master_range(sec)
        mom = self.state[i]["momentum"][e.offset - lo:e.offset - lo + e.numel].view(e.param.shape)
        grad = e.param.main_grad
        wd = float(self.spec.weight_decay)
        clip = self._clip
        for meta in e.metas:
            route = self.routes[meta.name]
            sl = (slice(None),) if meta.rows is None else (
                (slice(None), slice(*meta.rows)) if master.dim() == 3 else (slice(*meta.rows),))
            g = grad[sl] * clip
            m = mom[sl]
            w = master[sl]
            decay = wd if route.weight_decay else 0.0
            if sec.backend == "dion2":
                self._dion2_update(meta, route, g, m, w, lr, decay)
            else:
                self._muon_update(meta, route, g, m, w, lr, decay)
        if store.compute_dtype != torch.float32:
            store.write_entry_shadow(e, master)

    def _muon_update(self, meta, route, g, m, w, lr: float, wd: float) -> None:
        m.mul_(orth.MUON_MOMENTUM).add_(g, alpha=1.0 - orth.MUON_MOMENTUM)
        u = (1.0 - orth.MUON_MOMENTUM) * g + orth.MUON_MOMENTUM * m if orth.MUON_NESTEROV else m
        # storage is [out, in] = transpose of the logical [in, out]; orthogonalisation commutes with transposition
        logical_shape = meta.shape
        if route.backend == "dist_muon" and self.tp_size > 1:
            storage_axis = (len(meta.shape) - 1 - route.matrix_axis) if meta.transposed else route.matrix_axis
            plan = self.muon_plans.get(meta.name)
            if plan is not None and plan.execution != "duplicated":
                from research_b200.optim.distributed_ns import bucketed_distributed_zeropower

                o = bucketed_distributed_zeropower([u.to(torch.bfloat16)], [plan], [storage_axis], self.tp_group,
                                                   self._reducer())[0]
            else:
                full = _all_gather_axis(u.to(torch.bfloat16).contiguous(), storage_axis, self.tp_group)
                o_full = orth.zeropower_via_newton_schulz(full)
                o = o_full.chunk(self.tp_size, dim=storage_axis)[dist.get_rank(self.tp_group)]
        else:
            o = orth.zeropower_via_newton_schulz(u.to(torch.bfloat16))
        scale = lr * orth.rms_match_scale(logical_shape)
        if wd != 0.0:
            w.mul_(1.0 - lr * wd)
        w.add_(o.to(w.dtype), alpha=-scale)

    def _dion2_entry_fast(self, i: int, sec: Section, e: StorageEntry, lr: float) -> bool:
        """Dion2 for one storage entry with every logical matrix of it (all experts of a rank-3 stack) handled by
        the same batched ops: L1 norms, one top-k, one gather, a batched Polar Express on tcgen05 GEMMs, one
        scatter.  Same rules as ``_dion2_matrix`` (reference: src/jaxtitan/optim/dion2.py:34-125).  Returns False
        when the entry is not eligible and must take the per-matrix path."""

        store = self.store
        master = store.master_view(sec, e)
        if master is None or master.dim() not in (2, 3) or any(self.routes[m.name].backend != "dion2" for m in e.metas):
            return False
        if any(self._logical_split(m) is not None for m in e.metas):
            return False            # a shard of a logical matrix: the selection runs on the gathered matrix
        lo, _ = store.local_master_range(sec)
        mom = self.state[i]["momentum"][e.offset - lo:e.offset - lo + e.numel].view(e.param.shape)
        grad = e.param.main_grad
        wd = float(self.spec.weight_decay)
        lead = (slice(None),) if master.dim() == 3 else ()
        # the apply kernel writes the bf16 compute copy of the slices it updates when that copy has the master's layout
        shadow = None
        if store.compute_dtype == torch.bfloat16:
            shadow = (e.param.data if store.resident else store.shadow(e.offset, e.offset + e.numel)).view(master.shape)
        all_kernels = True
        for meta in e.metas:
            route = self.routes[meta.name]
            sl = lead + ((slice(None),) if meta.rows is None else (slice(*meta.rows),))
            m3 = mom[sl] if master.dim() == 3 else mom[sl].unsqueeze(0)
            g3 = grad[sl] if master.dim() == 3 else grad[sl].unsqueeze(0)
            w3 = master[sl] if master.dim() == 3 else master[sl].unsqueeze(0)
            n, rows, cols = m3.shape
            logical_axis = route.matrix_axis if route.matrix_axis is not None else 0
            if len(meta.shape) == 3:
                logical_axis -= 1
            axis = (1 - logical_axis) if meta.transposed else logical_axis      # 0: rows are selected, 1: columns
            k = max(1, math.ceil(orth.DION2_FRACTION * (rows if axis == 0 else cols)))
            if (k % 8) or (rows % 8) or (cols % 8):
                return False
            decay = 1.0 - lr * wd if (wd != 0.0 and route.weight_decay) else 1.0
            scale = lr * math.sqrt(meta.shape[-2] / meta.shape[-1])
            stride = m3.stride(0) if n > 1 else rows * cols
            kernels = (Fn.native_enabled() and m3.is_cuda and m3.dtype == torch.float32 and g3.dtype == torch.float32
                       and m3.stride(1) == cols and g3.stride(1) == cols and (n == 1 or g3.stride(0) == stride)
                       and native.dion2_supported(n, rows, cols, stride, axis)
                       and all(t.data_ptr() % 16 == 0 for t in (m3, g3, w3)))
            if kernels:
                clip = self._clip if isinstance(self._clip, torch.Tensor) else None
                stack, _, inv = native.dion2_select_stack(g3, m3, clip, n, rows, cols, stride, axis, k,
                                                          orth.DION2_EPSILON)
                o = orth.newton_schulz_stack_(stack, orth.DION2_POLAR_EXPRESS_COEFFICIENTS)
                sh3 = None
                if shadow is not None:
                    sh3 = shadow[sl] if master.dim() == 3 else shadow[sl].unsqueeze(0)
                native.dion2_apply(w3, m3, o, inv, sh3, n, rows, cols, k, stride, axis, decay, scale,
                                   orth.DION2_EF_DECAY)
                continue
            all_kernels = False
            m3.addcmul_(g3, self._clip)
            norms = torch.linalg.vector_norm(m3, ord=1, dim=2 if axis == 0 else 1)             # [n, rows | cols]
            idx = torch.topk(norms, k, dim=1).indices                                          # [n, k]
            gidx = idx[:, :, None].expand(n, k, cols) if axis == 0 else idx[:, None, :].expand(n, rows, k)
            selected = torch.gather(m3, 1 + axis, gidx)                                        # fp32
            stack = selected.to(torch.bfloat16).contiguous()
            sq = stack.float().pow(2).sum(dim=(1, 2))
            stack = stack / (sq.sqrt().to(torch.bfloat16)[:, None, None] * 1.02 + orth.DION2_EPSILON)
            o = orth.newton_schulz_stack_(stack.contiguous(), orth.DION2_POLAR_EXPRESS_COEFFICIENTS)
            if decay != 1.0:
                w3.mul_(decay)
            w3.scatter_add_(1 + axis, gidx, o.float() * (-scale))
            m3.scatter_(1 + axis, gidx, selected * orth.DION2_EF_DECAY)
        if all_kernels and shadow is not None:
            return True
        if store.compute_dtype != torch.float32:
            store.write_entry_shadow(e, master)
        return True

    def _logical_split(self, meta):
        """``(group, axis of the logical shape)`` when this rank holds a slice of the logical matrix along that axis -
        a tensor-parallel shard, or a routed expert whose intermediate dimension is split over ``expert_fsdp`` -
        else ``None``."""

        from research_b200.models.build import EXPERT_FSDP_AXIS, ROUTED_EXPERT_TAGS

        ex = self.store.result.execution
        if meta.tag in ROUTED_EXPERT_TAGS:
            return (ex.expert_fsdp_group, EXPERT_FSDP_AXIS[meta.tag]) if ex.efsdp_size > 1 else None
        if self.tp_size > 1 and meta.tp_axis is not None:
            return self.tp_group, meta.tp_axis
        return None

    def _dion2_update(self, meta, route, g, m, w, lr: float, wd: float) -> None:
        m.add_(g)
        if m.dim() == 3:
            for e in range(m.shape[0]):
                self._dion2_matrix(meta, route, m[e], w[e], lr, wd)
        else:
            self._dion2_matrix(meta, route, m, w, lr, wd)

    def _dion2_matrix(self, meta, route, m, w, lr: float, wd: float) -> None:
        logical_axis = route.matrix_axis if route.matrix_axis is not None else 0
        batched = len(meta.shape) == 3
        if batched:
            logical_axis -= 1
        storage_axis = (1 - logical_axis) if meta.transposed else logical_axis
        rows, cols = meta.shape[-2], meta.shape[-1]
        if wd != 0.0:
            w.mul_(1.0 - lr * wd)
        alpha = -lr * math.sqrt(rows / cols)
        split = self._logical_split(meta)
        if split is not None:
            # The rows and columns are picked by their norms over the whole logical matrix, as in one process: every
            # rank of the group that splits the matrix gathers the momentum, repeats the selection and keeps its own
            # slice of the result.
            group, split_logical = split
            split_logical -= 1 if batched else 0
            split_storage = (1 - split_logical) if meta.transposed else split_logical
            parts, rank = dist.get_world_size(group), dist.get_rank(group)
            full = _all_gather_axis(m.contiguous(), split_storage, group)
            selected, idx = orth.select_dion2_slices(full, select_axis=storage_axis)
            update = torch.zeros_like(full).index_add_(storage_axis, idx, orth.polar_express(selected).to(full.dtype))
            full.index_copy_(storage_axis, idx, selected * orth.DION2_EF_DECAY)
            w.add_(update.chunk(parts, dim=split_storage)[rank].to(w.dtype), alpha=alpha)
            m.copy_(full.chunk(parts, dim=split_storage)[rank])
            return
        selected, idx = orth.select_dion2_slices(m, select_axis=storage_axis)
        o = orth.polar_express(selected).to(w.dtype)
        w.index_add_(storage_axis, idx, o, alpha=alpha)
        m.index_copy_(storage_axis, idx, selected * orth.DION2_EF_DECAY)

    # ---- checkpoint state ---------------------------------------------------------------------------
    def state_dict(self) -> dict[str, Any]:
        return {"count": self.count,
                "sections": {str(i): {k: v for k, v in st.items()} for i, st in self.state.items()}}

    def load_state_dict(self, raw: dict[str, Any]) -> None:
        self.count = int(raw["count"])
        for i, st in raw["sections"].items():
            for k, v in st.items():
                self.state[int(i)][k].copy_(v)


def _all_gather_axis(x: torch.Tensor, axis: int, group) -> torch.Tensor:
    n = dist.get_world_size(group)
    xt = x.movedim(axis, 0).contiguous()
    out = torch.empty((n * xt.shape[0],) + tuple(xt.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, xt, group=group)
    return out.movedim(0, axis).contiguous()
