"""Train state <-> checkpoint leaves.

A checkpoint stores *logical* tensors under the reference's ``TrainState`` key paths (src/jaxtitan/state.py:23-32,
steps/train.py:41-50): ``step`` (int32), ``tokens_seen`` (uint32), ``model.<path>`` in the reference layout
(kernels ``[in, out]``, fp32), optimizer moments per logical parameter, the four RNG keys as ``uint32[2]`` raw key
data, and ``moe_balance.layers.<i>.momentum``.  Because leaves are logical (global) tensors, a checkpoint written
under one mesh restores under another.

Gathering works one parameter at a time: the shards of a parameter whose section is split over the ``fsdp`` axis
are summed into a zero buffer of that parameter's size (to the writer's rank only when saving), parameters split by
tensor or expert parallelism are concatenated along their split axis, and the leaf goes to the host before the next
one is touched.  Optimizer leaves are named after the state tree of the reference's optax chain
(:func:`optimizer_leaf_names`).  ``tokens_seen`` keeps the reference's uint32 leaf and adds ``tokens_seen_hi``.
"""

from __future__ import annotations

from typing import Any

import numpy as np
import torch
import torch.distributed as dist

from research_b200.errors import ContractError
from research_b200.models.build import EXPERT_FSDP_AXIS, ROUTED_EXPERT_TAGS, ParamMeta


def _entry_values(trainer, sec_index: int, sec, entry, kind: str, *, all_ranks: bool) -> torch.Tensor:
    """fp32 values of one storage entry for ``kind`` in ('master', 'mu', 'nu', 'momentum').

    Sections split over a shard axis hold only a range (AdamW) or only the owner's matrices (Muon / Dion2) on each
    rank: every rank writes its overlap with the entry into a zero buffer of the entry's size and the buffers are
    summed over the shard axis - to every rank (``all_ranks``) or only to the rank at coordinate 0 of the axis, which
    is where the checkpoint writer sits.  The largest temporary is one parameter, never a whole arena."""

    store, opt = trainer.store, trainer.optimizer
    buf = torch.zeros(entry.numel, dtype=torch.float32, device=store.device)
    src = sec.master if kind == "master" else opt.state[sec_index].get(kind)
    lo, hi = store.local_master_range(sec)
    a, b = max(entry.offset, lo), min(entry.offset + entry.numel, hi)
    if src is not None and src.numel() and b > a:
        buf[a - entry.offset:b - entry.offset].copy_(src[a - lo:b - lo])
    if sec.shard_axis is not None:
        group = store.mesh.group(sec.shard_axis)
        if group is not None:
            if all_ranks:
                dist.all_reduce(buf, group=group)
            else:
                dist.reduce(buf, dst=dist.get_global_rank(group, 0), group=group)
    return buf


def _gather_axis(t: torch.Tensor, axis: int, group) -> torch.Tensor:
    n = dist.get_world_size(group)
    parts = [torch.empty_like(t) for _ in range(n)]
    dist.all_gather(parts, t.contiguous(), group=group)
    return torch.cat(parts, dim=axis)


def _logical_from_storage(trainer, meta: ParamMeta, entry, values: torch.Tensor) -> torch.Tensor:
    res, ex = trainer.result, trainer.execution
    t = res.logical_view(meta, values.view(entry.param.shape)).contiguous()
    if meta.tp_axis is not None and ex.tp_size > 1:
        t = _gather_axis(t, meta.tp_axis, ex.tp_group)
    if meta.tag in ROUTED_EXPERT_TAGS and ex.efsdp_size > 1:
        t = _gather_axis(t, EXPERT_FSDP_AXIS[meta.tag], ex.expert_fsdp_group)
    if meta.tag in ROUTED_EXPERT_TAGS and ex.ep_size > 1:
        t = _gather_axis(t, 0, ex.ep_group)
    return t


_DION2_AXIS_NAMES = ("row", "col")


def optimizer_leaf_names(trainer) -> dict[tuple[str, str], str]:
    """``(kind, parameter name) -> checkpoint leaf name`` for the optimizer moments.

    The names follow the state tree of the reference's optax chain (src/jaxtitan/optim/build.py:176-202, 560-656):
    element 0 is the global-norm clip when configured (no arrays), then one masked transform per non-empty group in
    the order Muon with decay, Muon without, Dion2 rows with / without decay, Dion2 columns with / without decay,
    distributed Muon, AdamW.  A masked transform keeps its state under ``inner_state``; Muon and Dion2 states hold
    ``momentum``, ``optax.adamw`` is itself a chain whose element 0 holds ``mu`` and ``nu``."""

    spec = trainer.optimizer_build.spec
    groups: dict[str, list] = {}
    for a in trainer.optimizer_build.route_assignments:
        if a.backend == "muon":
            key = "muon_decay" if a.weight_decay else "muon_no_decay"
        elif a.backend == "dion2":
            key = f"dion2_{'col' if _is_col(a, trainer) else 'row'}_" + ("decay" if a.weight_decay else "no_decay")
        elif a.backend == "dist_muon":
            key = "dist_muon"
        else:
            key = "adamw"
        groups.setdefault(key, []).append(a)
    order = ["muon_decay", "muon_no_decay", "dion2_row_decay", "dion2_row_no_decay", "dion2_col_decay",
             "dion2_col_no_decay", "dist_muon", "adamw"]
    index = 1 if spec.grad_clip_norm is not None else 0
    out: dict[tuple[str, str], str] = {}
    for key in order:
        if key not in groups:
            continue
        for a in groups[key]:
            if key == "adamw":
                out[("mu", a.name)] = f"opt_state.{index}.inner_state.0.mu.{a.name}"
                out[("nu", a.name)] = f"opt_state.{index}.inner_state.0.nu.{a.name}"
            else:
                out[("momentum", a.name)] = f"opt_state.{index}.inner_state.momentum.{a.name}"
        index += 1
    return out


def _is_col(assignment, trainer) -> bool:
    """Dion2 selects columns when the split axis is the last logical axis of the matrix."""

    meta = next(m for m in trainer.result.metadata if m.name == assignment.name)
    axis = assignment.matrix_axis if assignment.matrix_axis is not None else 0
    return axis == len(meta.shape) - 1


_LEGACY_KINDS = {"mu": "opt_state.adamw.mu", "nu": "opt_state.adamw.nu", "momentum": "opt_state.matrix.momentum"}


def iter_state_tensors(trainer, *, writer_only: bool = False):
    """Yield ``(leaf name, host array or None)`` for every leaf of the train state, one parameter at a time.

    Collective: every rank must consume the whole iterator.  With ``writer_only`` the arrays are assembled on the
    checkpoint writer (global rank 0) alone and the other ranks get ``None`` values; otherwise every rank gets every
    array.  Peak extra memory is one parameter on the device and one on the host."""

    want = (not writer_only) or trainer.is_writer
    tokens = int(trainer.tokens_seen)

    def host(value, dtype):
        return np.asarray(value, dtype=dtype) if want else None

    yield "step", host(trainer.step, np.int32)
    # the reference counter is uint32 (steps/train.py:43-44); the high word keeps the exact count beyond 2^32 tokens
    yield "tokens_seen", host(tokens & 0xFFFFFFFF, np.uint32)
    yield "tokens_seen_hi", host(tokens >> 32, np.uint32)
    yield "opt_state.count", host(trainer.optimizer.count, np.int32)
    for name, key in trainer.rng.to_json().items():
        yield f"rng.{name}", host([key >> 32, key & 0xFFFFFFFF], np.uint32)
    store = trainer.store
    backend_of = trainer.optimizer_build.backend_by_name()
    leaf_of = optimizer_leaf_names(trainer)
    sec_index = {id(sec): i for i, sec in enumerate(store.sections)}
    entry_by_name = {e.name: e for e in store.entries}
    cache: dict[tuple[str, str], torch.Tensor] = {}      # values of the storage entry in hand, per kind

    def values(entry, sec, kind):
        key = (entry.name, kind)
        if key not in cache:
            for k in [k for k in cache if k[0] != entry.name]:
                del cache[k]
            cache[key] = _entry_values(trainer, sec_index[id(sec)], sec, entry, kind, all_ranks=not writer_only)
        return cache[key]

    for meta in trainer.result.metadata:
        entry = entry_by_name[meta.storage]
        sec = store.section_of(entry)
        kinds = ["master"]
        if meta.trainable:
            kinds += ["mu", "nu"] if backend_of.get(meta.name, "adamw") == "adamw" else ["momentum"]
        for kind in kinds:
            t = _logical_from_storage(trainer, meta, entry, values(entry, sec, kind))
            leaf = f"model.{meta.name}" if kind == "master" else leaf_of[(kind, meta.name)]
            yield leaf, (t.cpu().numpy() if want else None)
    if trainer.moe_balance is not None:
        for i, layer in enumerate(trainer.moe_balance.layers):
            yield f"moe_balance.layers.{i}.momentum", (layer.momentum.detach().float().cpu().numpy() if want else None)


def collect_state_tensors(trainer) -> dict[str, np.ndarray]:
    """Every rank takes part in the gathers; the returned host arrays are complete on every rank."""

    return dict(iter_state_tensors(trainer, writer_only=False))


def _local_from_logical(trainer, meta: ParamMeta, full: np.ndarray) -> torch.Tensor:
    ex = trainer.execution
    t = torch.from_numpy(np.ascontiguousarray(full))
    if tuple(t.shape) != tuple(meta.shape):
        raise ContractError(f"checkpoint leaf for {meta.name} has shape {tuple(t.shape)}, expected {meta.shape}")
    if meta.tp_axis is not None and ex.tp_size > 1:
        t = t.chunk(ex.tp_size, dim=meta.tp_axis)[ex.tp_rank]
    if meta.tag in ROUTED_EXPERT_TAGS and ex.ep_size > 1:
        t = t.chunk(ex.ep_size, dim=0)[ex.ep_rank]
    if meta.tag in ROUTED_EXPERT_TAGS and ex.efsdp_size > 1:
        t = t.chunk(ex.efsdp_size, dim=EXPERT_FSDP_AXIS[meta.tag])[ex.efsdp_rank]
    return t.transpose(-1, -2) if meta.transposed else t


def load_state_tensors(trainer, tensors: dict[str, np.ndarray]) -> None:
    store, opt, res = trainer.store, trainer.optimizer, trainer.result
    dev = store.device

    def need(name: str) -> np.ndarray:
        if name not in tensors:
            raise ContractError(f"checkpoint is missing leaf {name!r}")
        return tensors[name]

    trainer.step = int(np.asarray(need("step")).reshape(-1)[0])
    trainer.tokens_seen = int(np.asarray(need("tokens_seen")).reshape(-1)[0])
    if "tokens_seen_hi" in tensors:
        trainer.tokens_seen += int(np.asarray(tensors["tokens_seen_hi"]).reshape(-1)[0]) << 32
    opt.count = int(np.asarray(need("opt_state.count")).reshape(-1)[0])
    for name in ("train", "data", "eval", "sample"):
        hi, lo = (int(v) for v in np.asarray(need(f"rng.{name}")).reshape(-1)[:2])
        setattr(trainer.rng, name, (hi << 32) | lo)
    backend_of = trainer.optimizer_build.backend_by_name()
    leaf_of = optimizer_leaf_names(trainer)

    def moment_leaf(kind: str, name: str) -> str:
        leaf = leaf_of[(kind, name)]
        legacy = f"{_LEGACY_KINDS[kind]}.{name}"          # names written before the optax-chain naming
        return leaf if leaf in tensors or legacy not in tensors else legacy

    # one storage entry at a time: assemble its values from the logical leaves, then keep the range this rank owns
    sec_index = {id(sec): i for i, sec in enumerate(store.sections)}
    for entry in store.entries:
        sec = store.section_of(entry)
        i = sec_index[id(sec)]
        lo, hi = store.local_master_range(sec)
        a, b = max(entry.offset, lo), min(entry.offset + entry.numel, hi)
        kinds = {"master"}
        for meta in entry.metas:
            if meta.trainable:
                kinds |= {"mu", "nu"} if backend_of.get(meta.name, "adamw") == "adamw" else {"momentum"}
        for kind in sorted(kinds):
            storage = torch.zeros(entry.param.shape, dtype=torch.float32, device=dev)
            for meta in entry.metas:
                if kind != "master" and not meta.trainable:
                    continue
                leaf = f"model.{meta.name}" if kind == "master" else moment_leaf(kind, meta.name)
                res.storage_view(meta, storage).copy_(_local_from_logical(trainer, meta, need(leaf)).to(dev))
            flat = storage.reshape(-1)
            if kind == "master":
                store.load_shadow(entry, flat)
                if b > a and sec.master is not None and store.compute_dtype != torch.float32:
                    sec.master[a - lo:b - lo].copy_(flat[a - entry.offset:b - entry.offset])
            elif b > a and kind in opt.state[i]:
                opt.state[i][kind][a - lo:b - lo].copy_(flat[a - entry.offset:b - entry.offset])
    if not store.resident:
        store.refresh_resident_extras()          # weights sharded at rest: the per-step gathers start from the new values
    if trainer.moe_balance is not None:
        for i, layer in enumerate(trainer.moe_balance.layers):
            layer.momentum.copy_(torch.from_numpy(np.asarray(need(f"moe_balance.layers.{i}.momentum"))).to(dev))
