"""Train state <-> checkpoint leaves.

A checkpoint stores *logical* tensors under the reference's ``TrainState`` key paths (src/jaxtitan/state.py:23-32,
steps/train.py:41-50): ``step`` (int32), ``tokens_seen`` (uint32), ``model.<path>`` in the reference layout
(kernels ``[in, out]``, fp32), optimizer moments per logical parameter, the four RNG keys as ``uint32[2]`` raw key
data, and ``moe_balance.layers.<i>.momentum``.  Because leaves are logical (global) tensors, a checkpoint written
under one mesh restores under another.

Gathering: masters and optimizer moments of sections split over the ``fsdp`` axis are all-gathered to full local
arenas; parameters split by tensor or expert parallelism are concatenated along their split axis.
"""

from __future__ import annotations

from typing import Any

import numpy as np
import torch
import torch.distributed as dist

from research_b200.errors import ContractError
from research_b200.models.build import EXPERT_FSDP_AXIS, ROUTED_EXPERT_TAGS, ParamMeta


def _full_arena(trainer, kind: str) -> torch.Tensor:
    """A full-size local fp32 arena holding ``kind`` in ('master', 'mu', 'nu', 'momentum') for every section."""

    store, opt = trainer.store, trainer.optimizer
    arena = torch.zeros(store.total, dtype=torch.float32, device=store.device)
    for i, sec in enumerate(store.sections):
        if kind == "master":
            src = sec.master
        else:
            src = opt.state[i].get(kind)
        if src is None or src.numel() == 0:
            continue
        lo, hi = store.local_master_range(sec)
        arena[lo:hi].copy_(src)
        if sec.shard_axis is not None:
            group = store.mesh.group(sec.shard_axis)
            if group is not None:
                buf = arena[sec.start:sec.start + sec.length]
                dist.all_gather_into_tensor(buf, arena[lo:hi].clone(), group=group)
    return arena


def _gather_axis(t: torch.Tensor, axis: int, group) -> torch.Tensor:
    n = dist.get_world_size(group)
    parts = [torch.empty_like(t) for _ in range(n)]
    dist.all_gather(parts, t.contiguous(), group=group)
    return torch.cat(parts, dim=axis)


def _logical_from_arena(trainer, meta: ParamMeta, arena: torch.Tensor) -> torch.Tensor:
    res, ex = trainer.result, trainer.execution
    entry = next(e for e in trainer.store.entries if e.name == meta.storage)
    storage = arena[entry.offset:entry.offset + entry.numel].view(entry.param.shape)
    t = res.logical_view(meta, storage).contiguous()
    if meta.tp_axis is not None and ex.tp_size > 1:
        t = _gather_axis(t, meta.tp_axis, ex.tp_group)
    if meta.tag in ROUTED_EXPERT_TAGS and ex.efsdp_size > 1:
        t = _gather_axis(t, EXPERT_FSDP_AXIS[meta.tag], ex.expert_fsdp_group)
    if meta.tag in ROUTED_EXPERT_TAGS and ex.ep_size > 1:
        t = _gather_axis(t, 0, ex.ep_group)
    return t


def collect_state_tensors(trainer) -> dict[str, np.ndarray]:
    """Every rank takes part in the gathers; the returned host arrays are complete on every rank."""

    out: dict[str, np.ndarray] = {
        "step": np.asarray(trainer.step, dtype=np.int32),
        "tokens_seen": np.asarray(trainer.tokens_seen, dtype=np.uint32),
        "opt_state.count": np.asarray(trainer.optimizer.count, dtype=np.int32),
    }
    rng = trainer.rng.to_json()
    for name, key in rng.items():
        out[f"rng.{name}"] = np.asarray([key >> 32, key & 0xFFFFFFFF], dtype=np.uint32)
    master = _full_arena(trainer, "master")
    kinds = {"mu": "opt_state.adamw.mu", "nu": "opt_state.adamw.nu", "momentum": "opt_state.matrix.momentum"}
    arenas = {k: _full_arena(trainer, k) for k in kinds}
    backend_of = trainer.optimizer_build.backend_by_name()
    for meta in trainer.result.metadata:
        out[f"model.{meta.name}"] = _logical_from_arena(trainer, meta, master).cpu().numpy()
        if not meta.trainable:
            continue
        backend = backend_of.get(meta.name, "adamw")
        names = ("mu", "nu") if backend == "adamw" else ("momentum",)
        for k in names:
            out[f"{kinds[k]}.{meta.name}"] = _logical_from_arena(trainer, meta, arenas[k]).cpu().numpy()
    if trainer.moe_balance is not None:
        for i, layer in enumerate(trainer.moe_balance.layers):
            out[f"moe_balance.layers.{i}.momentum"] = layer.momentum.detach().cpu().numpy()
    return out


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
    opt.count = int(np.asarray(need("opt_state.count")).reshape(-1)[0])
    for name in ("train", "data", "eval", "sample"):
        hi, lo = (int(v) for v in np.asarray(need(f"rng.{name}")).reshape(-1)[:2])
        setattr(trainer.rng, name, (hi << 32) | lo)
    backend_of = trainer.optimizer_build.backend_by_name()
    full = {k: torch.zeros(store.total, dtype=torch.float32, device=dev) for k in ("master", "mu", "nu", "momentum")}
    kinds = {"mu": "opt_state.adamw.mu", "nu": "opt_state.adamw.nu", "momentum": "opt_state.matrix.momentum"}
    for meta in res.metadata:
        entry = next(e for e in store.entries if e.name == meta.storage)

        def put(kind: str, leaf: str) -> None:
            storage = full[kind][entry.offset:entry.offset + entry.numel].view(entry.param.shape)
            res.storage_view(meta, storage).copy_(_local_from_logical(trainer, meta, need(leaf)).to(dev))

        put("master", f"model.{meta.name}")
        if meta.trainable:
            backend = backend_of.get(meta.name, "adamw")
            for k in (("mu", "nu") if backend == "adamw" else ("momentum",)):
                put(k, f"{kinds[k]}.{meta.name}")
    for i, sec in enumerate(store.sections):
        lo, hi = store.local_master_range(sec)
        if sec.master is not None and sec.master.data_ptr() != store.compute_arena[lo:hi].data_ptr():
            sec.master.copy_(full["master"][lo:hi])
        for k, t in opt.state[i].items():
            t.copy_(full[k][lo:hi])
    store.compute_arena.copy_(full["master"])
    if trainer.moe_balance is not None:
        for i, layer in enumerate(trainer.moe_balance.layers):
            layer.momentum.copy_(torch.from_numpy(np.asarray(need(f"moe_balance.layers.{i}.momentum"))).to(dev))
