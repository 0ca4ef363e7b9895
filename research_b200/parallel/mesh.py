"""Named mesh axes -> ``torch.distributed`` process groups (one process per GPU).

The reference builds a ``jax.sharding.Mesh`` from the first N local devices reshaped row-major to the axis sizes
(src/jaxtitan/mesh/sharding.py:116-137), so the last axis is the fastest-varying device index; the same rank
layout is used here: ``rank = ravel_multi_index(coords, axis_sizes)``.  Axis names accept both spellings
(``tp``/``tensor``, ``cp``/``context``, ``ep``/``expert``); the reference spelling is canonical.
"""

from __future__ import annotations

import datetime
import os
from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch
import torch.distributed as dist

from research_b200.config.specs import SUPPORTED_AXES, MeshSpec, ParallelismSpec, resolve_expert_fsdp_axis, \
    resolve_expert_parallel_axis
from research_b200.errors import ContractError


@dataclass
class MeshContext:
    axis_names: tuple[str, ...]
    axis_sizes: tuple[int, ...]
    rank: int
    world_size: int
    coords: dict[str, int]
    groups: dict[str, Any] = field(default_factory=dict)        # axis name -> ProcessGroup (None when size 1)
    device: torch.device = torch.device("cpu")

    def size(self, axis: str) -> int:
        return self.axis_sizes[self.axis_names.index(axis)] if axis in self.axis_names else 1

    def coord(self, axis: str) -> int:
        return self.coords.get(axis, 0)

    def group(self, axis: str):
        return self.groups.get(axis)

    @property
    def sizes(self) -> dict[str, int]:
        return dict(zip(self.axis_names, self.axis_sizes, strict=True))

    def replica_axes(self) -> tuple[str, ...]:
        """Axes over which a data batch is split (gradients are summed over them)."""

        return tuple(a for a in ("data", "fsdp") if self.size(a) > 1)

    def describe(self) -> dict[str, Any]:
        return {"axis_names": list(self.axis_names), "axis_sizes": list(self.axis_sizes),
                "device_count": self.world_size, "rank": self.rank, "coords": dict(self.coords)}


def require_single_node_runtime(world_size: int) -> None:
    """Multi-node is out of scope, as in the reference (mesh/sharding.py:353-361 rejects multi-process JAX)."""

    local = int(os.environ.get("LOCAL_WORLD_SIZE", world_size))
    if local != world_size:
        raise ContractError(
            f"multi-node runs are not supported: world_size={world_size} but LOCAL_WORLD_SIZE={local}"
        )


_group_timeout_s: float | None = None        # the default group's collective timeout, handed on to the axis groups


def _axis_group_timeout():
    """Collective timeout of the per-axis groups: ``RESEARCH_B200_GROUP_TIMEOUT_S`` if set, else the timeout the
    default group was created with here, else the library's default (30 minutes).  Without it a subgroup ignores
    the timeout of the default group, and a rank waiting for a peer that left would wait for half an hour."""

    raw = os.environ.get("RESEARCH_B200_GROUP_TIMEOUT_S")
    seconds = float(raw) if raw else _group_timeout_s
    return None if seconds is None else datetime.timedelta(seconds=seconds)


def validate_runtime_mesh_spec(spec: MeshSpec) -> None:
    """What a mesh must satisfy before any process group is made: known axis names only, and as many devices as
    the launch has ranks (reference: src/jaxtitan/mesh/sharding.py ``validate_runtime_mesh_spec``)."""

    for name in spec.axis_names:
        if name not in SUPPORTED_AXES:
            raise ContractError(f"unsupported mesh axis {name!r}; supported axes: {sorted(SUPPORTED_AXES)}")
    world = dist.get_world_size() if dist.is_initialized() else int(os.environ.get("WORLD_SIZE", "1"))
    if spec.device_count != world:
        raise ContractError(f"mesh axis sizes {spec.axis_sizes} need {spec.device_count} devices but the job has "
                            f"{world} ranks")


def init_distributed(backend: str | None = None, timeout_s: float = 600.0) -> tuple[int, int]:
    """Initialise the default process group from the torchrun environment; returns (rank, world_size)."""

    global _group_timeout_s
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world == 1:
        return 0, 1
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kwargs: dict[str, Any] = {}
        if backend == "nccl":
            local_rank = int(os.environ.get("LOCAL_RANK", rank))
            torch.cuda.set_device(local_rank)
            kwargs["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
        _group_timeout_s = float(timeout_s)
    return rank, world


def build_mesh_context(spec: MeshSpec, *, device: torch.device | None = None) -> MeshContext:
    """Create the process groups of every mesh axis.  All ranks must call this in the same order."""

    for name in spec.axis_names:
        if name not in SUPPORTED_AXES:
            raise ContractError(f"unsupported mesh axis {name!r}; supported axes: {sorted(SUPPORTED_AXES)}")
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    need = spec.device_count
    if need != world:
        raise ContractError(
            f"mesh axis sizes {spec.axis_sizes} need {need} devices but the job has {world} ranks"
        )
    require_single_node_runtime(world)
    sizes = tuple(spec.axis_sizes)
    grid = np.arange(world).reshape(sizes)
    my = np.unravel_index(rank, sizes)
    coords = {name: int(c) for name, c in zip(spec.axis_names, my)}
    groups: dict[str, Any] = {}
    if world > 1:
        for ax, name in enumerate(spec.axis_names):
            if sizes[ax] == 1:
                groups[name] = None
                continue
            moved = np.moveaxis(grid, ax, -1).reshape(-1, sizes[ax])
            mine = None
            for ranks in moved:
                g = dist.new_group(ranks=[int(r) for r in ranks], timeout=_axis_group_timeout())
                if rank in ranks:
                    mine = g
            groups[name] = mine
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    return MeshContext(tuple(spec.axis_names), sizes, rank, world, coords, groups, device)


def execution_context_for(mesh: MeshContext, parallelism: ParallelismSpec, *, fused: bool = True):
    """The activation-side policy (:class:`ExecutionContext`) implied by a mesh and a parallelism spec."""

    from research_b200.models.execution import ExecutionContext

    sizes = mesh.sizes
    ep = resolve_expert_parallel_axis(parallelism, sizes)
    efsdp = resolve_expert_fsdp_axis(parallelism, sizes)
    dispatcher = "all_to_all"
    if ep.enabled and ep.axis == "data":
        dispatcher = "rdep_static"
    return ExecutionContext(
        tp_group=mesh.group("tp") if parallelism.tensor_parallel else None,
        cp_group=mesh.group("cp") if parallelism.context_parallel else None,
        ep_group=mesh.group(ep.axis) if ep.enabled else None,
        expert_fsdp_group=mesh.group("expert_fsdp") if efsdp.enabled else None,
        sequence_parallel=True,
        ep_dispatcher=dispatcher,
        ep_axis_name=ep.axis,
        ep_axis_sharing=ep.axis_sharing,
        cp_attention=parallelism.context_attention,
        fused=fused,
        vocab_parallel=bool(parallelism.vocab_parallel_head and parallelism.tensor_parallel),
    )
