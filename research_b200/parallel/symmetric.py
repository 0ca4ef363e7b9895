"""Symmetric device memory across the ranks of one node, and the pull collectives that run on it.

Every rank of a process group allocates an arena of the same size with CUDA virtual memory management, exports it
as a POSIX file descriptor, and maps all peers' arenas (descriptor exchange through the unix-socket broker of the
host library).  A kernel on one GPU can then load from and store to any rank's arena over NVLink.  The tail of
each arena holds flag blocks (one per channel) that the kernels use for their bounded cross-GPU waits; epochs are
counted on the host, identically on every rank.

Reference counterparts: third_party/ThunderKittens/include/types/system/vmm.cuh:15-93 (allocation and mapping),
include/pyutils/broker.cuh:38-140 (descriptor passing), include/pyutils/parallel_tensor.cuh:23-336 (tensor view).
"""

from __future__ import annotations

import ctypes
import os
import tempfile
import uuid
import weakref

import torch
import torch.distributed as dist

from research_b200.errors import ContractError, KernelError
from research_b200.native import hostlib
from research_b200.ops import native

_ALIGN = 4096
CHANNELS = 16
_EXCHANGE_TIMEOUT_MS = 60_000


class _DeviceSpan:
    """Adapter that lets ``torch.as_tensor`` wrap raw device memory (CUDA array interface, version 3)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def _comm_lib() -> ctypes.CDLL:
    lib = native.load()
    if not hasattr(lib, "b200c_vmm_alloc"):
        raise KernelError("the kernel library was built without the communication runtime")
    if not getattr(lib, "_b200c_declared", False):
        ull, vp, ci = ctypes.c_ulonglong, ctypes.c_void_p, ctypes.c_int
        lib.b200c_vmm_alloc.argtypes = [ull, ctypes.POINTER(vp), ctypes.POINTER(ci), ctypes.POINTER(ull)]
        lib.b200c_vmm_import.argtypes = [ci, ull, ctypes.POINTER(vp)]
        lib.b200c_vmm_free.argtypes = [vp, ull]
        lib.b200c_flag_block_bytes.argtypes = []
        lib.b200c_reduce_scatter_pull.argtypes = [ctypes.POINTER(vp), vp, ctypes.c_longlong, ctypes.c_float, vp,
                                                  ctypes.POINTER(vp), ci, ci, ctypes.c_uint, vp, vp, vp]
        lib.b200c_all_gather_pull.argtypes = [ctypes.POINTER(vp), vp, ctypes.c_longlong, ctypes.POINTER(vp), ci, ci,
                                              ctypes.c_uint, ci, vp, vp, vp]
        lib.b200c_barrier.argtypes = [ctypes.POINTER(vp), ci, ci, ctypes.c_uint, vp, vp]
        lib.b200c_barrier.restype = ci
        for fn in (lib.b200c_vmm_alloc, lib.b200c_vmm_import, lib.b200c_vmm_free, lib.b200c_flag_block_bytes,
                   lib.b200c_reduce_scatter_pull, lib.b200c_all_gather_pull):
            fn.restype = ci
        lib._b200c_declared = True
    return lib


def exchange_descriptors(group, fd: int, *, tag: str, timeout_ms: int = _EXCHANGE_TIMEOUT_MS) -> list[int]:
    """Every rank publishes ``fd``; returns one descriptor per rank of the group (own slot: ``fd`` itself)."""

    host = hostlib.load()
    if host is None or not hasattr(host, "b200h_fd_serve"):
        raise ContractError("the host library with the descriptor broker is not built")
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    base = [None]
    if rank == 0:
        base[0] = os.path.join(tempfile.gettempdir(), f"b200-{uuid.uuid4().hex[:12]}-{tag}")
    dist.broadcast_object_list(base, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    paths = [f"{base[0]}-{r}.sock" for r in range(world)]
    handle = host.b200h_fd_serve(paths[rank].encode(), fd, world - 1, timeout_ms)
    if handle < 0:
        raise ContractError(f"descriptor broker could not listen on {paths[rank]}: errno {-handle}")
    out = []
    for r in range(world):
        if r == rank:
            out.append(fd)
            continue
        got = host.b200h_fd_fetch(paths[r].encode(), timeout_ms)
        if got < 0:
            raise ContractError(f"rank {rank} could not fetch the descriptor of rank {r}: errno {-got}")
        out.append(got)
    delivered = host.b200h_fd_serve_join(handle)
    if delivered != world - 1:
        raise ContractError(f"descriptor broker of rank {rank} delivered {delivered} of {world - 1} descriptors")
    return out


_GUARD_BYTES = 256
_MAX_GUARDS = 32
_CANARY = 0x5AFEB200
_ARENAS: "weakref.WeakSet[SymmetricArena]" = weakref.WeakSet()


def check_all_canaries() -> None:
    """Check the guard words of every live arena of this process (tests, and every step when
    ``RESEARCH_B200_DEBUG=1``)."""

    for arena in list(_ARENAS):
        arena.check_canaries()


class SymmetricArena:
    """``nbytes`` of payload per rank plus flag blocks, mapped on every rank of ``group``."""

    def __init__(self, group, nbytes: int, *, device: torch.device | None = None, tag: str = "arena"):
        if not torch.cuda.is_available():
            raise ContractError("symmetric arenas need CUDA devices")
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ContractError(f"symmetric arenas cover the ranks of one node (at most 8), got {self.world}")
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        lib = _comm_lib()
        self._lib = lib
        self.flag_bytes = lib.b200c_flag_block_bytes()
        self.payload = (int(nbytes) + _GUARD_BYTES * _MAX_GUARDS + _ALIGN - 1) // _ALIGN * _ALIGN
        want = self.payload + CHANNELS * self.flag_bytes
        ptr, fd, padded = ctypes.c_void_p(), ctypes.c_int(-1), ctypes.c_ulonglong(0)
        with torch.cuda.device(self.device):
            rc = lib.b200c_vmm_alloc(want, ctypes.byref(ptr), ctypes.byref(fd), ctypes.byref(padded))
        if rc != 0:
            raise KernelError(f"b200c_vmm_alloc({want} bytes) failed with code {rc}")
        self.padded = int(padded.value)
        self.local_ptr = int(ptr.value)
        sizes = [None] * self.world
        dist.all_gather_object(sizes, self.padded, group=group)
        if len(set(sizes)) != 1:
            raise ContractError(f"ranks allocated arenas of different sizes: {sizes}")
        fds = exchange_descriptors(group, fd.value, tag=tag)
        self.ptrs: list[int] = []
        with torch.cuda.device(self.device):
            for r, peer_fd in enumerate(fds):
                if r == self.rank:
                    self.ptrs.append(self.local_ptr)
                    continue
                p = ctypes.c_void_p()
                rc = lib.b200c_vmm_import(peer_fd, self.padded, ctypes.byref(p))
                os.close(peer_fd)
                if rc != 0:
                    raise KernelError(f"mapping the arena of rank {r} failed with code {rc}")
                self.ptrs.append(int(p.value))
        os.close(fd.value)
        self.bytes = torch.as_tensor(_DeviceSpan(self.local_ptr, self.padded), device=self.device)
        self.bytes.zero_()
        self._epochs = [0] * CHANNELS
        self._cursor = 0
        self._guards: list[tuple[int, int]] = []      # (byte offset of the guard, offset of the buffer before it)
        _ARENAS.add(self)
        self.scratch = torch.zeros(1024, dtype=torch.float32, device=self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)  # nobody signals into an arena that is still being zeroed

    # ---- carving -------------------------------------------------------------------------------------
    def carve(self, numel: int, dtype: torch.dtype) -> tuple[torch.Tensor, int]:
        """A zero-filled tensor inside the local arena and its byte offset (the same on every rank)."""

        size = numel * torch.empty((), dtype=dtype).element_size()
        off = self._cursor
        guard = (off + size + 255) // 256 * 256
        if guard + _GUARD_BYTES > self.payload:
            raise ContractError(f"symmetric arena exhausted: {off} + {size} > {self.payload}")
        # a guard block of canary words follows every buffer: a kernel (local or on a peer) that writes past the end
        # of a buffer changes it, and check_canaries() names the buffer
        self.bytes[guard:guard + _GUARD_BYTES].view(torch.int32).fill_(_CANARY)
        self._guards.append((guard, off))
        self._cursor = guard + _GUARD_BYTES
        return self.bytes[off:off + size].view(dtype), off

    def check_canaries(self) -> None:
        """Raise when a guard block behind one of the carved buffers no longer holds its canary words."""

        if not self._guards:
            return
        words = torch.stack([self.bytes[g:g + _GUARD_BYTES].view(torch.int32) for g, _ in self._guards])
        bad = (words != _CANARY).any(dim=1).cpu().tolist()                      # one device-to-host read
        broken = [off for (_, off), hit in zip(self._guards, bad) if hit]
        if broken:
            raise KernelError(f"symmetric arena of rank {self.rank}: the guard words behind the buffers at byte "
                              f"offsets {broken} were overwritten (a write ran past the end of a buffer)")

    def peer_ptr(self, rank: int, offset: int) -> int:
        return self.ptrs[rank] + offset

    def flag_ptrs(self, channel: int) -> list[int]:
        return [p + self.payload + channel * self.flag_bytes for p in self.ptrs]

    def next_epoch(self, channel: int) -> int:
        self._epochs[channel] += 1
        return self._epochs[channel] & 0x7FFFFFFF

    def _ptr_array(self, values: list[int]):
        arr = (ctypes.c_void_p * self.world)()
        for i, v in enumerate(values):
            arr[i] = v
        return arr

    # ---- collectives ---------------------------------------------------------------------------------
    def reduce_scatter(self, offset: int, numel_per_rank: int, *, out: torch.Tensor | None = None, scale: float = 1.0,
                       sumsq: torch.Tensor | None = None, channel: int = 0) -> None:
        """fp32 region ``[offset, offset + world * numel_per_rank * 4)`` of every arena: this rank's slice becomes
        ``scale * sum over ranks`` (in place unless ``out`` is given); ``sumsq`` (1 element) accumulates the sum of
        squares of the result."""

        n = int(numel_per_rank)
        mine = offset + self.rank * n * 4
        src = self._ptr_array([self.peer_ptr(r, mine) for r in range(self.world)])
        flags = self._ptr_array(self.flag_ptrs(channel))
        dst = self.local_ptr + mine if out is None else out.data_ptr()
        rc = self._lib.b200c_reduce_scatter_pull(src, dst, n, float(scale), None if sumsq is None else sumsq.data_ptr(),
                                                 flags, self.world, self.rank, self.next_epoch(channel),
                                                 self.scratch.data_ptr(), native.status_word(self.device).data_ptr(),
                                                 native._stream())
        native._check(rc, "b200c_reduce_scatter_pull")

    def all_gather(self, offset: int, bytes_per_rank: int, *, channel: int = 1) -> None:
        """Region ``[offset, offset + world * bytes_per_rank)``: every rank's own slice is copied to all ranks."""

        b = int(bytes_per_rank)
        src = self._ptr_array([self.peer_ptr(r, offset + r * b) for r in range(self.world)])
        flags = self._ptr_array(self.flag_ptrs(channel))
        rc = self._lib.b200c_all_gather_pull(src, self.local_ptr + offset, b, flags, self.world, self.rank,
                                             self.next_epoch(channel), 0, self.scratch.data_ptr(),
                                             native.status_word(self.device).data_ptr(), native._stream())
        native._check(rc, "b200c_all_gather_pull")

    def barrier(self, channel: int = 4) -> None:
        """Stream-ordered barrier over the ranks of the arena (a one-block kernel with bounded waits)."""

        flags = self._ptr_array(self.flag_ptrs(channel))
        rc = self._lib.b200c_barrier(flags, self.world, self.rank, self.next_epoch(channel),
                                     native.status_word(self.device).data_ptr(), native._stream())
        native._check(rc, "b200c_barrier")

    def close(self) -> None:
        if getattr(self, "ptrs", None):
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
            for p in self.ptrs:
                self._lib.b200c_vmm_free(p, self.padded)
            self.ptrs = []
            self._guards = []          # the memory is gone: nothing left to check
            _ARENAS.discard(self)


def build_collectively(group, factory, what: str):
    """Run ``factory()`` (which allocates symmetric memory, a collective operation) on every rank of ``group`` and
    return its result only if it succeeded everywhere; otherwise every rank gets ``None`` and the caller takes its
    NCCL formulation.  The reason is printed once per rank, so a box whose driver refuses shareable allocations
    still trains."""

    import sys

    obj, err = None, None
    try:
        obj = factory()
    except Exception as exc:  # noqa: BLE001 - any failure means "do not use peer memory"
        err = exc
    ok = torch.tensor([0 if err is not None else 1], dtype=torch.int32,
                      device=torch.device("cuda", torch.cuda.current_device()))
    dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
    if int(ok.item()) == 1:
        return obj
    print(f"research_b200: {what} unavailable on rank {dist.get_rank(group)}"
          f"{'' if err is None else f' ({type(err).__name__}: {err})'}; using the NCCL path", file=sys.stderr)
    return None
