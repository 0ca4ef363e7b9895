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
ALIGN_CHANNEL = 15         # step-start alignment barrier (align_ranks)
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
        lib.b200c_vmm_alloc.argtypes = [ull, ull, ctypes.POINTER(vp), ctypes.POINTER(ci), ctypes.POINTER(ull)]
        lib.b200c_vmm_import.argtypes = [ci, ull, ctypes.POINTER(vp)]
        lib.b200c_vmm_free.argtypes = [vp, ull]
        lib.b200c_flag_block_bytes.argtypes = []
        lib.b200c_reduce_scatter_pull.argtypes = [ctypes.POINTER(vp), vp, ctypes.c_longlong, ctypes.c_float, vp,
                                                  ctypes.POINTER(vp), ci, ci, ctypes.c_uint, ci, vp, vp, vp]
        lib.b200c_reduce_scatter_nvls.argtypes = [vp, vp, ctypes.c_longlong, ctypes.c_float, vp, ctypes.POINTER(vp),
                                                  ci, ci, ctypes.c_uint, ci, vp, vp, vp]
        lib.b200c_all_gather_nvls.argtypes = [vp, vp, ctypes.c_longlong, ctypes.POINTER(vp), ci, ci, ctypes.c_uint,
                                              vp, vp, vp]
        lib.b200c_copy_pieces.argtypes = [vp, ci, ci, vp]
        lib.b200c_copy_pieces.restype = ci
        lib.b200c_mc_supported.argtypes = []
        lib.b200c_mc_granularity.argtypes = [ci, ull]
        lib.b200c_mc_granularity.restype = ull
        lib.b200c_mc_create.argtypes = [ull, ci, ctypes.POINTER(ci), ctypes.POINTER(ull)]
        lib.b200c_mc_import.argtypes = [ci, ctypes.POINTER(ull)]
        lib.b200c_mc_add_device.argtypes = [ull]
        lib.b200c_mc_bind_and_map.argtypes = [ull, vp, ull, ctypes.POINTER(vp)]
        lib.b200c_mc_release.argtypes = [ull, vp, ull]
        lib.b200c_all_gather_pull.argtypes = [ctypes.POINTER(vp), vp, ctypes.c_longlong, ctypes.POINTER(vp), ci, ci,
                                              ctypes.c_uint, ci, vp, vp, vp]
        lib.b200c_barrier.argtypes = [ctypes.POINTER(vp), ci, ci, ctypes.c_uint, vp, vp]
        lib.b200c_barrier.restype = ci
        for fn in (lib.b200c_vmm_alloc, lib.b200c_vmm_import, lib.b200c_vmm_free, lib.b200c_flag_block_bytes,
                   lib.b200c_reduce_scatter_pull, lib.b200c_all_gather_pull, lib.b200c_reduce_scatter_nvls,
                   lib.b200c_all_gather_nvls, lib.b200c_mc_supported, lib.b200c_mc_create, lib.b200c_mc_import,
                   lib.b200c_mc_add_device, lib.b200c_mc_bind_and_map, lib.b200c_mc_release):
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


def broadcast_descriptor(group, fd: int | None, *, tag: str, timeout_ms: int = _EXCHANGE_TIMEOUT_MS) -> int:
    """Rank 0 of ``group`` hands ``fd`` to every other rank through the descriptor broker; returns the local
    descriptor (rank 0: ``fd`` itself)."""

    host = hostlib.load()
    if host is None or not hasattr(host, "b200h_fd_serve"):
        raise ContractError("the host library with the descriptor broker is not built")
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    base = [None]
    if rank == 0:
        base[0] = os.path.join(tempfile.gettempdir(), f"b200-{uuid.uuid4().hex[:12]}-{tag}.sock")
    dist.broadcast_object_list(base, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    if rank == 0:
        handle = host.b200h_fd_serve(base[0].encode(), fd, world - 1, timeout_ms)
        if handle < 0:
            raise ContractError(f"descriptor broker could not listen on {base[0]}: errno {-handle}")
        delivered = host.b200h_fd_serve_join(handle)
        if delivered != world - 1:
            raise ContractError(f"descriptor broker delivered {delivered} of {world - 1} descriptors")
        return fd
    got = host.b200h_fd_fetch(base[0].encode(), timeout_ms)
    if got < 0:
        raise ContractError(f"rank {rank} could not fetch the multicast descriptor: errno {-got}")
    return got


def copy_pieces(table: torch.Tensor, n_pieces: int, ctas_per_piece: int = 8) -> None:
    """One launch that copies ``n_pieces`` byte ranges described by ``table`` (int64 ``[n, 3]``: source address,
    destination address, byte count; sources may be peers' arenas) on the current stream."""

    rc = _comm_lib().b200c_copy_pieces(table.data_ptr(), int(n_pieces), int(ctas_per_piece), native._stream())
    native._check(rc, "b200c_copy_pieces")


def nvls_requested() -> bool:
    """``RESEARCH_B200_NVLS``: 1 binds symmetric arenas to an NVLink multicast object and runs the reduce-scatter /
    all-gather through ``multimem`` instructions; 0 (the default) keeps plain peer loads.  Tests that let a rank
    leave while others keep running must keep it 0: a rank that dies with memory bound to a multicast object can
    raise NVLink faults on the other ranks' GPUs."""

    return os.environ.get("RESEARCH_B200_NVLS", "0") == "1"


_GUARD_BYTES = 256
_MAX_GUARDS = 32
_CANARY = 0x5AFEB200
_ARENAS: "weakref.WeakSet[SymmetricArena]" = weakref.WeakSet()
_ARENA_ORDER: "list[weakref.ref[SymmetricArena]]" = []      # creation order, the same on every rank of a group


def align_ranks() -> None:
    """One stream-ordered barrier per live arena, in creation order.  Called at the start of a training step: the
    barrier's wait carries the long host-skew limit (``native.peer_wait_limit_ms``), so the peer-memory kernels
    that follow see ranks that are already aligned on the device and only ever wait for device-side skew."""

    for ref in list(_ARENA_ORDER):
        arena = ref()
        if arena is None or not arena.ptrs:
            _ARENA_ORDER.remove(ref)
            continue
        arena.barrier(channel=ALIGN_CHANNEL)


def close_all_arenas() -> None:
    """Close every live arena of this process in creation order (collective over each arena's group)."""

    for ref in list(_ARENA_ORDER):
        arena = ref()
        if arena is not None:
            arena.close()
    _ARENA_ORDER.clear()


def check_all_canaries() -> None:
    """Check the guard words of every live arena of this process (tests, and every step when
    ``RESEARCH_B200_DEBUG=1``)."""

    for arena in list(_ARENAS):
        arena.check_canaries()


class SymmetricArena:
    """``nbytes`` of payload per rank plus flag blocks, mapped on every rank of ``group``."""

    def __init__(self, group, nbytes: int, *, device: torch.device | None = None, tag: str = "arena",
                 multicast: bool | None = None):
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
        self.mc_ptr = 0                      # multicast address of the arena (0: not bound)
        self._mc_handle = 0
        want_mc = nvls_requested() if multicast is None else bool(multicast)
        align = 0
        with torch.cuda.device(self.device):
            if want_mc and lib.b200c_mc_supported():
                align = int(lib.b200c_mc_granularity(self.world, want))
            rc = lib.b200c_vmm_alloc(want, align, ctypes.byref(ptr), ctypes.byref(fd), ctypes.byref(padded))
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
        _ARENA_ORDER.append(weakref.ref(self))
        # per channel: a CTA counter and per-CTA partial sums, so that collectives on different streams never share them
        self.scratch = torch.zeros(CHANNELS, 1024, dtype=torch.float32, device=self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)  # nobody signals into an arena that is still being zeroed
        if want_mc:
            self._bind_multicast(align, tag)

    # ---- NVLink multicast ----------------------------------------------------------------------------
    def _bind_multicast(self, align: int, tag: str) -> None:
        """Create one multicast object over all ranks' arenas, bind the local arena and map the object.  Collective;
        on any failure every rank ends with ``mc_ptr == 0`` and the plain peer kernels keep running."""

        lib, group = self._lib, self.group
        dev = self.device

        def all_ok(flag: bool) -> bool:
            t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
            return bool(int(t.item()))

        with torch.cuda.device(dev):
            ok = bool(lib.b200c_mc_supported()) and align > 0 and self.padded % align == 0
            if not all_ok(ok):
                return
            handle, fd = ctypes.c_ulonglong(0), ctypes.c_int(-1)
            created = True
            if self.rank == 0:
                created = lib.b200c_mc_create(self.padded, self.world, ctypes.byref(fd), ctypes.byref(handle)) == 0
            if not all_ok(created):
                return
            local_fd = broadcast_descriptor(group, fd.value if self.rank == 0 else None, tag=f"{tag}-mc")
            imported = True
            if self.rank != 0:
                imported = lib.b200c_mc_import(local_fd, ctypes.byref(handle)) == 0
            os.close(local_fd)
            added = imported and lib.b200c_mc_add_device(handle.value) == 0
            if not all_ok(added):       # the reduction doubles as the barrier "every device has been added"
                return
            mc = ctypes.c_void_p()
            bound = lib.b200c_mc_bind_and_map(handle.value, self.local_ptr, self.padded, ctypes.byref(mc)) == 0
            if bound:
                self._mc_handle, self.mc_ptr = int(handle.value), int(mc.value)
            if not all_ok(bound):
                self._release_multicast()

    def _release_multicast(self) -> None:
        if self._mc_handle:
            with torch.cuda.device(self.device):
                self._lib.b200c_mc_release(self._mc_handle, self.mc_ptr or None, self.padded)
        self._mc_handle, self.mc_ptr = 0, 0

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
                       sumsq: torch.Tensor | None = None, channel: int = 0, nvls: bool | None = None,
                       max_ctas: int = 0) -> None:
        """fp32 region at byte ``offset`` of every arena, ``numel_per_rank`` elements (may differ between ranks, may
        be 0): it becomes ``scale * sum over ranks`` on this rank (in place unless ``out`` is given); ``sumsq``
        (1 element) accumulates the sum of squares of the result.  ``offset`` is where THIS rank's slice starts.
        ``nvls`` (default: whenever the arena is bound to a multicast object) reads the slice once through the
        switch with ``multimem.ld_reduce`` instead of once per peer.  ``max_ctas`` caps the grid."""

        n = int(numel_per_rank)
        flags = self._ptr_array(self.flag_ptrs(channel))
        dst = self.local_ptr + offset if out is None else out.data_ptr()
        use_nvls = bool(self.mc_ptr) if nvls is None else (bool(nvls) and bool(self.mc_ptr))
        scratch = self.scratch[channel].data_ptr()
        ss = None if sumsq is None else sumsq.data_ptr()
        status = native.status_word(self.device).data_ptr()
        if use_nvls:
            rc = self._lib.b200c_reduce_scatter_nvls(self.mc_ptr + offset, dst, n, float(scale), ss, flags, self.world,
                                                     self.rank, self.next_epoch(channel), int(max_ctas), scratch,
                                                     status, native._stream())
            native._check(rc, "b200c_reduce_scatter_nvls")
            return
        src = self._ptr_array([self.peer_ptr(r, offset) for r in range(self.world)])
        rc = self._lib.b200c_reduce_scatter_pull(src, dst, n, float(scale), ss, flags, self.world, self.rank,
                                                 self.next_epoch(channel), int(max_ctas), scratch, status,
                                                 native._stream())
        native._check(rc, "b200c_reduce_scatter_pull")

    def all_gather(self, offset: int, bytes_per_rank: int, *, channel: int = 1, nvls: bool | None = None) -> None:
        """Region ``[offset, offset + world * bytes_per_rank)``: every rank's own slice is copied to all ranks (pulled
        over peer loads, or pushed with ``multimem.st`` when the arena is bound to a multicast object)."""

        b = int(bytes_per_rank)
        flags = self._ptr_array(self.flag_ptrs(channel))
        use_nvls = bool(self.mc_ptr) if nvls is None else (bool(nvls) and bool(self.mc_ptr))
        scratch = self.scratch[channel].data_ptr()
        status = native.status_word(self.device).data_ptr()
        if use_nvls:
            mine = offset + self.rank * b
            rc = self._lib.b200c_all_gather_nvls(self.local_ptr + mine, self.mc_ptr + mine, b, flags, self.world,
                                                 self.rank, self.next_epoch(channel), scratch, status, native._stream())
            native._check(rc, "b200c_all_gather_nvls")
            return
        src = self._ptr_array([self.peer_ptr(r, offset + r * b) for r in range(self.world)])
        rc = self._lib.b200c_all_gather_pull(src, self.local_ptr + offset, b, flags, self.world, self.rank,
                                             self.next_epoch(channel), 0, scratch, status, native._stream())
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
            self._release_multicast()
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
