"""ctypes binding of the host-side C++ runtime library (``ops/_lib/libb200host.so``): threaded chunk IO for
checkpoints and the token-window gather of the sequential / shuffle data pipelines.  Every function degrades to
``False`` (caller falls back to NumPy) when the library has not been built."""

from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np

_LIB_PATH = Path(__file__).resolve().parent.parent / "ops" / "_lib" / "libb200host.so"
_lib = None
_tried = False


def load():
    global _lib, _tried
    if _tried:
        return _lib
    _tried = True
    if not _LIB_PATH.exists():
        try:
            from research_b200.kernels.build import build_host_only

            build_host_only()
        except Exception:
            return None
    if _LIB_PATH.exists():
        try:
            lib = ctypes.CDLL(str(_LIB_PATH))
        except OSError:
            return None
        lib.b200h_write_file.argtypes = [ctypes.c_char_p, ctypes.c_void_p, ctypes.c_ulonglong, ctypes.c_int]
        lib.b200h_write_file.restype = ctypes.c_int
        lib.b200h_read_file.argtypes = [ctypes.c_char_p, ctypes.c_void_p, ctypes.c_ulonglong, ctypes.c_int]
        lib.b200h_read_file.restype = ctypes.c_int
        lib.b200h_gather_windows.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                             ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        lib.b200h_gather_windows.restype = ctypes.c_int
        if hasattr(lib, "b200h_fd_serve"):
            lib.b200h_fd_serve.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
            lib.b200h_fd_serve.restype = ctypes.c_int
            lib.b200h_fd_serve_join.argtypes = [ctypes.c_int]
            lib.b200h_fd_serve_join.restype = ctypes.c_int
            lib.b200h_fd_fetch.argtypes = [ctypes.c_char_p, ctypes.c_int]
            lib.b200h_fd_fetch.restype = ctypes.c_int
        _lib = lib
    return _lib


def write_file(path: Path, arr: np.ndarray, threads: int = 0) -> bool:
    lib = load()
    if lib is None:
        return False
    arr = np.ascontiguousarray(arr)
    rc = lib.b200h_write_file(str(path).encode(), arr.ctypes.data_as(ctypes.c_void_p), arr.nbytes, threads)
    if rc != 0:
        raise OSError(rc, f"native write of {path} failed")
    return True


def read_file(path: Path, out: np.ndarray, threads: int = 0) -> bool:
    lib = load()
    if lib is None:
        return False
    rc = lib.b200h_read_file(str(path).encode(), out.ctypes.data_as(ctypes.c_void_p), out.nbytes, threads)
    if rc != 0:
        raise OSError(rc, f"native read of {path} failed")
    return True


def gather_windows(shards: list[np.ndarray], shard_starts: list[int], starts: np.ndarray, window: int,
                   inputs: np.ndarray, targets: np.ndarray, threads: int = 4) -> bool:
    lib = load()
    if lib is None:
        return False
    n = len(shards)
    ptrs = (ctypes.c_void_p * n)(*[s.ctypes.data for s in shards])
    bounds = np.asarray(list(shard_starts), dtype=np.int64)
    st = np.ascontiguousarray(starts, dtype=np.int64)
    rc = lib.b200h_gather_windows(ctypes.cast(ptrs, ctypes.c_void_p), bounds.ctypes.data_as(ctypes.c_void_p), n,
                                  st.ctypes.data_as(ctypes.c_void_p), len(st), window,
                                  inputs.ctypes.data_as(ctypes.c_void_p), targets.ctypes.data_as(ctypes.c_void_p),
                                  threads)
    if rc != 0:
        raise IndexError("token window leaves the dataset shards")
    return True
