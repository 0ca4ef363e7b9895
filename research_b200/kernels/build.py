"""In-tree nvcc build of the sm_100a kernel library and the host-side C++ runtime library.

The kernels are plain CUDA translation units with ``extern "C"`` launchers (no torch headers), so a
full rebuild takes seconds.  Objects and the shared libraries live next to the sources under
``research_b200/ops/_lib`` and are keyed by a sha256 of sources + flags, so an unchanged tree is not
rebuilt.  Counterpart of the reference's make-driven build cache with a sha256 manifest
(src/jaxtitan/kernels/build.py:146-220); the architecture is fixed to sm_100a here.
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import json
import os
import shutil
import subprocess
from dataclasses import dataclass
from pathlib import Path

from research_b200.errors import ContractError

PKG_ROOT = Path(__file__).resolve().parent.parent
CSRC_DIR = PKG_ROOT / "ops" / "csrc"
NATIVE_DIR = PKG_ROOT / "native"
LIB_DIR = PKG_ROOT / "ops" / "_lib"
KERNEL_LIB = LIB_DIR / "libb200ops.so"
HOST_LIB = LIB_DIR / "libb200host.so"
MANIFEST = LIB_DIR / "build_manifest.json"

ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")
NVCC_FLAGS = ("-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr")
CXX_FLAGS = ("-O3", "-std=c++17", "-fPIC", "-pthread")


@dataclass(frozen=True)
class BuildResult:
    kernel_lib: Path
    host_lib: Path | None
    rebuilt: bool
    sources: tuple[str, ...]
    digest: str


def nvcc_path() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise ContractError("nvcc not found; the sm_100a kernel library cannot be built")
    return found


def kernel_sources() -> list[Path]:
    return sorted(CSRC_DIR.glob("*.cu"))


def host_sources() -> list[Path]:
    return sorted(NATIVE_DIR.glob("*.cpp"))


def _digest(paths: list[Path], flags: tuple[str, ...]) -> str:
    h = hashlib.sha256()
    for p in sorted(paths + sorted(CSRC_DIR.glob("*.cuh")) + sorted(NATIVE_DIR.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise ContractError(f"build command failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")


def build_all(*, force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> BuildResult:
    """Compile every ``.cu`` under ops/csrc for sm_100a and link the kernel library; build the host library."""

    LIB_DIR.mkdir(parents=True, exist_ok=True)
    cu = kernel_sources()
    cpp = host_sources()
    flags = ARCH_FLAGS + NVCC_FLAGS + CXX_FLAGS
    digest = _digest(cu + cpp, flags)
    if not force and KERNEL_LIB.exists() and MANIFEST.exists():
        try:
            old = json.loads(MANIFEST.read_text())
        except (OSError, json.JSONDecodeError):
            old = {}
        if old.get("digest") == digest and (not cpp or HOST_LIB.exists()):
            return BuildResult(KERNEL_LIB, HOST_LIB if cpp else None, False, tuple(p.name for p in cu), digest)

    nvcc = nvcc_path()
    objs: list[Path] = []

    def compile_one(src: Path) -> Path:
        obj = LIB_DIR / (src.stem + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC_DIR), "-c", str(src), "-o", str(obj)]
        if ptxas_info:
            cmd[1:1] = ["-Xptxas", "-v"]
        if verbose:
            print(" ".join(cmd))
        _run(cmd)
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(cu)))) as pool:
        objs = list(pool.map(compile_one, cu))
    _run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(KERNEL_LIB), *[str(o) for o in objs]])

    host_lib = None
    if cpp:
        gxx = shutil.which("g++") or "g++"
        _run([gxx, *CXX_FLAGS, "-shared", "-I", str(NATIVE_DIR), "-o", str(HOST_LIB), *[str(s) for s in cpp]])
        host_lib = HOST_LIB
    MANIFEST.write_text(
        json.dumps(
            {
                "digest": digest,
                "arch": "sm_100a",
                "nvcc_flags": list(ARCH_FLAGS + NVCC_FLAGS),
                "sources": [p.name for p in cu],
                "host_sources": [p.name for p in cpp],
            },
            sort_keys=True,
            indent=1,
        )
    )
    return BuildResult(KERNEL_LIB, host_lib, True, tuple(p.name for p in cu), digest)


def ensure_current() -> BuildResult | None:
    """Rebuild the libraries when they are missing or were built from other sources than the ones on disk.

    Called when the kernel library is loaded: a stale shared object whose exported functions no longer match the
    Python bindings fails in confusing ways, so the sha256 of the sources is checked every time (a few milliseconds)
    and a mismatch triggers the in-tree build.  Several ranks starting at once serialise on a lock file; the
    first one builds, the others find the digest up to date.  Without nvcc an existing library is used as it is
    (with a warning on stderr)."""

    import fcntl
    import sys

    LIB_DIR.mkdir(parents=True, exist_ok=True)
    with open(LIB_DIR / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            return build_all()
        except ContractError as exc:
            if KERNEL_LIB.exists() and "nvcc not found" in str(exc):
                print("research_b200: nvcc not found, using the existing kernel library without checking that it "
                      "matches the sources", file=sys.stderr)
                return None
            raise
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def build_host_only() -> Path | None:
    """Build just the host C++ library (used when only ``libb200host.so`` is missing)."""

    cpp = host_sources()
    if not cpp:
        return None
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    gxx = shutil.which("g++") or "g++"
    _run([gxx, *CXX_FLAGS, "-shared", "-I", str(NATIVE_DIR), "-o", str(HOST_LIB), *[str(s) for s in cpp]])
    return HOST_LIB


if __name__ == "__main__":
    res = build_all(force=bool(os.environ.get("B200_FORCE_BUILD")), verbose=True)
    print(f"kernel library: {res.kernel_lib} (rebuilt={res.rebuilt})")
