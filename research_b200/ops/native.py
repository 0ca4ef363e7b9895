"""ctypes binding of the in-tree sm_100a kernel library (``ops/_lib/libb200ops.so``).

Every wrapper takes torch CUDA tensors, launches on torch's current stream and raises
:class:`KernelError` if the launcher rejects its arguments.  Kernels with bounded device-side waits
report through a per-device status word that :func:`check_status` reads (a synchronising call meant
for tests and for the end of a step, not for the hot path).

``LAUNCHES`` counts kernel launches issued through this module; ``bench.py`` reports it.
"""

from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

from research_b200.errors import KernelError

_LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libb200ops.so"
_lib: ctypes.CDLL | None = None
_lock = threading.Lock()
_status: dict[int, torch.Tensor] = {}
_scratch: dict[tuple[int, str], torch.Tensor] = {}

LAUNCHES = 0

# Debugging switch (``RESEARCH_B200_DETERMINISTIC=1``): every sum whose order depends on which CTA or GPU arrives first
# takes a fixed-order form instead, so that a whole training step is bit-for-bit repeatable (slower).
_DETERMINISTIC = os.environ.get("RESEARCH_B200_DETERMINISTIC", "0") == "1"


def deterministic() -> bool:
    return _DETERMINISTIC


def set_deterministic(enabled: bool) -> None:
    global _DETERMINISTIC
    _DETERMINISTIC = bool(enabled)

c_void_p, c_int, c_ll, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def load() -> ctypes.CDLL:
    """Load the kernel library, building it first when the shared object is missing or stale."""

    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            from research_b200.kernels.build import ensure_current

            ensure_current()          # builds when missing, rebuilds when the sources changed since the last build
            if not _LIB_PATH.exists():
                raise KernelError(f"native kernel library is missing: {_LIB_PATH}")
            lib = ctypes.CDLL(str(_LIB_PATH))
            _declare(lib)
            _lib = lib
    return _lib


def _declare(lib: ctypes.CDLL) -> None:
    def sig(name: str, *argtypes) -> None:
        fn = getattr(lib, name, None)
        if fn is None:
            return
        fn.argtypes = list(argtypes)
        fn.restype = c_int

    sig("b200_gemm_bf16", c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_ll, c_ll, c_ll,
        c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p)
    sig("b200_rmsnorm_fwd", c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p)
    sig("b200_rmsnorm_bwd", c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p)
    sig("b200_qknorm_rope_fwd", c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int,
        c_float, c_float, c_int, c_void_p)
    sig("b200_qknorm_rope_bwd", c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_void_p,
        c_ll, c_int, c_int, c_float, c_int, c_void_p)
    sig("b200_qknorm_rope_fwd_qk", c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int,
        c_int, c_int, c_float, c_float, c_int, c_void_p)
    sig("b200_qknorm_rope_bwd_qk", c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_void_p,
        c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_float, c_int, c_void_p)
    sig("b200_swiglu_fwd", c_void_p, c_void_p, c_ll, c_int, c_void_p)
    sig("b200_swiglu_bwd", c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p)
    sig("b200_sigmoid_gate_fwd", c_void_p, c_void_p, c_void_p, c_ll, c_void_p)
    sig("b200_sigmoid_gate_bwd", c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_void_p)
    sig("b200_embedding_fwd", c_void_p, c_void_p, c_void_p, c_ll, c_int, c_float, c_void_p)
    sig("b200_embedding_bwd", c_void_p, c_void_p, c_void_p, c_ll, c_int, c_float, c_void_p)
    sig("b200_ce_fwd_bwd", c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
        c_float, c_int, c_void_p, c_void_p)
    sig("b200_adamw", c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_ll, c_float, c_float, c_float,
        c_float, c_float, c_float, c_float, c_void_p)
    sig("b200_sumsq", c_void_p, c_int, c_ll, c_void_p, c_void_p, c_int, c_void_p)
    sig("b200_cast_f32_bf16", c_void_p, c_void_p, c_ll, c_float, c_void_p)
    sig("b200_gemm_bf16_grouped_rows", c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_ll,
        c_int, c_int, c_int, c_void_p, c_void_p, c_void_p)
    sig("b200_gemm_bf16_grouped_k", c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_ll,
        c_int, c_int, c_void_p, c_void_p, c_void_p)
    sig("b200_muon_momentum", c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_float, c_int, c_void_p)
    sig("b200_muon_apply", c_void_p, c_void_p, c_void_p, c_ll, c_float, c_float, c_void_p)
    sig("b200_muon_momentum_batched", c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_int, c_float,
        c_int, c_void_p)
    sig("b200_muon_apply_batched", c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_int, c_float, c_float, c_void_p)
    sig("b200_scale_by_inv_norm", c_void_p, c_void_p, c_ll, c_int, c_float, c_void_p)
    sig("b200_affine_identity", c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_void_p)
    sig("b200_dion2_accumulate", c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_int,
        c_int, c_void_p)
    sig("b200_dion2_select", c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p)
    sig("b200_dion2_gather", c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_ll, c_int, c_float,
        c_void_p)
    sig("b200_dion2_apply", c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_ll, c_int,
        c_float, c_float, c_float, c_void_p)
    sig("b200_gemm_bf16_splitk_acc", c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_int,
        c_int, c_void_p, c_void_p)
    sig("b200_gemm_bf16_splitk", c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_void_p,
        c_void_p)
    sig("b200_gemm_bf16_splitk_fused", c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_ll,
        c_ll, c_ll, c_ll, c_void_p, c_void_p)
    sig("b200_sample_topk", c_void_p, c_ll, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p)
    sig("b200_decode_attn_splits", c_int, c_int, c_int, c_int)
    sig("b200_decode_attn", c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
        c_int, c_int, c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_int, c_float, c_int, c_void_p)
    sig("b200_decode_attn_paged", c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
        c_int, c_int, c_int, c_ll, c_ll, c_ll, c_int, c_float, c_int, c_ll, c_void_p, c_void_p)
    sig("b200_decode_attn_paged_splits", c_int, c_int, c_int, c_int)
    sig("b200_splitk_finish", c_void_p, c_void_p, c_ll, c_void_p)
    sig("b200_kv_append", c_void_p, c_void_p, c_ll, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_ll, c_ll, c_int,
        c_int, c_int, c_int, c_void_p)
    sig("b200_attn_fwd", c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
        c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_float, c_int, c_ll, c_void_p, c_void_p)
    sig("b200_attn_bwd", c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
        c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_ll,
        c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_float, c_int, c_ll, c_void_p, c_void_p)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def peer_wait_limit_ms() -> int:
    """Limit of one cross-GPU wait inside a kernel, in milliseconds (``RESEARCH_B200_PEER_WAIT_MS``, default 30 s).

    It has to sit well above the skew between ranks that the host can cause (a trace export on one rank, a slow
    data read, a garbage-collection pause): a wait that gives up makes its kernel skip the dependent work."""

    return max(1, int(os.environ.get("RESEARCH_B200_PEER_WAIT_MS", "30000")))


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    """Four int32 words per device that every kernel with a bounded wait gets: [0] first error code (0 = none),
    [2] the cross-GPU wait limit in milliseconds (read by the kernels), [1] and [3] unused."""

    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    if dev is None:
        dev = torch.cuda.current_device()
    buf = _status.get(dev)
    if buf is None:
        buf = torch.tensor([0, 0, peer_wait_limit_ms(), 0], dtype=torch.int32, device=f"cuda:{dev}")
        _status[dev] = buf
    return buf


def set_peer_wait_limit_ms(ms: int, device: torch.device | int | None = None) -> None:
    """Change the cross-GPU wait limit of the kernels launched after this call on ``device``."""

    status_word(device)[2:3].fill_(max(1, int(ms)))


def status_code_tensor(device: torch.device | int | None = None) -> torch.Tensor:
    """The error-code word as a 1-element device tensor (no synchronisation): callers fold it into a device vector
    that goes to the host anyway."""

    return status_word(device)[0:1]


def raise_for_status_code(code: int, device: torch.device | int | None = None) -> None:
    """Raise :class:`KernelError` for a non-zero status code that the caller already holds on the host, and clear
    the device word so that the next check starts clean."""

    if int(code) != 0:
        status_word(device)[0:1].zero_()
        raise KernelError(f"device-side bounded wait ran out (status code {int(code)})")


def check_status(device: torch.device | int | None = None) -> None:
    """Synchronise and raise if a kernel's bounded wait ran out since the last check."""

    raise_for_status_code(int(status_word(device)[0].item()), device)


def scratch(name: str, numel: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    key = (device.index if device.index is not None else torch.cuda.current_device(), name)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < numel or buf.dtype != dtype:
        buf = torch.empty(numel, dtype=dtype, device=device)
        _scratch[key] = buf
    return buf


def _check(rc: int, what: str) -> None:
    global LAUNCHES
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")
    LAUNCHES += 1


# --------------------------------------------------------------------------------------------------
# GEMM
# --------------------------------------------------------------------------------------------------
def gemm(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = True,
         out: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16, accumulate: bool = False,
         bn: int = 0) -> torch.Tensor:
    """``C = op(A) @ op(B)`` with bf16 inputs and fp32 accumulation on the tcgen05 tensor cores.

    ``trans_a=False``: ``a`` is ``[..., M, K]``; ``True``: ``a`` is ``[..., K, M]``.
    ``trans_b=True`` : ``b`` is ``[..., N, K]`` (``y = x @ w.T``); ``False``: ``b`` is ``[..., K, N]``.
    Leading batch dimension (at most one) must match.  Rows may be strided; the last dim is dense.
    """

    lib = load()
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise KernelError("gemm expects bf16 operands")
    if a.dim() == 2:
        a3, b3 = a.unsqueeze(0), b.unsqueeze(0)
    else:
        a3, b3 = a, b
    if a3.dim() != 3 or b3.dim() != 3 or a3.shape[0] != b3.shape[0]:
        raise KernelError(f"gemm batch shapes do not match: {tuple(a.shape)} x {tuple(b.shape)}")
    if a3.stride(-1) != 1 or b3.stride(-1) != 1:
        raise KernelError("gemm operands need a dense last dimension")
    batch = a3.shape[0]
    M, K = (a3.shape[2], a3.shape[1]) if trans_a else (a3.shape[1], a3.shape[2])
    N, Kb = (b3.shape[1], b3.shape[2]) if trans_b else (b3.shape[2], b3.shape[1])
    if K != Kb:
        raise KernelError(f"gemm inner dimensions differ: {K} vs {Kb}")
    if out is None:
        shape = (batch, M, N) if a.dim() == 3 else (M, N)
        out = torch.empty(shape, dtype=out_dtype, device=a.device)
        if accumulate:
            out.zero_()
    c3 = out.unsqueeze(0) if out.dim() == 2 else out
    if c3.stride(-1) != 1 or c3.shape != (batch, M, N):
        raise KernelError("gemm output has the wrong shape or a strided last dimension")
    rc = lib.b200_gemm_bf16(
        a3.data_ptr(), b3.data_ptr(), c3.data_ptr(), M, N, K, batch,
        a3.stride(1), b3.stride(1), c3.stride(1),
        a3.stride(0) if batch > 1 else 0, b3.stride(0) if batch > 1 else 0, c3.stride(0) if batch > 1 else 0,
        int(trans_a), int(not trans_b), int(out.dtype == torch.float32), int(accumulate), bn,
        status_word(a.device).data_ptr(), _stream())
    _check(rc, "b200_gemm_bf16")
    return out


# --------------------------------------------------------------------------------------------------
# normalisation / activation / embedding / loss / optimizer
# --------------------------------------------------------------------------------------------------
def wave_splits(m: int, n: int, k: int, sms: int = 148, max_splits: int = 8) -> int:
    """K slices for an accumulated product with few output tiles: the smallest count (a divisor of ``k / 64``,
    slices of at least 1024) whose ``tiles * splits`` fills whole waves of ``sms`` CTAs best."""

    tiles = ((m + 127) // 128) * ((n + 255) // 256)
    kblocks = k // 64
    best, best_eff = 1, 0.0
    for s in range(1, max_splits + 1):
        if kblocks % s or k // s < 1024:
            continue
        work = tiles * s
        eff = work / (-(-work // sms) * sms)
        if eff > best_eff + 0.02:
            best, best_eff = s, eff
    return best


def gemm_wgrad(dy: torch.Tensor, x: torch.Tensor, grad: torch.Tensor) -> None:
    """``grad[M, N] (fp32) += dy[K, M]^T @ x[K, N]`` with the contraction over tokens cut into slices so that the
    few output tiles fill whole waves of CTAs (the partial sums are reduce-added into ``grad`` either way)."""

    K, M = dy.shape
    N = x.shape[1]
    splits = 1
    if (K % 64 == 0 and dy.stride(1) == 1 and x.stride(1) == 1 and grad.dim() == 2 and grad.stride(1) == 1
            and not _DETERMINISTIC):         # slices are reduce-added in arrival order
        splits = wave_splits(M, N, K)
    if splits == 1:
        gemm(dy, x, trans_a=True, trans_b=False, out=grad, accumulate=True)
        return
    lib = load()
    rc = lib.b200_gemm_bf16_splitk_acc(dy.data_ptr(), x.data_ptr(), grad.data_ptr(), M, N, K, splits, dy.stride(0),
                                       x.stride(0), grad.stride(0), 1, 1, status_word(dy.device).data_ptr(), _stream())
    _check(rc, "b200_gemm_bf16_splitk_acc")


def splitk_factor(n: int, k: int, sms: int = 148) -> int:
    """How many K slices a skinny ``[rows, k] x [n, k]^T`` product should be cut into so that about one CTA per SM
    streams the weight (its four-stage ring keeps enough bytes in flight; more slices only add reduce traffic:
    measured 39 us against 45 us per decoder layer with two CTAs per SM): a divisor of ``k / 64`` that leaves
    slices of at least 128."""

    tiles = (n + 255) // 256
    kblocks = k // 64
    best = 1
    for d in range(1, kblocks + 1):
        if kblocks % d or k // d < 128 or tiles * d > sms:
            continue
        best = d
    return best


def gemm_skinny(a: torch.Tensor, b: torch.Tensor, fused_finish: bool | None = None) -> torch.Tensor:
    """``a [rows, K] @ b [N, K]^T`` for a handful of rows (decode): split-K so that the whole device streams ``b``.
    Returns bf16 ``[rows, N]``.  ``fused_finish``: let the CTA that adds the last slice of a tile convert it inside the
    product (default: ``RESEARCH_B200_SPLITK_FUSED``, off: inside a CUDA graph the separate 3 us finishing kernel
    measured cheaper than the counters, fences and barriers that the fused form adds to every CTA)."""

    lib = load()
    rows, K = a.shape
    N = b.shape[0]
    if K % 64 or a.stride(1) != 1 or b.stride(1) != 1:
        return gemm(a, b, trans_b=True)
    splits = splitk_factor(N, K)
    if splits == 1:
        return gemm(a, b, trans_b=True)
    if N % 4:
        c = torch.zeros((rows, N), dtype=torch.float32, device=a.device)
        rc = lib.b200_gemm_bf16_splitk(a.data_ptr(), b.data_ptr(), c.data_ptr(), rows, N, K, splits, a.stride(0),
                                       b.stride(0), c.stride(0), status_word(a.device).data_ptr(), _stream())
        _check(rc, "b200_gemm_bf16_splitk")
        return c.to(torch.bfloat16)
    # the slices add into a persistent fp32 workspace that is zero between calls; a finishing pass (a small kernel,
    # or the CTA that adds the last slice of a tile) converts the sums to bf16 and clears the workspace behind it,
    # so a decode step runs no fill and no cast per linear
    ws = _splitk_workspace(rows * N, a.device)
    out = torch.empty((rows, N), dtype=torch.bfloat16, device=a.device)
    try:
        if rows <= 128 and (fused_finish if fused_finish is not None
                            else os.environ.get("RESEARCH_B200_SPLITK_FUSED", "0") == "1"):
            counters = _splitk_counters(a.device)
            rc = lib.b200_gemm_bf16_splitk_fused(a.data_ptr(), b.data_ptr(), ws.data_ptr(), out.data_ptr(),
                                                 counters.data_ptr(), rows, N, K, splits, a.stride(0), b.stride(0), N,
                                                 N, status_word(a.device).data_ptr(), _stream())
            _check(rc, "b200_gemm_bf16_splitk_fused")
            return out
        rc = lib.b200_gemm_bf16_splitk(a.data_ptr(), b.data_ptr(), ws.data_ptr(), rows, N, K, splits, a.stride(0),
                                       b.stride(0), N, status_word(a.device).data_ptr(), _stream())
        _check(rc, "b200_gemm_bf16_splitk")
        _check(lib.b200_splitk_finish(ws.data_ptr(), out.data_ptr(), rows * N, _stream()), "b200_splitk_finish")
    except Exception:
        _splitk_ws.pop(_device_index(a.device), None)      # its contents are unknown now: start from a fresh one
        _splitk_cnt.pop(_device_index(a.device), None)
        raise
    return out


_splitk_ws: dict[int, torch.Tensor] = {}
_splitk_cnt: dict[int, torch.Tensor] = {}


def _splitk_counters(device: torch.device) -> torch.Tensor:
    """One uint32 per output tile of a fused split-K product (N up to 2^20 columns); zero between launches."""

    key = _device_index(device)
    cnt = _splitk_cnt.get(key)
    if cnt is None:
        cnt = torch.zeros(8192, dtype=torch.int32, device=device)
        _splitk_cnt[key] = cnt
    return cnt


def _device_index(device: torch.device) -> int:
    return device.index if device.index is not None else torch.cuda.current_device()


def _splitk_workspace(numel: int, device: torch.device) -> torch.Tensor:
    key = _device_index(device)
    ws = _splitk_ws.get(key)
    if ws is None or ws.numel() < numel:
        ws = torch.zeros(max(numel, 1 << 20), dtype=torch.float32, device=device)
        _splitk_ws[key] = ws
    return ws


def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float, delta: torch.Tensor | None = None):
    """Returns ``(y, rstd, residual)``; ``residual = x + delta`` when ``delta`` is given, else ``x``."""

    lib = load()
    H = x.shape[-1]
    rows = x.numel() // H
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    res = torch.empty_like(x) if delta is not None else None
    rc = lib.b200_rmsnorm_fwd(x.data_ptr(), _ptr(delta), w.data_ptr(), _ptr(res), y.data_ptr(), rstd.data_ptr(), rows, H,
                              eps, _stream())
    _check(rc, "b200_rmsnorm_fwd")
    return y, rstd, (res if res is not None else x)


def rmsnorm_bwd(x: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor, dy: torch.Tensor, dw: torch.Tensor,
                dres: torch.Tensor | None = None) -> torch.Tensor:
    """dx (+ dres); ``dw`` (fp32) is accumulated into."""

    lib = load()
    H = x.shape[-1]
    rows = x.numel() // H
    dx = torch.empty_like(x)
    rc = lib.b200_rmsnorm_bwd(x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dy.data_ptr(), _ptr(dres), dx.data_ptr(),
                              dw.data_ptr(), rows, H, _stream())
    _check(rc, "b200_rmsnorm_bwd")
    return dx


def qknorm_rope_fwd(inp: torch.Tensor, out: torch.Tensor, w: torch.Tensor | None, positions: torch.Tensor,
                    heads: int, head_dim: int, eps: float, theta: float, rope: bool):
    """inp/out: 2-D ``[tokens, row_stride]`` views whose first ``heads*head_dim`` columns are the heads."""

    lib = load()
    tokens = inp.shape[0]
    rstd = torch.empty(tokens * heads, dtype=torch.float32, device=inp.device) if w is not None else None
    rc = lib.b200_qknorm_rope_fwd(inp.data_ptr(), inp.stride(0), out.data_ptr(), out.stride(0), _ptr(w),
                                  positions.data_ptr(), _ptr(rstd), tokens, heads, head_dim, eps, theta, int(rope),
                                  _stream())
    _check(rc, "b200_qknorm_rope_fwd")
    return rstd


def qknorm_rope_bwd(inp: torch.Tensor, dout: torch.Tensor, din: torch.Tensor, w: torch.Tensor | None,
                    positions: torch.Tensor, rstd: torch.Tensor | None, dw: torch.Tensor | None, heads: int,
                    head_dim: int, theta: float, rope: bool) -> None:
    lib = load()
    rc = lib.b200_qknorm_rope_bwd(inp.data_ptr(), inp.stride(0), dout.data_ptr(), dout.stride(0), din.data_ptr(),
                                  din.stride(0), _ptr(w), positions.data_ptr(), _ptr(rstd), _ptr(dw), inp.shape[0],
                                  heads, head_dim, theta, int(rope), _stream())
    _check(rc, "b200_qknorm_rope_bwd")


def qknorm_rope_fwd_qk(inp: torch.Tensor, out: torch.Tensor, wq, wk, positions: torch.Tensor, heads_q: int,
                       heads_k: int, head_dim: int, eps: float, theta: float, rope: bool):
    """Query and key heads of a packed projection in one launch (``wq`` / ``wk``: both given or both None).
    Returns ``rstd`` ``[tokens * (heads_q + heads_k)]`` (None without norm weights)."""

    lib = load()
    tokens = inp.shape[0]
    rstd = None
    if wq is not None:
        rstd = torch.empty(tokens * (heads_q + heads_k), dtype=torch.float32, device=inp.device)
    rc = lib.b200_qknorm_rope_fwd_qk(inp.data_ptr(), inp.stride(0), out.data_ptr(), out.stride(0), _ptr(wq), _ptr(wk),
                                     positions.data_ptr(), _ptr(rstd), tokens, heads_q, heads_k, head_dim, eps, theta,
                                     int(rope), _stream())
    _check(rc, "b200_qknorm_rope_fwd_qk")
    return rstd


def qknorm_rope_bwd_qk(inp: torch.Tensor, dout: torch.Tensor, din: torch.Tensor, wq, wk, positions: torch.Tensor,
                       rstd, dwq, dwk, heads_q: int, heads_k: int, head_dim: int, theta: float, rope: bool) -> None:
    lib = load()
    rc = lib.b200_qknorm_rope_bwd_qk(inp.data_ptr(), inp.stride(0), dout.data_ptr(), dout.stride(0), din.data_ptr(),
                                     din.stride(0), _ptr(wq), _ptr(wk), positions.data_ptr(), _ptr(rstd), _ptr(dwq),
                                     _ptr(dwk), inp.shape[0], heads_q, heads_k, head_dim, theta, int(rope), _stream())
    _check(rc, "b200_qknorm_rope_bwd_qk")


def swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    lib = load()
    inter = gu.shape[-1] // 2
    rows = gu.numel() // (2 * inter)
    h = torch.empty(*gu.shape[:-1], inter, dtype=gu.dtype, device=gu.device)
    _check(lib.b200_swiglu_fwd(gu.data_ptr(), h.data_ptr(), rows, inter, _stream()), "b200_swiglu_fwd")
    return h


def swiglu_bwd(gu: torch.Tensor, dh: torch.Tensor) -> torch.Tensor:
    lib = load()
    inter = gu.shape[-1] // 2
    rows = gu.numel() // (2 * inter)
    dgu = torch.empty_like(gu)
    _check(lib.b200_swiglu_bwd(gu.data_ptr(), dh.data_ptr(), dgu.data_ptr(), rows, inter, _stream()), "b200_swiglu_bwd")
    return dgu


def sigmoid_gate_fwd(a: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    lib = load()
    out = torch.empty_like(a)
    _check(lib.b200_sigmoid_gate_fwd(a.data_ptr(), gate.data_ptr(), out.data_ptr(), a.numel(), _stream()),
           "b200_sigmoid_gate_fwd")
    return out


def sigmoid_gate_bwd(a: torch.Tensor, gate: torch.Tensor, dout: torch.Tensor):
    lib = load()
    da, dg = torch.empty_like(a), torch.empty_like(gate)
    _check(lib.b200_sigmoid_gate_bwd(a.data_ptr(), gate.data_ptr(), dout.data_ptr(), da.data_ptr(), dg.data_ptr(),
                                     a.numel(), _stream()), "b200_sigmoid_gate_bwd")
    return da, dg


def embedding_fwd(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    lib = load()
    H = table.shape[1]
    out = torch.empty(*ids.shape, H, dtype=table.dtype, device=table.device)
    _check(lib.b200_embedding_fwd(ids.data_ptr(), table.data_ptr(), out.data_ptr(), ids.numel(), H, scale, _stream()),
           "b200_embedding_fwd")
    return out


def embedding_bwd(ids: torch.Tensor, dout: torch.Tensor, dtable: torch.Tensor, scale: float = 1.0) -> None:
    lib = load()
    H = dtable.shape[1]
    _check(lib.b200_embedding_bwd(ids.data_ptr(), dout.data_ptr(), dtable.data_ptr(), ids.numel(), H, scale, _stream()),
           "b200_embedding_bwd")


def ce_fwd_bwd(logits: torch.Tensor, targets: torch.Tensor, mask: torch.Tensor, grad_scale: float, z_weight: float,
               write_grad: bool = True):
    """Per-row loss and lse^2 for one ``[rows, V]`` bf16 chunk; ``logits`` becomes ``dlogits`` in place."""

    lib = load()
    rows, V = logits.shape
    loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    z = torch.empty(rows, dtype=torch.float32, device=logits.device)
    lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
    rc = lib.b200_ce_fwd_bwd(logits.data_ptr(), logits.stride(0), targets.data_ptr(), mask.data_ptr(), loss.data_ptr(),
                             z.data_ptr(), lse.data_ptr(), rows, V, grad_scale, z_weight, int(write_grad),
                             status_word(logits.device).data_ptr(), _stream())
    _check(rc, "b200_ce_fwd_bwd")
    return loss, z, lse


def adamw(p: torch.Tensor, m: torch.Tensor, v: torch.Tensor, g: torch.Tensor, shadow: torch.Tensor | None,
          gscale: torch.Tensor | None, lr: float, b1: float, b2: float, eps: float, wd: float, step: int) -> None:
    lib = load()
    bc1 = 1.0 - b1 ** step
    bc2 = 1.0 - b2 ** step
    rc = lib.b200_adamw(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), int(g.dtype == torch.bfloat16),
                        _ptr(shadow), _ptr(gscale), p.numel(), lr, b1, b2, eps, wd, bc1, bc2, _stream())
    _check(rc, "b200_adamw")


def sumsq(x: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    global LAUNCHES
    lib = load()
    sc = scratch("sumsq", 1024, torch.float32, x.device)
    rc = lib.b200_sumsq(x.data_ptr(), int(x.dtype == torch.bfloat16), x.numel(), sc.data_ptr(), out.data_ptr(),
                        int(accumulate), _stream())
    _check(rc, "b200_sumsq")
    LAUNCHES += 1


def cast_f32_bf16(x: torch.Tensor, y: torch.Tensor, scale: float = 1.0) -> None:
    lib = load()
    _check(lib.b200_cast_f32_bf16(x.data_ptr(), y.data_ptr(), x.numel(), scale, _stream()), "b200_cast_f32_bf16")


# --------------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------------
def _check_bshd(t: torch.Tensor, name: str) -> None:
    if t.dim() != 4 or t.stride(3) != 1 or t.stride(2) != t.shape[3]:
        raise KernelError(f"{name} must be a [B,S,H,D] view with heads D elements apart and a dense last dim")


def attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = True,
             lo: torch.Tensor | None = None, scale: float | None = None, q_offset: int = 0):
    """Flash attention forward.  q: ``[B,S,Hq,D]``, k/v: ``[B,S,Hkv,D]`` (views into a packed buffer are fine).

    ``lo`` (int32 ``[B,S]``, non-decreasing along S) is the first kv position each query row may attend to.
    k/v may be longer than q (context parallelism): ``q_offset`` (a multiple of 128) is the global position of
    query row 0 among the kv positions.  Returns ``(o [B,S,Hq,D] bf16, lse [B,Hq,S] fp32)``.
    """

    lib = load()
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_bshd(t, n)
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    o = torch.empty((B, S, Hq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)
    if scale is None:
        scale = D ** -0.5
    rc = lib.b200_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), _ptr(lo), B, S, Hq,
                           Hkv, D, q.stride(1), q.stride(0), k.stride(1), k.stride(0), v.stride(1), v.stride(0),
                           o.stride(1), o.stride(0), scale, int(causal), k.shape[1] | (int(q_offset) << 32),
                           status_word(q.device).data_ptr(), _stream())
    _check(rc, "b200_attn_fwd")
    return o, lse


def kv_visibility_upper_bound(lo: torch.Tensor, kv_len: int | None = None, q_offset: int = 0) -> torch.Tensor:
    """kv-side view of a per-query lower bound: ``hi[b,k]`` = last (global) query position that may attend to
    kv ``k``.  ``lo`` must be non-decreasing along the sequence, so ``hi[k] = q_offset + #{q : lo[q] <= k} - 1``.
    """

    B, S = lo.shape
    n = S if kv_len is None else kv_len
    k = torch.arange(n, device=lo.device, dtype=lo.dtype).expand(B, n).contiguous()
    return (torch.searchsorted(lo.contiguous(), k, right=True) - 1 + q_offset).to(torch.int32)


def attn_bwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, d_o: torch.Tensor,
             lse: torch.Tensor, *, causal: bool = True, lo: torch.Tensor | None = None,
             hi: torch.Tensor | None = None, scale: float | None = None,
             out: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None, q_offset: int = 0):
    """Flash attention backward; returns ``(dq, dk, dv)`` shaped like q, k, v.

    ``out`` may give three ``[B,S,H,D]`` views to write into (for example column ranges of one packed
    gradient buffer); otherwise dense tensors are allocated.
    """

    global LAUNCHES
    lib = load()
    for t, n in ((q, "q"), (k, "k"), (v, "v"), (o, "o"), (d_o, "d_o")):
        _check_bshd(t, n)
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    if scale is None:
        scale = D ** -0.5
    if lo is not None and hi is None:
        hi = kv_visibility_upper_bound(lo)
    if out is None:
        dq = torch.empty((B, S, Hq, D), dtype=q.dtype, device=q.device)
        dk = torch.empty((B, k.shape[1], Hkv, D), dtype=q.dtype, device=q.device)
        dv = torch.empty((B, k.shape[1], Hkv, D), dtype=q.dtype, device=q.device)
    else:
        dq, dk, dv = out
        for t, n in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
            _check_bshd(t, n)
    delta = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)
    rc = lib.b200_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr(),
                           delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), _ptr(lo), _ptr(hi), B, S, Hq,
                           Hkv, D, q.stride(1), q.stride(0), k.stride(1), k.stride(0), v.stride(1), v.stride(0),
                           o.stride(1), o.stride(0), d_o.stride(1), d_o.stride(0), dq.stride(1), dq.stride(0),
                           dk.stride(1), dk.stride(0), dv.stride(1), dv.stride(0), scale, int(causal),
                           k.shape[1] | (int(q_offset) << 32),
                           status_word(q.device).data_ptr(), _stream())
    _check(rc, "b200_attn_bwd")
    LAUNCHES += 2
    return dq, dk, dv


# --------------------------------------------------------------------------------------------------
# Muon element-wise stages
# --------------------------------------------------------------------------------------------------
def muon_momentum(g: torch.Tensor, m: torch.Tensor, u: torch.Tensor, sumsq_slot: torch.Tensor,
                  clip: torch.Tensor | None, beta: float, nesterov: bool) -> None:
    """g, m: fp32 contiguous; u: bf16 contiguous (same numel); sumsq_slot: 1-element fp32 accumulator."""

    lib = load()
    _check(lib.b200_muon_momentum(g.data_ptr(), m.data_ptr(), u.data_ptr(), sumsq_slot.data_ptr(), _ptr(clip),
                                  g.numel(), beta, int(nesterov), _stream()), "b200_muon_momentum")


def muon_momentum_batched(g: torch.Tensor, m: torch.Tensor, u: torch.Tensor, sumsq: torch.Tensor,
                          clip: torch.Tensor | None, per: int, stride: int, batch: int, beta: float,
                          nesterov: bool) -> None:
    """``batch`` matrices of ``per`` elements, ``stride`` elements apart from the first element of ``g`` / ``m``
    (fp32); ``u`` is the dense bf16 ``[batch, per]`` stack; ``sumsq`` has ``batch`` fp32 slots."""

    lib = load()
    _check(lib.b200_muon_momentum_batched(g.data_ptr(), m.data_ptr(), u.data_ptr(), sumsq.data_ptr(), _ptr(clip), per,
                                          stride, batch, beta, int(nesterov), _stream()), "b200_muon_momentum_batched")


def muon_apply_batched(w: torch.Tensor, o: torch.Tensor, shadow: torch.Tensor | None, per: int, stride: int, batch: int,
                       decay: float, step: float) -> None:
    lib = load()
    _check(lib.b200_muon_apply_batched(w.data_ptr(), o.data_ptr(), _ptr(shadow), per, stride, batch, decay, step,
                                       _stream()), "b200_muon_apply_batched")


def muon_apply(w: torch.Tensor, o: torch.Tensor, shadow: torch.Tensor | None, decay: float, step: float) -> None:
    lib = load()
    _check(lib.b200_muon_apply(w.data_ptr(), o.data_ptr(), _ptr(shadow), w.numel(), decay, step, _stream()),
           "b200_muon_apply")


def scale_by_inv_norm(x: torch.Tensor, sumsq_vec: torch.Tensor, eps: float) -> None:
    """x: [batch, ...] bf16 contiguous; every slab is divided by max(sqrt(sumsq[b]), eps)."""

    lib = load()
    batch = x.shape[0]
    _check(lib.b200_scale_by_inv_norm(x.data_ptr(), sumsq_vec.data_ptr(), x.numel() // batch, batch, eps, _stream()),
           "b200_scale_by_inv_norm")


def dion2_supported(n: int, rows: int, cols: int, stride: int, axis: int) -> bool:
    """Size rules of the Dion2 kernels: 16-byte rows, at most 12288 slices on the selected axis."""

    return cols % 4 == 0 and stride % 4 == 0 and 0 < n <= 65535 and (rows if axis == 0 else cols) <= 12288


def dion2_select_stack(g: torch.Tensor, m: torch.Tensor, clip: torch.Tensor | None, n: int, rows: int, cols: int,
                       stride: int, axis: int, k: int, eps: float):
    """First half of a Dion2 update of ``n`` fp32 matrices ``[rows, cols]`` that start ``stride`` elements apart at
    ``g`` / ``m`` (tensors whose first element is the first matrix's first element): ``m += clip * g``, the ``k``
    row (``axis`` 0) or column (``axis`` 1) slices of largest L1 norm, and the normalised bf16 stack of them
    (``[n, k, cols]`` or ``[n, rows, k]``, slices in order of decreasing norm, ties by index).  Returns
    ``(stack, idx [n, k] int32, inv [n, dim] int32)`` where ``inv`` maps a slice to its place in the stack or -1."""

    lib = load()
    dev = m.device
    dim = rows if axis == 0 else cols
    splits = 1
    if axis == 1:
        strips = n * ((cols + 127) // 128)
        splits = max(1, min(16, -(-592 // strips), rows // 64 or 1))
    norms = torch.empty((2, splits, n, dim), dtype=torch.float32, device=dev)
    idx = torch.empty((n, k), dtype=torch.int32, device=dev)
    inv = torch.empty((n, dim), dtype=torch.int32, device=dev)
    sq_sel = torch.empty((n, k), dtype=torch.float32, device=dev)
    stack = torch.empty((n, k, cols) if axis == 0 else (n, rows, k), dtype=torch.bfloat16, device=dev)
    st = _stream()
    _check(lib.b200_dion2_accumulate(g.data_ptr(), m.data_ptr(), _ptr(clip), norms[0].data_ptr(), norms[1].data_ptr(),
                                     n, rows, cols, stride, axis, splits, st), "b200_dion2_accumulate")
    _check(lib.b200_dion2_select(norms[0].data_ptr(), norms[1].data_ptr(), splits, n, dim, k, idx.data_ptr(),
                                 inv.data_ptr(), sq_sel.data_ptr(), st), "b200_dion2_select")
    _check(lib.b200_dion2_gather(m.data_ptr(), idx.data_ptr(), sq_sel.data_ptr(), stack.data_ptr(), n, rows, cols, k,
                                 stride, axis, eps, st), "b200_dion2_gather")
    return stack, idx, inv


def dion2_apply(w: torch.Tensor, m: torch.Tensor, o: torch.Tensor, inv: torch.Tensor, shadow: torch.Tensor | None,
                n: int, rows: int, cols: int, k: int, stride: int, axis: int, decay: float, step: float,
                ef: float) -> None:
    """Second half: ``w <- w * decay - step * o`` on the selected slices (``decay`` everywhere), ``m <- ef * m`` on the
    selected slices, and the bf16 compute copy of all of ``w`` into ``shadow`` (same element offsets as ``w``)."""

    lib = load()
    _check(lib.b200_dion2_apply(w.data_ptr(), m.data_ptr(), o.data_ptr(), inv.data_ptr(), _ptr(shadow), n, rows, cols,
                                k, stride, axis, decay, step, ef, _stream()), "b200_dion2_apply")


def affine_identity(a: torch.Tensor, alpha: float, beta: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """``alpha * I + beta * a`` for a stack of square bf16 matrices ``[batch, d, d]``."""

    lib = load()
    if out is None:
        out = torch.empty_like(a)
    _check(lib.b200_affine_identity(a.data_ptr(), out.data_ptr(), a.shape[-1], a.numel() // (a.shape[-1] ** 2), alpha,
                                    beta, _stream()), "b200_affine_identity")
    return out


# --------------------------------------------------------------------------------------------------
# sampler
# --------------------------------------------------------------------------------------------------
def sample_topk(logits: torch.Tensor, uniform: torch.Tensor, temperature: float, top_k: int | None):
    """logits ``[B, V]`` (bf16 or fp32, dense rows), uniform ``[B]`` fp32 in [0, 1) -> (token int64 [B], logprob fp32 [B])."""

    lib = load()
    if logits.dtype not in (torch.bfloat16, torch.float32) or logits.stride(1) != 1:
        raise KernelError("sample_topk needs bf16 or fp32 logits with a dense last dimension")
    B, V = logits.shape
    token = torch.empty(B, dtype=torch.int64, device=logits.device)
    logprob = torch.empty(B, dtype=torch.float32, device=logits.device)
    uniform = uniform.to(torch.float32).contiguous()
    rc = lib.b200_sample_topk(logits.data_ptr(), logits.stride(0), int(logits.dtype == torch.bfloat16),
                              uniform.data_ptr(), token.data_ptr(), logprob.data_ptr(), B, V, float(temperature),
                              0 if top_k is None else int(top_k), _stream())
    _check(rc, "b200_sample_topk")
    return token, logprob
