"""``kernels bench``: p50 / p90 / p99 latency of a native kernel against its PyTorch restatement
(reference: src/jaxtitan/kernels/bench.py:28-74, which benchmarks the RMSNorm kernel against pure JAX)."""

from __future__ import annotations

from typing import Any

import torch

from research_b200.config.specs import RunSpec
from research_b200.errors import ContractError


def _percentiles(ms: list[float]) -> dict[str, float]:
    s = sorted(ms)

    def pick(q: float) -> float:
        return s[min(len(s) - 1, int(round(q * (len(s) - 1))))]

    return {"p50_ms": pick(0.5), "p90_ms": pick(0.9), "p99_ms": pick(0.99), "min_ms": s[0]}


def _time(fn, warmup: int, iters: int) -> list[float]:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b))
    return out


def benchmark_kernel(op: str, spec: RunSpec, *, rows: list[int], warmup: int = 5, iters: int = 20) -> dict[str, Any]:
    if not torch.cuda.is_available():
        raise ContractError("kernels bench needs a CUDA device")
    from research_b200.ops import functional as Fn
    from research_b200.ops import native

    H = spec.model.hidden_size
    dev = torch.device("cuda")
    cases = []
    for r in rows:
        if op == "rmsnorm":
            x = torch.randn(r, H, device=dev, dtype=torch.bfloat16)
            w = torch.ones(H, device=dev)
            mine = lambda: native.rmsnorm_fwd(x, w, spec.model.norm_epsilon)
            ref = lambda: Fn._rmsnorm_ref(x, w, spec.model.norm_epsilon)
        elif op == "gemm":
            a = torch.randn(r, H, device=dev, dtype=torch.bfloat16)
            b = torch.randn(spec.model.intermediate_size, H, device=dev, dtype=torch.bfloat16)
            mine = lambda: native.gemm(a, b)
            ref = lambda: a @ b.t()
        elif op == "attention":
            D, hq, hkv = spec.model.head_dim, spec.model.num_heads, spec.model.n_kv_heads
            q = torch.randn(1, r, hq, D, device=dev, dtype=torch.bfloat16)
            k = torch.randn(1, r, hkv, D, device=dev, dtype=torch.bfloat16)
            v = torch.randn(1, r, hkv, D, device=dev, dtype=torch.bfloat16)
            mine = lambda: native.attn_fwd(q, k, v, causal=True)
            ref = lambda: torch.nn.functional.scaled_dot_product_attention(
                q.transpose(1, 2), k.transpose(1, 2).repeat_interleave(hq // hkv, 1),
                v.transpose(1, 2).repeat_interleave(hq // hkv, 1), is_causal=True)
        else:
            raise ContractError(f"unknown kernel op {op!r}")
        cases.append({"rows": r, "native": _percentiles(_time(mine, warmup, iters)),
                      "pytorch": _percentiles(_time(ref, warmup, iters))})
    native.check_status()
    return {"schema_version": 1, "op": op, "hidden_size": H, "device": torch.cuda.get_device_name(0),
            "warmup": warmup, "iters": iters, "cases": cases}
