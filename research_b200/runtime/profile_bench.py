"""``profile bench {moe,muon}``: deterministic microbenchmarks of the two communication-heavy components
(reference: src/jaxtitan/runtime/profile_bench.py:17-220 - MoE all-to-all dispatcher forward+backward on 4 devices;
muon_bench.py - distributed-Muon candidates).  Runs on however many ranks the process group has (1 is fine)."""

from __future__ import annotations

import json
import time
from pathlib import Path
from typing import Any

import torch

from research_b200.errors import ContractError


def _timeit(fn, warmup: int, iters: int, device: torch.device) -> dict[str, float]:
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        if device.type == "cuda":
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        else:
            t0 = time.perf_counter()
            fn()
            times.append((time.perf_counter() - t0) * 1e3)
    times.sort()
    return {"median_ms": times[len(times) // 2], "min_ms": times[0], "max_ms": times[-1]}


def benchmark_moe(*, warmup: int, iters: int) -> dict[str, Any]:
    from research_b200.config.specs import ModelSpec, MoeBalanceSpec, TrinityMoeSpec, TrinitySpec
    from research_b200.models.execution import ExecutionContext
    from research_b200.models.moe import SparseMoE

    device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    cases = []
    for hidden, inter, experts, top_k, tokens in ((256, 128, 8, 2, 2048), (1024, 512, 8, 2, 4096), (2048, 1024, 64, 8, 8192)):
        if device.type == "cpu" and hidden > 256:
            continue
        moe_spec = TrinityMoeSpec(num_experts=experts, top_k=top_k, expert_intermediate_size=inter,
                                  balance=MoeBalanceSpec())
        spec = ModelSpec(name="trinity", variant="bench", vocab_size=256, hidden_size=hidden, intermediate_size=inter,
                         num_layers=2, num_heads=max(hidden // 128, 1) if hidden >= 128 else 2, max_seq_len=tokens,
                         trinity=TrinitySpec(initial_dense_layers=1, local_window=16, local_layers_per_global=1, moe=moe_spec))
        ex = ExecutionContext()
        with torch.device(device):
            layer = SparseMoE(spec, spec.trinity.moe, ex)
        for p in layer.parameters():
            if p.dtype.is_floating_point and p.requires_grad:
                torch.nn.init.normal_(p, std=0.02)
        layer = layer.to(dtype)
        x = torch.randn(1, tokens, hidden, device=device, dtype=dtype, requires_grad=True)

        def step():
            y, _, _ = layer(x, ex, name="bench", layer_index=0)
            y.float().sum().backward()

        t = _timeit(step, warmup, iters, device)
        flops = 3 * 2 * 3 * tokens * top_k * hidden * inter
        cases.append({"hidden": hidden, "expert_intermediate": inter, "experts": experts, "top_k": top_k,
                      "tokens": tokens, **t, "tflops": flops / (t["median_ms"] * 1e-3) / 1e12})
    return {"schema_version": 1, "component": "moe", "device": str(device), "dtype": str(dtype), "cases": cases}


def benchmark_component(component: str, *, warmup: int = 3, iters: int = 10, artifact_dir: str | None = None,
                        trace: bool = False) -> dict[str, Any]:
    if trace and not artifact_dir:
        raise ContractError("--trace requires --artifact-dir")
    if component == "moe":
        report = benchmark_moe(warmup=warmup, iters=iters)
    elif component == "muon":
        from research_b200.runtime.muon_bench import benchmark_muon

        report = benchmark_muon(warmup=warmup, iters=iters, artifact_dir=artifact_dir)
    else:
        raise ContractError(f"unknown benchmark component {component!r}")
    if artifact_dir:
        out = Path(artifact_dir)
        out.mkdir(parents=True, exist_ok=True)
        (out / f"{component}_bench.json").write_text(json.dumps(report, sort_keys=True, separators=(",", ":")))
    return report
