"""``profile bench {moe,muon}``: deterministic microbenchmarks of the two communication-heavy components
(reference: src/jaxtitan/runtime/profile_bench.py:17-220 - MoE dispatcher forward+backward under balanced and skewed
routing; muon_bench.py - distributed-Muon candidates).

Runs on the ranks of the current launch (one is fine): with more than one rank the MoE cases shard the experts over
an ``ep`` axis made of all ranks, and with four ranks also over ``ep=2 x expert_fsdp=2`` with each expert's
intermediate dimension split over the second axis (the counterpart of the reference's ``tp2_ep2`` mesh).  Inputs,
weights and routing are fixed functions of their indices; routing is forced (every token to its round-robin experts,
or every token to the first ``top_k`` experts) so that a run measures the dispatch / grouped GEMM / combine path under
a known load and not the router.  Timings are directional: ``timing_is_acceptance_gate`` is false.
"""

from __future__ import annotations

import json
import time
from pathlib import Path
from statistics import median
from typing import Any, Mapping

import torch

from research_b200.errors import ContractError

PROFILE_BENCHMARK_SCHEMA_VERSION = 1
MOE_SHAPES = (  # hidden, expert intermediate, experts, top_k, tokens
    (32, 64, 4, 2, 16),
    (256, 128, 8, 2, 2048),
    (1024, 512, 8, 2, 4096),
    (2048, 1024, 64, 8, 8192),
)


def percentile(ordered: list[float], fraction: float) -> float:
    if len(ordered) == 1:
        return float(ordered[0])
    position = fraction * (len(ordered) - 1)
    lower = int(position)
    upper = min(lower + 1, len(ordered) - 1)
    weight = position - lower
    return float(ordered[lower] * (1.0 - weight) + ordered[upper] * weight)


def timing_summary(values: list[float]) -> dict[str, float]:
    ordered = sorted(values)
    return {"median": float(median(ordered)), "p10": percentile(ordered, 0.10), "p90": percentile(ordered, 0.90),
            "min": float(ordered[0]), "max": float(ordered[-1])}


def _timeit(fn, warmup: int, iters: int, device: torch.device) -> dict[str, float]:
    """Milliseconds per call: CUDA events on the launching stream, wall clock on the CPU."""

    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        if device.type == "cuda":
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        else:
            t0 = time.perf_counter()
            fn()
            times.append((time.perf_counter() - t0) * 1e3)
    return timing_summary(times)


class FixedRouter(torch.nn.Module):
    """Stands in for a layer's router: the same expert ids and weights for every call."""

    def __init__(self, expert_ids: torch.Tensor, num_experts: int):
        super().__init__()
        self.expert_ids = expert_ids
        k = expert_ids.shape[-1]
        self.weights = torch.full(expert_ids.shape, 1.0 / k, dtype=torch.float32, device=expert_ids.device)
        self.scores = torch.full((*expert_ids.shape[:-1], num_experts), 1.0 / num_experts, dtype=torch.float32,
                                 device=expert_ids.device)

    def forward(self, x: torch.Tensor, expert_bias: torch.Tensor):
        return self.expert_ids, self.weights, self.scores


def routing_ids(kind: str, tokens: int, top_k: int, num_experts: int, device: torch.device) -> torch.Tensor:
    if kind == "balanced":
        ids = torch.arange(tokens * top_k, device=device, dtype=torch.int64).view(1, tokens, top_k) % num_experts
    elif kind == "skewed":
        ids = torch.arange(top_k, device=device, dtype=torch.int64).expand(1, tokens, top_k).contiguous()
    else:
        raise ContractError(f"unknown routing {kind!r}")
    return ids


def _moe_meshes(world: int) -> list[tuple[str, dict[str, int], dict[str, Any]]]:
    if world == 1:
        return [("local", {"data": 1}, {})]
    meshes = [(f"ep{world}", {"data": 1, "ep": world}, {"expert_parallel": True})]
    if world == 4:
        # the experts over two ranks and each expert's intermediate dimension over the other two
        meshes.append(("ep2_efsdp2", {"fsdp": 1, "ep": 2, "expert_fsdp": 2},
                       {"mode": "fsdp", "expert_parallel": True}))
    return meshes


def benchmark_moe(*, warmup: int, iters: int) -> list[dict[str, Any]]:
    import torch.distributed as dist

    from research_b200.config.specs import (MeshSpec, ModelSpec, MoeBalanceSpec, ParallelismSpec, TrinityMoeSpec,
                                            TrinitySpec)
    from research_b200.models.moe import SparseMoE
    from research_b200.parallel.mesh import build_mesh_context, execution_context_for, init_distributed

    init_distributed()
    device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    world = dist.get_world_size() if dist.is_initialized() else 1
    cases = []
    for mesh_name, axes, par in _moe_meshes(world):
        parallelism = ParallelismSpec(**{"mode": "ddp", **par})
        mesh = build_mesh_context(MeshSpec(axis_names=tuple(axes), axis_sizes=tuple(axes.values())), device=device)
        ex = execution_context_for(mesh, parallelism)
        for hidden, inter, experts, top_k, tokens in MOE_SHAPES:
            if device.type == "cpu" and hidden > 256:
                continue
            if experts % max(ex.ep_size, 1) or tokens % max(ex.ep_size, 1):
                continue
            moe_spec = TrinityMoeSpec(num_experts=experts, top_k=top_k, expert_intermediate_size=inter,
                                      capacity_factor=None, balance=MoeBalanceSpec())
            spec = ModelSpec(name="trinity", variant="bench", vocab_size=256, hidden_size=hidden,
                             intermediate_size=inter, num_layers=2, num_heads=max(hidden // 128, 2),
                             max_seq_len=tokens,
                             trinity=TrinitySpec(initial_dense_layers=1, local_window=16, local_layers_per_global=1,
                                                 moe=moe_spec))
            with torch.device(device):
                layer = SparseMoE(spec, spec.trinity.moe, ex)
            with torch.no_grad():
                for p in layer.parameters():
                    if p.dtype.is_floating_point and p.numel() > experts:
                        # a fixed function of the index, the same on every rank and run
                        flat = torch.arange(p.numel(), device=device, dtype=torch.float32)
                        p.copy_((((flat * 0.6180339887) % 1.0) - 0.5).mul_(0.04).view_as(p))
            layer = layer.to(dtype)
            base = torch.arange(tokens * hidden, device=device, dtype=torch.float32).view(1, tokens, hidden)
            x = (((base * 0.7548776662) % 1.0) - 0.5).to(dtype).requires_grad_(True)
            for routing in ("balanced", "skewed"):
                layer.router = FixedRouter(routing_ids(routing, tokens, top_k, experts, device), experts)

                def step():
                    y, _, _ = layer(x, ex, name="bench", layer_index=0)
                    y.float().square().mean().backward()

                started = time.perf_counter()
                step()                                  # first call: workspaces, plans, kernels loaded
                if device.type == "cuda":
                    torch.cuda.synchronize()
                first_call_sec = time.perf_counter() - started
                timing = _timeit(step, warmup, iters, device)
                flops = 3 * 2 * 3 * tokens * top_k * hidden * inter
                cases.append({
                    "name": f"{mesh_name}_{routing}_h{hidden}", "mesh": dict(axes), "routing": routing,
                    "shape": {"tokens": tokens, "hidden": hidden, "intermediate": inter, "experts": experts,
                              "top_k": top_k},
                    "workload": "forward_backward", "dtype": str(dtype).replace("torch.", ""),
                    "compile_sec": first_call_sec, "timing_ms": timing,
                    "tflops": flops / (timing["median"] * 1e-3) / 1e12,
                    "max_tokens_on_one_expert": tokens if routing == "skewed" else -(-tokens * top_k // experts)})
    return cases


def benchmark_component(component: str, *, warmup: int = 3, iters: int = 10, artifact_dir: str | None = None,
                        trace: bool = False) -> dict[str, Any]:
    if component not in ("moe", "muon"):
        raise ContractError(f"unsupported profile benchmark component {component!r}")
    if warmup < 0:
        raise ContractError(f"profile benchmark warmup must be non-negative, got {warmup}")
    if iters <= 0:
        raise ContractError(f"profile benchmark iterations must be positive, got {iters}")
    if trace and not artifact_dir:
        raise ContractError("profile benchmark tracing requires --artifact-dir")
    if trace and component != "muon":
        raise ContractError("profile benchmark tracing is currently supported only for Muon")
    device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    envelope = {
        "schema_version": PROFILE_BENCHMARK_SCHEMA_VERSION, "component": component,
        "kind": "directional_local_microbenchmark", "backend": device.type,
        "device_kind": torch.cuda.get_device_name(device) if device.type == "cuda" else "cpu",
        "device": str(device), "warmup": warmup, "iters": iters, "timing_is_acceptance_gate": False,
    }
    if component == "moe":
        cases = benchmark_moe(warmup=warmup, iters=iters)
        import torch.distributed as dist

        report = {**envelope, "device_count": dist.get_world_size() if dist.is_initialized() else 1,
                  "dtype": cases[0]["dtype"] if cases else None, "correctness_is_checked": False,
                  "known_correctness_constraint": None, "measurement_contract": None, "cases": cases}
    else:
        from research_b200.runtime.muon_bench import benchmark_muon

        muon = benchmark_muon(warmup=warmup, iters=iters, artifact_dir=artifact_dir)
        report = {**envelope, **muon, "device_count": muon.get("tp_size"), "correctness_is_checked": True,
                  "known_correctness_constraint": "duplicated_five_step_calibrated_envelope",
                  "measurement_contract": {**muon["contract"], "reducer": "median",
                                           "timer": "host_clock_around_a_synchronised_step_max_over_ranks"}}
    if artifact_dir:
        out = Path(artifact_dir)
        out.mkdir(parents=True, exist_ok=True)
        (out / f"{component}_bench.json").write_text(benchmark_to_json(report))
    return report


def benchmark_to_json(payload: Mapping[str, Any]) -> str:
    return json.dumps(payload, sort_keys=True, separators=(",", ":"))


def format_benchmark(payload: Mapping[str, Any]) -> str:
    """One line per case; the Muon cases list their candidates (reference: profile_bench.py:101-127)."""

    lines = [f"profile benchmark: component={payload['component']} backend={payload['backend']} "
             f"device={payload['device_kind']} devices={payload.get('device_count')} timing_gate=false "
             f"correctness_check={str(bool(payload['correctness_is_checked'])).lower()}"]
    for case in payload["cases"]:
        if "timing_ms" in case:
            t = case["timing_ms"]
            lines.append(f"  {case['name']}: first_call={case['compile_sec']:.3f}s median={t['median']:.3f}ms "
                         f"p10={t['p10']:.3f}ms p90={t['p90']:.3f}ms tflops={case['tflops']:.2f}")
            continue
        name = case.get("case", case.get("name"))
        if "skipped" in case:
            lines.append(f"  {name}: skipped ({case['skipped']})")
            continue
        lines.append(f"  {name}: shape={case.get('logical_shape')} leaves={case.get('leaf_count')} "
                     f"selected={case.get('selected')}")
        for cand in case.get("candidates") or []:
            med = (cand.get("timing_ms") or {}).get("median")
            lines.append(f"    {cand.get('execution')}: median={'n/a' if med is None else f'{med:.3f}ms'} "
                         f"correct={str(bool(cand.get('correctness_gate'))).lower()}")
    return "\n".join(lines)
