"""Kernel registry and plan: which hot ops run on this package's sm_100a kernels for a given run.

The reference's registry is diagnostic - every candidate op falls back to XLA (src/jaxtitan/kernels/registry.py:
29-154).  Here the plan reports kernels that are actually active: on a CUDA device with bf16 compute every listed
op runs natively; on CPU or in fp32 the PyTorch restatement runs and the plan says so.
"""

from __future__ import annotations

from typing import Any

import torch

from research_b200.config.specs import RunSpec
from research_b200.errors import ContractError

KERNEL_CANDIDATES = (
    {"op": "gemm", "source": "gemm.cu", "symbol": "b200_gemm_bf16", "engine": "tcgen05+TMA+TMEM"},
    {"op": "grouped_expert_gemm", "source": "gemm.cu", "symbol": "b200_gemm_bf16_grouped_rows", "engine": "tcgen05+TMA+TMEM"},
    {"op": "attention_forward", "source": "attention_fwd.cu", "symbol": "b200_attn_fwd", "engine": "tcgen05+TMA+TMEM"},
    {"op": "attention_backward", "source": "attention_bwd.cu", "symbol": "b200_attn_bwd", "engine": "tcgen05+TMA+TMEM"},
    {"op": "rmsnorm", "source": "elementwise.cu", "symbol": "b200_rmsnorm_fwd", "engine": "SIMT 128-bit"},
    {"op": "qk_norm_rope", "source": "elementwise.cu", "symbol": "b200_qknorm_rope_fwd", "engine": "SIMT 128-bit"},
    {"op": "swiglu", "source": "elementwise.cu", "symbol": "b200_swiglu_fwd", "engine": "SIMT 128-bit"},
    {"op": "cross_entropy", "source": "elementwise.cu", "symbol": "b200_ce_fwd_bwd", "engine": "SIMT 128-bit"},
    {"op": "embedding", "source": "elementwise.cu", "symbol": "b200_embedding_fwd", "engine": "SIMT 128-bit"},
    {"op": "optimizer_adamw", "source": "elementwise.cu", "symbol": "b200_adamw", "engine": "SIMT"},
    {"op": "optimizer_matrix_update", "source": "gemm.cu", "symbol": "b200_gemm_bf16", "engine": "tcgen05 (Newton-Schulz)"},
    {"op": "decode_attention", "source": "decode.cu", "symbol": "b200_decode_attn", "engine": "SIMT split-KV"},
    {"op": "kv_cache_append", "source": "decode.cu", "symbol": "b200_kv_append", "engine": "SIMT 128-bit"},
    {"op": "sampler", "source": "sampler.cu", "symbol": "b200_sample_topk", "engine": "SIMT radix select"},
    {"op": "moe_dispatch_combine", "source": "moe.cu", "symbol": "b200_moe_gather", "engine": "SIMT + NVLink peer stores/loads"},
    {"op": "moe_routing_plan", "source": "moe.cu", "symbol": "b200_moe_rank", "engine": "SIMT match_any"},
    {"op": "optimizer_muon_elementwise", "source": "optimizer.cu", "symbol": "b200_muon_momentum_batched", "engine": "SIMT"},
    {"op": "gemm_allgather", "source": "comm_gemm.cu", "symbol": "b200_gemm_allgather", "engine": "tcgen05 + TMA peer loads"},
    {"op": "gemm_reduce_scatter", "source": "comm_gemm.cu", "symbol": "b200_gemm_reducescatter", "engine": "tcgen05 + TMA peer reduce-add"},
    {"op": "grad_reduce_scatter", "source": "comm_runtime.cu", "symbol": "b200c_reduce_scatter_pull", "engine": "SIMT peer loads"},
    {"op": "weight_all_gather", "source": "comm_runtime.cu", "symbol": "b200c_all_gather_pull", "engine": "SIMT peer loads"},
)

# ops that only some runs need (generation, multi-GPU layouts, MoE): never a reason for kernels.strict to refuse
OPTIONAL_OPS = ("decode_attention", "kv_cache_append", "sampler", "moe_dispatch_combine", "moe_routing_plan",
                "gemm_allgather", "gemm_reduce_scatter", "grad_reduce_scatter", "weight_all_gather",
                "grouped_expert_gemm")


def kernel_registry() -> list[dict[str, Any]]:
    from research_b200.ops import native

    lib = native.load() if native.available() else None
    out = []
    for item in KERNEL_CANDIDATES:
        row = dict(item)
        row["built"] = bool(lib is not None and hasattr(lib, item["symbol"]))
        out.append(row)
    return out


def kernel_plan(spec: RunSpec, *, device: torch.device | None = None) -> dict[str, Any]:
    from research_b200.ops import native

    device = device or (torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu"))
    bf16 = spec.training.precision != "fp32" and spec.model.compute_dtype == "bfloat16"
    active = device.type == "cuda" and bf16
    reason = None if active else ("no CUDA device" if device.type != "cuda" else "fp32 compute uses the PyTorch path")
    ops = []
    for item in kernel_registry():
        ops.append({"op": item["op"], "symbol": item["symbol"], "engine": item["engine"], "built": item["built"],
                    "selected": bool(active and item["built"]),
                    "fallback": None if (active and item["built"]) else "pytorch",
                    "fallback_reason": reason if not active else (None if item["built"] else "symbol not built")})
    selected = [op["op"] for op in ops if op["selected"]]
    unavailable = [op["op"] for op in ops if not op["built"]]
    fallback = [op["op"] for op in ops if not op["selected"] and op["built"]]
    return {"schema_version": 1, "arch": "sm_100a", "enabled": True, "strict": spec.kernels.strict,
            "compile": spec.kernels.compile, "library": str(native.lib_path()), "library_present": native.available(),
            "active": active, "device_kind": device.type, "active_count": len(selected),
            "fallback_count": len(fallback), "disabled_count": 0, "unavailable_count": len(unavailable), "ops": ops}


def require_kernel_plan_supported(plan: dict[str, Any], spec: RunSpec) -> None:
    """``[kernels] strict = true`` refuses to run when a selected-by-policy op would fall back."""

    if not spec.kernels.strict:
        return
    missing = [op["op"] for op in plan["ops"] if not op["selected"] and op["op"] not in OPTIONAL_OPS]
    if missing:
        raise ContractError(f"kernels.strict=true but these ops would not run natively: {missing}")


def kernel_registry_payload() -> dict[str, Any]:
    return {"schema_version": 1, "kernels": kernel_registry()}


def format_kernel_registry(rows: list[dict[str, Any]] | None = None) -> str:
    rows = kernel_registry() if rows is None else rows
    return "\n".join(f"{r['op']:<26} {r['symbol']:<32} {r['engine']:<28} built={r['built']}" for r in rows)


def kernel_plan_to_json(plan: dict[str, Any]) -> str:
    import json

    return json.dumps(plan, sort_keys=True, separators=(",", ":"))


def format_kernel_plan(plan: dict[str, Any]) -> str:
    lines = [f"kernel plan: active={plan['active']} library_present={plan['library_present']} "
             f"active_count={plan['active_count']} fallback={plan['fallback_count']} "
             f"unavailable={plan['unavailable_count']} device={plan['device_kind']}"]
    lines += [f"  {op['op']:<26} selected={op['selected']} fallback={op['fallback']}" for op in plan["ops"]]
    return "\n".join(lines)


def load_cache_manifest() -> dict[str, Any] | None:
    """The manifest the in-tree build wrote next to the libraries (sources, flags, digest), if there is one."""

    import json

    from research_b200.kernels import build

    try:
        return json.loads(build.MANIFEST.read_text())
    except (OSError, json.JSONDecodeError):
        return None


def enrich_kernel_plan_with_cache(plan: dict[str, Any]) -> dict[str, Any]:
    """The plan plus what the build cache says: whether the libraries on disk were built from the sources on disk."""

    from research_b200.kernels import build

    manifest = load_cache_manifest()
    current = build._digest(build.kernel_sources() + build.host_sources(),
                            build.ARCH_FLAGS + build.NVCC_FLAGS + build.CXX_FLAGS)
    out = dict(plan)
    out.update({"cache_dir": build.LIB_DIR.as_posix(), "cached_count": 0 if manifest is None else len(manifest["sources"]),
                "cache_digest": None if manifest is None else manifest.get("digest"), "source_digest": current,
                "stale_cache": manifest is not None and manifest.get("digest") != current,
                "missing_cache": manifest is None})
    return out


def compile_kernel_plan(spec: RunSpec, *, force: bool = False) -> dict[str, Any]:
    """Build the kernel and host libraries in the tree (a no-op when they are current) and report the plan."""

    from research_b200.kernels.build import build_all

    result = build_all(force=force)
    return {"schema_version": 1, "arch": "sm_100a", "library": str(result.kernel_lib), "rebuilt": result.rebuilt,
            "sources": list(result.sources), "digest": result.digest, "plan": kernel_plan(spec)}


def format_compile_result(payload: dict[str, Any]) -> str:
    return (f"built {payload['library']} (rebuilt={payload['rebuilt']}) from {len(payload['sources'])} sources "
            f"for {payload['arch']}, digest {payload['digest'][:16]}")
