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
