"""SMEBU: aux-loss-free expert load balancing by a momentum-smoothed bias on the router's selection scores.

Per MoE layer (reference: src/jaxtitan/steps/moe_balance.py:97-162): ``violation = (mean - count) / mean``;
``delta = load_lr * tanh(clamp * violation)``, mean-centred; ``momentum <- f * momentum + (1 - f) * delta``;
``expert_bias += momentum``.  Counts are the global per-expert assignment counts of the step.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from research_b200.config.specs import MoeBalanceSpec
from research_b200.errors import ContractError


@dataclass
class MoeBalanceLayer:
    path: str
    bias: torch.Tensor        # fp32 [E]: the parameter's data, or its fp32 master when the compute copy is narrower
    momentum: torch.Tensor    # [E] fp32
    entry: Any = None         # the parameter store's entry of the bias when ``bias`` is a master that has a copy


@dataclass
class MoeBalanceState:
    name: str
    load_lr: float
    momentum_factor: float
    clamp: float
    layers: list[MoeBalanceLayer]
    kernel: Any = None        # device pointer table of the native update, built on first use
    store: Any = None         # parameter store that holds compute-precision copies of the biases


def init_moe_balance(model, balance: MoeBalanceSpec | None, store=None) -> MoeBalanceState | None:
    """With a parameter store whose compute copies are narrower than fp32 the bias that is balanced is the fp32
    master of the store (the reference keeps ``expert_bias`` in fp32, models/components/moe.py:165-167): the router
    reads it through ``mlp.bias_master`` and the compute copy is refreshed after every update."""

    if balance is None or balance.name == "none":
        return None
    if balance.name != "smebu":
        raise ContractError(f"unsupported MoE balance policy {balance.name!r}")
    by_param = {} if store is None else {id(e.param): e for e in store.entries}
    layers = []
    for i, layer in enumerate(model.layers):
        if getattr(layer, "is_moe", False):
            param = layer.mlp.expert_bias
            bias, entry = param.data, by_param.get(id(param))
            if entry is not None:
                master = store.master_view(store.section_of(entry), entry)
                if master is not None and master.dtype == torch.float32 and param.data.dtype != torch.float32:
                    bias = master
                    layer.mlp.bias_master = master
                else:
                    entry = None
            layers.append(MoeBalanceLayer(f"layers.{i}.mlp.expert_bias", bias,
                                          torch.zeros_like(bias, dtype=torch.float32), entry))
    if not layers:
        return None
    return MoeBalanceState("smebu", float(balance.load_lr), float(balance.momentum), float(balance.clamp), layers,
                           store=store)


def _refresh_compute_copies(state: MoeBalanceState) -> None:
    for layer in state.layers:
        if layer.entry is not None:
            state.store.write_entry_shadow(layer.entry, layer.bias)


@torch.no_grad()
def apply_moe_balance_update(state: MoeBalanceState | None, router_counts: torch.Tensor | None) -> dict[str, Any]:
    """router_counts: [moe_layers, E] global assignment counts.  Updates biases in place; returns metrics."""

    if state is None or router_counts is None:
        return {}
    if router_counts.shape[0] != len(state.layers):
        raise ContractError(f"router count shape must match MoE balance state, got {tuple(router_counts.shape)}")
    from research_b200.ops import router as router_ops

    biases = [layer.bias for layer in state.layers]
    momenta = [layer.momentum for layer in state.layers]
    if router_ops.smebu_native_ok(router_counts, biases, momenta):
        # one launch for all layers (csrc/router.cu); the pointer table is rebuilt if a tensor moved
        if state.kernel is None or not state.kernel.matches(biases, momenta):
            state.kernel = router_ops.SmebuKernelState(biases, momenta)
        bias_sq, mom_sq = router_ops.smebu_update(state.kernel, router_counts, state.load_lr, state.clamp,
                                                  state.momentum_factor)
        _refresh_compute_copies(state)
        return {"smebu_bias_norm": bias_sq.sqrt(), "smebu_momentum_norm": mom_sq.sqrt()}
    bias_sq = torch.zeros((), device=router_counts.device)
    mom_sq = torch.zeros((), device=router_counts.device)
    for layer, counts in zip(state.layers, router_counts.float()):
        mean = counts.sum() / counts.shape[0]
        violation = (mean - counts) / mean.clamp_min(1e-6)
        delta = state.load_lr * torch.tanh(state.clamp * violation)
        delta = delta - delta.mean()
        layer.momentum.mul_(state.momentum_factor).add_(delta, alpha=1.0 - state.momentum_factor)
        layer.bias.add_(layer.momentum.to(layer.bias.dtype))
        bias_sq = bias_sq + layer.bias.float().pow(2).sum()
        mom_sq = mom_sq + layer.momentum.pow(2).sum()
    _refresh_compute_copies(state)
    return {"smebu_bias_norm": bias_sq.sqrt(), "smebu_momentum_norm": mom_sq.sqrt()}


def router_diagnostics(counts: torch.Tensor, importance: torch.Tensor) -> dict[str, Any]:
    """Run-level router health from ``[layers, E]`` counts / importance (reference: steps/train.py:605-646)."""

    def entropy(rows):
        p = rows / rows.sum(dim=-1, keepdim=True).clamp_min(1e-6)
        return -(torch.where(p > 0, p * torch.log(torch.where(p > 0, p, torch.ones_like(p))), torch.zeros_like(p))).sum(-1)

    def cv(rows):
        mean = rows.mean(dim=-1)
        return rows.std(dim=-1, unbiased=False) / mean.clamp_min(1e-6)

    counts, importance = counts.float(), importance.float()
    means = counts.sum(-1) / counts.shape[-1]
    load_entropy, load_cv = entropy(counts), cv(counts)
    return {
        "router_max_vio": ((counts.max(-1).values - means) / means.clamp_min(1e-6)).max(),
        "router_load_min": counts.min(),
        "router_load_max": counts.max(),
        "router_load_entropy": load_entropy.mean(),
        "router_mean_load_cv": load_cv.mean(),
        "router_std_load_cv": load_cv.std(unbiased=False),
        "router_mean_load_entropy": load_entropy.mean(),
        "router_min_load_entropy": load_entropy.min(),
        "router_dead_experts_count": (counts <= 0).sum().float(),
        "router_experts_active_mean": (counts > 0).sum(-1).float().mean(),
        "router_mean_importance_cv": cv(importance).mean(),
        "router_mean_importance_entropy": entropy(importance).mean(),
    }
