"""Router math after the router GEMM as native kernels (``csrc/router.cu``), with PyTorch restatements.

``route``: logits ``[T, E]`` -> (expert ids ``[T, k]``, weights ``[T, k]``, scores ``[T, E]``), differentiable in
the logits through ``weights`` and ``scores``.  ``load_statistics``: per-expert counts, importance and the load
summary in one launch.  ``smebu_update``: the bias update of every MoE layer in one launch.

Reference: src/jaxtitan/models/components/moe.py:98-147 (router), 794-840 (statistics);
src/jaxtitan/steps/moe_balance.py:97-162 (SMEBU).
"""

from __future__ import annotations

import ctypes as _ct

import torch

from research_b200.ops import native

MAX_EXPERTS = 1024
MAX_TOP_K = 32


def _lib():
    lib = native.load()
    if not getattr(lib, "_router_declared", False):
        vp, ci, ll, cf = _ct.c_void_p, _ct.c_int, _ct.c_longlong, _ct.c_float
        lib.b200_router_fwd.argtypes = [vp, ci, ll, vp, ci, ci, ci, ci, cf, vp, vp, vp, vp]
        lib.b200_router_bwd.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, cf, vp, ci, ll, vp]
        lib.b200_router_stats_floats.argtypes = [ci]
        lib.b200_router_stats.argtypes = [vp, vp, ci, ci, vp, vp]
        lib.b200_smebu_update.argtypes = [vp, vp, ci, ci, cf, cf, cf, vp, vp]
        for fn in (lib.b200_router_fwd, lib.b200_router_bwd, lib.b200_router_stats_floats, lib.b200_router_stats,
                   lib.b200_smebu_update):
            fn.restype = ci
        lib._router_declared = True
    return lib


def _native_enabled() -> bool:
    from research_b200.ops import functional as Fn

    return Fn.native_enabled()


def native_route_ok(logits: torch.Tensor, num_experts: int, top_k: int) -> bool:
    return (logits.is_cuda and native.available() and _native_enabled() and logits.dtype in (torch.bfloat16, torch.float32)
            and num_experts <= MAX_EXPERTS and top_k <= MAX_TOP_K)


def route_reference(logits: torch.Tensor, bias: torch.Tensor, top_k: int, kind: str, route_scale: float):
    """The same math in PyTorch ops (CPU path and test oracle)."""

    logits = logits.float()
    scores = torch.softmax(logits, dim=-1) if kind == "softmax" else torch.sigmoid(logits)
    _, expert_ids = torch.topk(scores + bias.detach().float(), top_k, dim=-1)
    top = scores.gather(-1, expert_ids)
    if kind == "softmax":
        weights = top * route_scale
    else:
        weights = top / (top.sum(dim=-1, keepdim=True) + 1e-20) * route_scale
    return expert_ids, weights, scores


class _RouteFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, bias, top_k, softmax, route_scale):
        lib = _lib()
        shape = logits.shape
        E = shape[-1]
        flat = logits.reshape(-1, E)
        if flat.stride(-1) != 1:
            flat = flat.contiguous()
        T = flat.shape[0]
        dev = logits.device
        ids = torch.empty(T, top_k, dtype=torch.int32, device=dev)
        weights = torch.empty(T, top_k, dtype=torch.float32, device=dev)
        scores = torch.empty(T, E, dtype=torch.float32, device=dev)
        bias32 = bias.detach().float().contiguous()
        rc = lib.b200_router_fwd(flat.data_ptr(), int(flat.dtype == torch.bfloat16), flat.stride(0), bias32.data_ptr(),
                                 T, E, top_k, int(softmax), float(route_scale), ids.data_ptr(), weights.data_ptr(),
                                 scores.data_ptr(), native._stream())
        native._check(rc, "b200_router_fwd")
        ctx.save_for_backward(scores, ids)
        ctx.meta = (shape, logits.dtype, top_k, softmax, route_scale)
        ids64 = ids.long().view(*shape[:-1], top_k)
        ctx.mark_non_differentiable(ids64)
        return ids64, weights.view(*shape[:-1], top_k), scores.view(shape)

    @staticmethod
    def backward(ctx, _dids, dweights, dscores):
        scores, ids = ctx.saved_tensors
        shape, dtype, top_k, softmax, route_scale = ctx.meta
        T, E = scores.shape
        if dweights is None and dscores is None:
            return None, None, None, None, None
        dw = None if dweights is None else dweights.reshape(T, top_k).float().contiguous()
        ds = None if dscores is None else dscores.reshape(T, E).float().contiguous()
        dlogits = torch.empty(T, E, dtype=dtype, device=scores.device)
        rc = _lib().b200_router_bwd(scores.data_ptr(), ids.data_ptr(), None if dw is None else dw.data_ptr(),
                                    None if ds is None else ds.data_ptr(), T, E, top_k, int(softmax),
                                    float(route_scale), dlogits.data_ptr(), int(dtype == torch.bfloat16), E,
                                    native._stream())
        native._check(rc, "b200_router_bwd")
        return dlogits.view(shape), None, None, None, None


def route(logits: torch.Tensor, bias: torch.Tensor, top_k: int, kind: str, route_scale: float):
    """logits ``[..., E]`` -> (ids ``[..., k]`` int64, weights ``[..., k]`` fp32, scores ``[..., E]`` fp32)."""

    if native_route_ok(logits, logits.shape[-1], top_k):
        return _RouteFn.apply(logits, bias, int(top_k), kind == "softmax", float(route_scale))
    return route_reference(logits, bias, top_k, kind, route_scale)


def load_statistics_reference(expert_ids: torch.Tensor, weights: torch.Tensor, num_experts: int):
    ids = expert_ids.reshape(-1).long()
    dev = ids.device
    counts = torch.zeros(num_experts, dtype=torch.float32, device=dev).index_add_(
        0, ids, torch.ones_like(ids, dtype=torch.float32))
    importance = torch.zeros(num_experts, dtype=torch.float32, device=dev).index_add_(
        0, ids, weights.reshape(-1).float())
    total = counts.sum()
    mean = total / num_experts
    load_max, load_min = counts.max(), counts.min()
    max_vio = (load_max - mean) / mean.clamp_min(1e-6)
    prob = counts / total.clamp_min(1e-6)
    entropy = -(torch.where(prob > 0, prob * torch.log(torch.where(prob > 0, prob, torch.ones_like(prob))),
                            torch.zeros_like(prob))).sum()
    return counts, importance, total, mean, load_min, load_max, max_vio, entropy


@torch.no_grad()
def load_statistics(expert_ids: torch.Tensor, weights: torch.Tensor, num_experts: int):
    """(counts [E], importance [E], total, mean, min, max, max violation, entropy), all fp32 device tensors."""

    if not (expert_ids.is_cuda and native.available() and _native_enabled() and num_experts <= MAX_EXPERTS
            and expert_ids.numel() > 0 and not native.deterministic()):   # importance: fp32 atomics
        return load_statistics_reference(expert_ids, weights, num_experts)
    lib = _lib()
    ids = expert_ids.reshape(-1).to(torch.int32).contiguous()
    w = weights.detach().reshape(-1).float().contiguous()
    E = num_experts
    out = torch.zeros(lib.b200_router_stats_floats(E), dtype=torch.float32, device=ids.device)
    native._check(lib.b200_router_stats(ids.data_ptr(), w.data_ptr(), ids.numel(), E, out.data_ptr(),
                                        native._stream()), "b200_router_stats")
    s = out[2 * E:2 * E + 6]
    return out[:E], out[E:2 * E], s[0], s[1], s[2], s[3], s[4], s[5]


class SmebuKernelState:
    """Device table of the (bias, momentum) pointers of every MoE layer, built once."""

    def __init__(self, biases, momenta):
        self.biases, self.momenta = list(biases), list(momenta)
        table = []
        for b, m in zip(self.biases, self.momenta):
            table += [b.data_ptr(), m.data_ptr()]
        dev = self.biases[0].device
        self.ptrs = torch.tensor(table, dtype=torch.int64, device=dev)
        self.signature = tuple(table)
        self.sq = torch.empty(len(self.biases), 2, dtype=torch.float32, device=dev)

    def matches(self, biases, momenta) -> bool:
        table = []
        for b, m in zip(biases, momenta):
            table += [b.data_ptr(), m.data_ptr()]
        return tuple(table) == self.signature


def smebu_native_ok(counts: torch.Tensor, biases, momenta) -> bool:
    return (counts.is_cuda and native.available() and _native_enabled()
            and all(t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() for t in (*biases, *momenta)))


@torch.no_grad()
def smebu_update(state: SmebuKernelState, counts: torch.Tensor, load_lr: float, clamp: float, factor: float):
    """counts ``[layers, E]``; updates every layer's momentum and bias in place; returns (bias_sq, momentum_sq)."""

    c = counts.float().contiguous()
    L, E = c.shape
    native._check(_lib().b200_smebu_update(c.data_ptr(), state.ptrs.data_ptr(), L, E, float(load_lr), float(clamp),
                                           float(factor), state.sq.data_ptr(), native._stream()), "b200_smebu_update")
    sums = state.sq.sum(dim=0)
    return sums[0], sums[1]
