"""Sparse mixture-of-experts feed-forward layer.

Router, expert math, statistics and the sequence balance loss restate the reference
(src/jaxtitan/models/components/moe.py:98-147 router, 150-195 experts, 367-479 layer, 794-840 statistics):
``scores = sigmoid(x W_r)``; experts are picked by ``top_k(scores + expert_bias)`` but weighted by the
unbiased scores, normalised over the selected experts and multiplied by ``route_scale``; ``expert_bias`` gets
no gradient.  Added here (optional, off by default): a softmax router, capacity-factor token dropping and a
Switch-style load-balance loss.

Dispatch is expert-major: assignments are sorted by expert, every expert's rows are padded to a multiple
of 128 so that one grouped tcgen05 GEMM (B operand picked per row tile) covers all local experts; with
expert parallelism the sorted rows travel through an all-to-all first (:mod:`research_b200.parallel.expert`).
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from research_b200.config.specs import ModelSpec, TrinityMoeSpec
from research_b200.errors import ContractError
from research_b200.models.output import AuxLoss, RouterStats
from research_b200.ops import functional as Fn


def router_stats(name: str, layer_index: int, expert_ids: torch.Tensor, weights: torch.Tensor, num_experts: int,
                 dropped: torch.Tensor | None = None) -> RouterStats:
    from research_b200.ops.router import load_statistics

    counts, importance, total, mean, load_min, load_max, max_vio, entropy = load_statistics(
        expert_ids, weights, num_experts)
    return RouterStats(name=name, layer_index=layer_index, expert_counts=counts, importance=importance,
                       total_assignments=total, load_min=load_min, load_max=load_max, load_mean=mean,
                       max_vio=max_vio, load_entropy=entropy, dropped=dropped)


def _sum_over_sequence_shards(x: torch.Tensor, replicated_groups, summed_groups) -> tuple[torch.Tensor, int]:
    """Add ``x`` up over the groups that split the sequence; returns the sum and the number of shards.

    ``replicated_groups``: their ranks run one objective in copies (tensor-parallel ranks with a sequence-parallel
    residual stream): a rank's share of the gradient is the one through its own tokens.  ``summed_groups``: their
    ranks' objectives are added up (context-parallel ranks), so the gradient comes back from every rank's copy.
    """

    from research_b200.models.execution import all_reduce_sum, all_reduce_sum_summed_objectives

    shards = 1
    for group in replicated_groups:
        x = all_reduce_sum(x, group)
        shards *= torch.distributed.get_world_size(group)
    for group in summed_groups:
        x = all_reduce_sum_summed_objectives(x, group)
        shards *= torch.distributed.get_world_size(group)
    return x, shards


def sequence_balance_loss(expert_ids: torch.Tensor, scores: torch.Tensor, top_k: int, replicated_groups=(),
                          summed_groups=()) -> torch.Tensor:
    """``sum_e f_e p_e`` per sequence, averaged over the batch; scores: [B,S,E], expert_ids: [B,S,k].

    The two group lists name the process groups that split the sequence dimension (see
    :func:`_sum_over_sequence_shards`): the per-sequence sums are added up over them so that a sharded sequence gives
    the loss, and the gradient, of the whole one.
    """

    if scores.dim() != 3:
        raise ContractError(f"router scores must have shape [batch, seq, experts], got {tuple(scores.shape)}")
    B, S, E = scores.shape
    flat_ids = expert_ids.reshape(B, -1).long()                          # [B, S*k]
    sel_sum = torch.zeros(B, E, dtype=torch.float32, device=scores.device).scatter_add_(
        1, flat_ids, torch.ones_like(flat_ids, dtype=torch.float32))     # [B,E] picks per sequence and expert
    normalised = scores / scores.sum(dim=-1, keepdim=True).clamp_min(1e-20)
    both, shards = _sum_over_sequence_shards(torch.stack([sel_sum, normalised.sum(dim=1)]), replicated_groups,
                                             summed_groups)
    total_S = S * shards
    f = (E / (top_k * total_S)) * both[0].detach()
    p = both[1] / total_S
    return (f * p).sum() / B


def switch_balance_loss(expert_ids: torch.Tensor, probs: torch.Tensor, top_k: int, replicated_groups=(),
                        summed_groups=()) -> torch.Tensor:
    """Switch-transformer style ``E * sum_e (fraction routed to e) * (mean router probability of e)`` over the
    tokens of this rank's batch rows, whole sequences even where the sequence is split over ranks."""

    E = probs.shape[-1]
    flat_ids = expert_ids.reshape(-1).long()
    picks = torch.zeros(E, dtype=torch.float32, device=probs.device).index_add_(
        0, flat_ids, torch.ones_like(flat_ids, dtype=torch.float32))
    flat_probs = probs.reshape(-1, E).float()
    both, shards = _sum_over_sequence_shards(torch.stack([picks, flat_probs.sum(dim=0)]), replicated_groups,
                                             summed_groups)
    f = both[0].detach() / max(flat_ids.numel() * shards, 1)
    p = both[1] / max(flat_probs.shape[0] * shards, 1)
    return E * (f * p).sum()


class Router(nn.Module):
    def __init__(self, hidden: int, num_experts: int, top_k: int, route_scale: float, kind: str):
        super().__init__()
        if top_k <= 0 or num_experts <= 0 or top_k > num_experts:
            raise ContractError("router top_k must be positive and <= num_experts")
        self.proj = nn.Parameter(torch.empty(num_experts, hidden, dtype=torch.float32))
        self.num_experts, self.top_k, self.route_scale, self.kind = num_experts, top_k, float(route_scale), kind

    def forward(self, x: torch.Tensor, expert_bias: torch.Tensor):
        """x: [..., H] -> (expert_ids [...,k] int64, weights [...,k] fp32, scores [...,E] fp32)."""

        from research_b200.ops.router import route

        # the native GEMM needs 16-byte output rows: eight or more experts
        native_ok = Fn.use_native(x) and self.proj.shape[0] % 8 == 0
        logits = Fn.linear(x, self.proj) if native_ok else F.linear(x.float(), self.proj.float())
        expert_ids, weights, scores = route(logits, expert_bias, self.top_k, self.kind, self.route_scale)
        return expert_ids, weights, scores


class Experts(nn.Module):
    """``E_local`` SwiGLU experts with fused gate|up storage ``[E, 2I, H]`` and down ``[E, H, I]``."""

    def __init__(self, hidden: int, inter: int, num_local: int):
        super().__init__()
        self.hidden, self.inter, self.num_local = hidden, inter, num_local
        self.w_gate_up = nn.Parameter(torch.empty(num_local, 2 * inter, hidden, dtype=torch.float32))
        self.w_down = nn.Parameter(torch.empty(num_local, hidden, inter, dtype=torch.float32))

    def forward(self, rows: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
        """rows: [R, H] sorted by local expert; counts: [E_local] rows per expert (host or device ints)."""

        from research_b200.ops.grouped import grouped_expert_ffn

        return grouped_expert_ffn(rows, counts, self.w_gate_up, self.w_down)


class SharedSwiGLU(nn.Module):
    def __init__(self, hidden: int, inter: int, ex):
        super().__init__()
        tp = ex.tp_size
        self.w_gate_up = nn.Parameter(torch.empty(2 * (inter // tp), hidden, dtype=torch.float32))
        self.w_down = nn.Parameter(torch.empty(hidden, inter // tp, dtype=torch.float32))

    def forward(self, x: torch.Tensor, ex) -> torch.Tensor:
        h = Fn.swiglu(Fn.linear(x, self.w_gate_up))
        return Fn.linear(h, self.w_down)


class SparseMoE(nn.Module):
    def __init__(self, spec: ModelSpec, moe: TrinityMoeSpec, ex):
        super().__init__()
        if moe.expert_intermediate_size is None:
            raise ContractError("model.trinity.moe.expert_intermediate_size must be resolved before model construction")
        self.moe = moe
        self.hidden = spec.hidden_size
        self.num_experts = moe.num_experts
        ep = ex.ep_size
        if self.num_experts % ep != 0:
            raise ContractError(f"num_experts ({self.num_experts}) must be divisible by the expert axis size ({ep})")
        self.num_local = self.num_experts // ep
        shards = ex.efsdp_size
        if moe.expert_intermediate_size % shards != 0:
            raise ContractError(f"expert_intermediate_size ({moe.expert_intermediate_size}) must be divisible by the "
                                f"expert_fsdp axis size ({shards})")
        self.router = Router(spec.hidden_size, moe.num_experts, moe.top_k, moe.route_scale, moe.router)
        self.expert_bias = nn.Parameter(torch.zeros(moe.num_experts, dtype=torch.float32), requires_grad=False)
        # fp32 master of the bias when the parameter itself is held in a narrower compute precision (set by the
        # balance policy): selection then sees the exact bias
        self.bias_master: torch.Tensor | None = None
        self.experts = Experts(spec.hidden_size, moe.expert_intermediate_size // shards, self.num_local)
        self.shared_experts = None
        if moe.num_shared_experts > 0:
            self.shared_experts = SharedSwiGLU(spec.hidden_size, moe.expert_intermediate_size * moe.num_shared_experts, ex)

    @staticmethod
    def _layer_slot(ex, layer_index: int) -> int:
        """Index of this MoE layer among the MoE layers seen so far (stable over steps): selects the layer's own
        forward inbox in the expert-parallel workspace."""

        slots = ex.extras.setdefault("moe_layer_slots", {})
        if layer_index not in slots:
            slots[layer_index] = len(slots)
        return slots[layer_index]

    def _dedicated_axis_fused(self, x: torch.Tensor, expert_ids: torch.Tensor, weights: torch.Tensor, ex,
                              layer_index: int = 0):
        """Dedicated ``ep`` axis on CUDA: tokens are replicated over the axis, so every rank routes its slice of
        them through the peer-memory dispatch / combine kernels and the results are gathered back (the reference
        slices the sequence inside its shard_map, components/moe.py:538-696).  The capacity applies per sender
        slice.  Returns (y ``[T, H]``, masked weights ``[B, S, k]``, dropped count) or None when peer memory is
        not available."""

        from research_b200.models.execution import all_gather_replicated, slice_dim
        from research_b200.parallel import expert_fused

        B, S, H = x.shape
        k = expert_ids.shape[-1]
        ep, rank, group = ex.ep_size, ex.ep_rank, ex.ep_group
        T = B * S
        t_local = T // ep
        capacity = capacity_rows(self.moe.capacity_factor, t_local, k, self.num_experts)
        ids_local = expert_ids.reshape(T, k)[rank * t_local:(rank + 1) * t_local].contiguous()
        plan = expert_fused.ExpertParallelPlan(ids_local, self.num_experts, capacity, ex, H,
                                               layer_slot=self._layer_slot(ex, layer_index))
        if plan.ws is None:
            return None
        keep = plan.kept_mask
        w_local = slice_dim(weights.reshape(T, k), group, 0) * keep.to(weights.dtype)
        x_local = slice_dim(x.reshape(T, H), group, 0)
        y_local = expert_fused.dispatch_and_combine_fused(self.experts, x_local, w_local, plan)
        y = all_gather_replicated(y_local, group, 0)
        w_all = all_gather_replicated(w_local.detach(), group, 0).view(B, S, k)      # for the load statistics
        dropped = (~keep).sum()
        torch.distributed.all_reduce(dropped, group=group)
        return y, w_all, dropped

    def forward(self, x: torch.Tensor, ex, *, name: str, layer_index: int):
        """x: this rank's ``[B, S_local, H]`` shard of the residual stream -> (y, aux_losses, router_stats).

        Routed experts work on the local tokens (under sequence parallelism every tensor-parallel rank routes
        its own slice); the shared expert is an ordinary tensor-parallel SwiGLU on the gathered sequence.
        """

        from research_b200.models.execution import all_reduce_sum
        from research_b200.parallel.expert import dispatch_and_combine

        B, S, H = x.shape
        expert_ids, weights, scores = self.router(x, self.expert_bias if self.bias_master is None else self.bias_master)
        dropped = None
        plan = None
        y_routed = None          # set when a path below has already run dispatch, experts and combine
        if Fn.use_native(x) and x.dtype == torch.bfloat16 and H % 8 == 0:
            # device-side routing plan: ranks in token order, capacity, padded expert-major layout (no sort)
            from research_b200.ops.grouped import RoutingPlan

            capacity = None
            if self.moe.capacity_factor is not None:
                capacity = capacity_rows(self.moe.capacity_factor, B * S, expert_ids.shape[-1], self.num_experts)
            if ex.ep_size == 1:
                plan = RoutingPlan(expert_ids.reshape(B * S, -1), self.num_experts, capacity)
            else:
                from research_b200.parallel import expert_fused

                if ex.ep_axis_sharing == "dedicated_ep":
                    if expert_fused.fused_available(ex, x, capacity) and (B * S) % ex.ep_size == 0 \
                            and ex.efsdp_size == 1:
                        done = self._dedicated_axis_fused(x, expert_ids, weights, ex, layer_index)
                        if done is not None:
                            y_routed, weights, dropped = done
                elif expert_fused.fused_available(ex, x, capacity):
                    plan = expert_fused.ExpertParallelPlan(expert_ids.reshape(B * S, -1), self.num_experts, capacity, ex,
                                                           H, layer_slot=self._layer_slot(ex, layer_index))
                    if plan.ws is None:
                        plan = None
            if y_routed is not None:
                pass
            elif plan is None and capacity is not None:
                weights, dropped = apply_capacity(expert_ids, weights, self.num_experts, self.moe.capacity_factor)
            elif capacity is not None:
                keep = plan.kept_mask.view(expert_ids.shape)
                weights = weights * keep.to(weights.dtype)
                dropped = (~keep).sum()
        elif self.moe.capacity_factor is not None:
            weights, dropped = apply_capacity(expert_ids, weights, self.num_experts, self.moe.capacity_factor)
        if y_routed is not None:
            y = y_routed
        else:
            x_routed, w_routed = x.reshape(B * S, H), weights.reshape(B * S, -1)
            if ex.efsdp_size > 1:
                # expert FSDP: every rank of the axis sees the same tokens and holds a slice of each expert's
                # intermediate dimension; partial outputs are summed over the axis (reference: moe.py:642-643), and
                # the gradients of the replicated inputs are summed on the way back
                from research_b200.models.execution import copy_to_group

                x_routed = copy_to_group(x_routed, ex.expert_fsdp_group)
                w_routed = copy_to_group(w_routed, ex.expert_fsdp_group)
            y = dispatch_and_combine(self.experts, x_routed, expert_ids.reshape(B * S, -1), w_routed,
                                     num_experts=self.num_experts, ex=ex, plan=plan)
            if ex.efsdp_size > 1:
                y = all_reduce_sum(y, ex.expert_fsdp_group)
        y = y.view(B, S, H)
        if self.shared_experts is not None:
            y = y + ex.reduce_scatter_sequence(self.shared_experts(ex.gather_sequence(x), ex))
        stats = router_stats(name, layer_index, expert_ids, weights, self.num_experts, dropped)
        aux = []
        bal = self.moe.balance
        # the sequence is split over tensor-parallel ranks (sequence-parallel stream) and context-parallel ranks
        replicated = [ex.tp_group] if ex.sp and ex.tp_group is not None else []
        summed = [ex.cp_group] if ex.cp_group is not None else []
        if bal.name == "smebu" and bal.sequence_aux_loss_weight > 0.0:
            aux.append(AuxLoss("moe_sequence_balance",
                               sequence_balance_loss(expert_ids, scores, self.moe.top_k, replicated, summed),
                               float(bal.sequence_aux_loss_weight)))
        if self.moe.aux_loss_coef > 0.0:
            aux.append(AuxLoss("moe_load_balance", switch_balance_loss(expert_ids, scores, self.moe.top_k, replicated, summed),
                               float(self.moe.aux_loss_coef)))
        return y, tuple(aux), (stats,)


def capacity_rows(capacity_factor: float, tokens: int, k: int, num_experts: int) -> int:
    """Rows an expert accepts: ceil(capacity_factor * tokens * k / E)."""

    return int(-(-capacity_factor * tokens * k // num_experts))


def apply_capacity(expert_ids: torch.Tensor, weights: torch.Tensor, num_experts: int, capacity_factor: float):
    """Zero the weights of assignments beyond each expert's capacity (token order priority).

    Capacity = ceil(capacity_factor * tokens * k / E).  Returns (weights, number of dropped assignments).
    """

    shape = expert_ids.shape
    k = shape[-1]
    flat = expert_ids.reshape(-1).long()
    tokens = flat.numel() // k
    capacity = capacity_rows(capacity_factor, tokens, k, num_experts)
    onehot = F.one_hot(flat, num_experts)
    position = (onehot.cumsum(dim=0) * onehot).sum(dim=-1) - 1     # rank of each assignment inside its expert
    keep = position < capacity
    w = weights.reshape(-1) * keep.to(weights.dtype)
    return w.view(shape), (~keep).sum()
