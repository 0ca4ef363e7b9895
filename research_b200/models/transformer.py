"""Decoder-only language models: the baseline decoder and the Trinity recipe.

Semantics follow the reference components: pre-norm blocks ``x += attn(norm(x)); x += ffn(norm(x))``
(models/components/blocks.py:22-85), GQA attention with QK-RMSNorm before interleaved RoPE
(components/attention.py:42-266), SwiGLU ``down(silu(gate(x)) * up(x))`` (components/ffn.py:13-51); Trinity adds
local sliding-window+RoPE / global NoPE layers, sandwich norms with depth-scaled post-norm init, sqrt(hidden)
embedding scale, a sigmoid attention output gate and sparse MoE layers (models/trinity.py:22-215,
components/blocks.py:88-282).

Storage differs from the reference on purpose: projection weights are ``[out, in]`` (K-major for the forward
tcgen05 GEMM) and q|k|v as well as gate|up live in one fused parameter so that each block issues one GEMM per
fused group; :mod:`research_b200.models.build` exposes the reference's logical parameter paths
(``layers.0.attn.q.kernel`` as ``[in, out]``...) as views of that storage for optimizers and checkpoints.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from research_b200.config.specs import ModelSpec, TrinityMoeSpec
from research_b200.errors import ContractError
from research_b200.models.execution import ExecutionContext
from research_b200.models.moe import SparseMoE
from research_b200.models.output import AuxLoss, ModelOutput, RouterStats
from research_b200.ops import functional as Fn


@dataclass(frozen=True)
class AttentionConfig:
    position: str = "rope"          # "rope" | "none"
    mask: str = "causal"            # "causal" | "sliding_window"
    local_window: int | None = None
    qk_norm: bool = True
    gate: bool = False


@dataclass
class ForwardInputs:
    """Per-batch tensors shared by every layer."""

    positions: torch.Tensor              # int32 [B*S]: global sequence position of every local row
    B: int
    S: int
    chunks: tuple[tuple[int, int], ...] = ()   # context parallelism: (first global position, length) of local chunks
    lo_causal: torch.Tensor | None = None    # int32 [B,S]: document starts (or None)
    hi_causal: torch.Tensor | None = None
    lo_window: dict[int, tuple[torch.Tensor, torch.Tensor | None]] | None = None  # per window size

    def bounds(self, window: int | None):
        if window is None:
            return self.lo_causal, self.hi_causal
        if self.lo_window is None:
            self.lo_window = {}
        if window not in self.lo_window:
            idx = self.positions.view(self.B, self.S)
            lo = (idx - (window - 1)).clamp_min(0)
            if self.lo_causal is not None:
                lo = torch.maximum(lo, self.lo_causal)
            self.lo_window[window] = (lo.contiguous(), None)
        return self.lo_window[window]


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, init_value: float = 1.0):
        super().__init__()
        self.scale = nn.Parameter(torch.full((dim,), float(init_value), dtype=torch.float32))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return Fn.rmsnorm(x, self.scale, self.eps)

    def add_forward(self, x: torch.Tensor, delta: torch.Tensor | None):
        if delta is None:
            return Fn.rmsnorm(x, self.scale, self.eps), x
        return Fn.add_rmsnorm(x, delta, self.scale, self.eps)


class Attention(nn.Module):
    """GQA attention with fused q|k|v projection.  Under tensor parallelism the heads are split across ranks."""

    def __init__(self, spec: ModelSpec, cfg: AttentionConfig, ex: ExecutionContext):
        super().__init__()
        tp = ex.tp_size
        self.cfg = cfg
        self.hidden = spec.hidden_size
        self.head_dim = spec.head_dim
        self.hq_total, self.hkv_total = spec.num_heads, spec.n_kv_heads
        self.hq, self.hkv = spec.num_heads // tp, spec.n_kv_heads // tp
        self.theta = spec.rope_theta
        self.eps = spec.norm_epsilon
        D = self.head_dim
        self.wqkv = nn.Parameter(torch.empty((self.hq + 2 * self.hkv) * D, self.hidden, dtype=torch.float32))
        self.wo = nn.Parameter(torch.empty(self.hidden, self.hq * D, dtype=torch.float32))
        if cfg.qk_norm:
            self.q_norm = nn.Parameter(torch.ones(D, dtype=torch.float32))
            self.k_norm = nn.Parameter(torch.ones(D, dtype=torch.float32))
        else:
            self.q_norm = self.k_norm = None
        self.wgate = nn.Parameter(torch.empty(self.hq * D, self.hidden, dtype=torch.float32)) if cfg.gate else None

    def forward(self, x: torch.Tensor, inp: ForwardInputs, ex: ExecutionContext) -> torch.Tensor:
        if self.wgate is None and ex.sp:
            # SP: [B, S/tp, H] -> [B, S, 3 groups of local heads]; the row gather runs inside the GEMM kernel
            qkv3 = ex.column_linear(x, self.wqkv)
            B, S = qkv3.shape[0], qkv3.shape[1]
            qkv, x2 = qkv3.reshape(B * S, -1), None
        else:
            x = ex.gather_sequence(x)                   # SP: [B, S/tp, H] -> [B, S, H]
            B, S = x.shape[0], x.shape[1]
            x2 = x.reshape(B * S, self.hidden)
            qkv = Fn.linear(x2, self.wqkv)
        window = self.cfg.local_window if self.cfg.mask == "sliding_window" else None
        lo, hi = inp.bounds(window)
        o = ex.attention(qkv, self.q_norm, self.k_norm, inp.positions, B=B, S=S, hq=self.hq, hkv=self.hkv,
                         D=self.head_dim, eps=self.eps, theta=self.theta, rope=self.cfg.position == "rope",
                         lo=lo, hi=hi, chunks=inp.chunks)
        if self.wgate is not None:
            o = Fn.sigmoid_gate(o.reshape(B * S, -1), Fn.linear(x2, self.wgate)).view(B, S, -1)
        return ex.row_linear(o if o.dim() == 3 else o.view(B, S, -1), self.wo)  # partial sums -> SP shard

    # ---- inference -------------------------------------------------------------------------------
    def project_qkv(self, x: torch.Tensor, positions: torch.Tensor):
        """x: [B,T,H]; positions int32 [B,T] -> q [B,T,hq,D], k, v [B,T,hkv,D] (normalised / rotated)."""

        B, T = x.shape[0], x.shape[1]
        D = self.head_dim
        x2 = x.reshape(B * T, self.hidden)
        qkv = Fn.linear(x2, self.wqkv)
        qk = Fn.qk_norm_rope(qkv, self.q_norm, self.k_norm, positions.reshape(-1).to(torch.int32), self.hq, self.hkv,
                             D, self.eps, self.theta, self.cfg.position == "rope")
        q = qk[:, : self.hq * D].reshape(B, T, self.hq, D)
        k = qk[:, self.hq * D:].reshape(B, T, self.hkv, D)
        v = qkv[:, (self.hq + self.hkv) * D:].reshape(B, T, self.hkv, D)
        return q, k, v, x2

    def finish(self, o: torch.Tensor, x2: torch.Tensor, ex: ExecutionContext | None = None) -> torch.Tensor:
        B, T = o.shape[0], o.shape[1]
        if self.wgate is not None:
            o = Fn.sigmoid_gate(o.reshape(B * T, -1), Fn.linear(x2, self.wgate)).view(B, T, -1)
        y = Fn.linear(o.reshape(B, T, -1), self.wo)
        if ex is not None and ex.tp_size > 1:
            # the output projection is row-parallel: every rank holds the product over its own heads
            from research_b200.models.execution import all_reduce_sum

            y = all_reduce_sum(y, ex.tp_group)
        return y


class SwiGLU(nn.Module):
    def __init__(self, hidden: int, intermediate: int, ex: ExecutionContext):
        super().__init__()
        tp = ex.tp_size
        self.inter = intermediate // tp
        self.w_gate_up = nn.Parameter(torch.empty(2 * self.inter, hidden, dtype=torch.float32))
        self.w_down = nn.Parameter(torch.empty(hidden, self.inter, dtype=torch.float32))

    def forward(self, x: torch.Tensor, ex: ExecutionContext) -> torch.Tensor:
        h = Fn.swiglu(ex.column_linear(x, self.w_gate_up))
        return ex.row_linear(h, self.w_down)


class DecoderBlock(nn.Module):
    """``x += attn(pre_norm(x)); x += mlp(post_norm(x))`` with the residual adds fused into the norms."""

    def __init__(self, spec: ModelSpec, ex: ExecutionContext):
        super().__init__()
        self.pre_norm = RMSNorm(spec.hidden_size, spec.norm_epsilon)
        self.attn = Attention(spec, AttentionConfig(qk_norm=spec.qk_norm), ex)
        self.post_norm = RMSNorm(spec.hidden_size, spec.norm_epsilon)
        self.mlp = SwiGLU(spec.hidden_size, spec.intermediate_size, ex)

    def forward(self, x, delta, inp: ForwardInputs, ex: ExecutionContext):
        h, x = self.pre_norm.add_forward(x, delta)
        a = self.attn(h, inp, ex)
        h, x = self.post_norm.add_forward(x, a)
        return x, self.mlp(h, ex), (), ()


class TrinityBlock(nn.Module):
    """Sandwich-norm block: ``x += attn_post_norm(attn(attn_pre_norm(x))); x += ffn_post_norm(ffn(ffn_pre_norm(x)))``."""

    def __init__(self, spec: ModelSpec, cfg: AttentionConfig, moe: TrinityMoeSpec | None, post_scale: float,
                 ex: ExecutionContext, layer_index: int):
        super().__init__()
        H, eps = spec.hidden_size, spec.norm_epsilon
        self.layer_index = layer_index
        self.attn_pre_norm = RMSNorm(H, eps)
        self.attn = Attention(spec, cfg, ex)
        self.attn_post_norm = RMSNorm(H, eps, post_scale)
        self.ffn_pre_norm = RMSNorm(H, eps)
        self.mlp = SparseMoE(spec, moe, ex) if moe is not None else SwiGLU(H, spec.intermediate_size, ex)
        self.ffn_post_norm = RMSNorm(H, eps, post_scale)
        self.is_moe = moe is not None

    def forward(self, x, delta, inp: ForwardInputs, ex: ExecutionContext):
        h, x = self.attn_pre_norm.add_forward(x, delta)
        a = self.attn_post_norm(self.attn(h, inp, ex))
        h, x = self.ffn_pre_norm.add_forward(x, a)
        aux, stats = (), ()
        if self.is_moe:
            m, aux, stats = self.mlp(h, ex, name=f"layers.{self.layer_index}.mlp", layer_index=self.layer_index)
        else:
            m = self.mlp(h, ex)
        return x, self.ffn_post_norm(m), aux, stats


def trinity_layer_attention_kind(index: int, local_layers_per_global: int) -> str:
    return "global" if (index + 1) % (local_layers_per_global + 1) == 0 else "local"


def trinity_post_norm_scale(spec: ModelSpec) -> float:
    if spec.trinity is not None and spec.trinity.norm_policy == "afmoe_dual":
        return 1.0
    return 1.0 / math.sqrt(spec.num_layers)


class TransformerLM(nn.Module):
    """Embedding -> blocks -> final norm -> lm_head, for both ``model.name`` values."""

    def __init__(self, spec: ModelSpec, ex: ExecutionContext | None = None):
        super().__init__()
        ex = ex or ExecutionContext()
        self.spec = spec
        self.ex = ex
        H, V = spec.hidden_size, spec.vocab_size
        # default: the lm_head stays whole on every tensor-parallel rank and each rank scores its own sequence shard;
        # with ``vocab_parallel`` each rank holds V / tp rows of it and scores them for all tokens
        self.vocab_parallel = bool(ex.vocab_parallel and ex.tp_size > 1 and not spec.tied_embeddings)
        if ex.vocab_parallel and ex.tp_size > 1 and spec.tied_embeddings:
            raise ContractError("parallelism.vocab_parallel_head needs untied embeddings (model.tied_embeddings=false)")
        if self.vocab_parallel and V % ex.tp_size:
            raise ContractError(f"vocab_size {V} is not divisible by the tensor-parallel size {ex.tp_size}")
        self.vocab_local = V // ex.tp_size if self.vocab_parallel else V
        self.embed = nn.Parameter(torch.empty(V, H, dtype=torch.float32))
        self.embed_scale = 1.0
        layers: list[nn.Module] = []
        if spec.name == "trinity":
            tr = spec.trinity
            if tr is None:
                raise ContractError("model.name='trinity' requires [model.trinity]")
            self.embed_scale = math.sqrt(H)
            post_scale = trinity_post_norm_scale(spec)
            for i in range(spec.num_layers):
                kind = trinity_layer_attention_kind(i, tr.local_layers_per_global)
                cfg = AttentionConfig(
                    position="none" if kind == "global" else "rope",
                    mask="causal" if kind == "global" else "sliding_window",
                    local_window=None if kind == "global" else tr.local_window,
                    qk_norm=tr.qk_norm, gate=tr.attention_gate)
                moe = tr.moe if (tr.moe is not None and i >= tr.initial_dense_layers) else None
                layers.append(TrinityBlock(spec, cfg, moe, post_scale, ex, i))
        elif spec.name == "decoder":
            layers = [DecoderBlock(spec, ex) for _ in range(spec.num_layers)]
        else:
            raise ContractError(f"unsupported model.name {spec.name!r}")
        self.layers = nn.ModuleList(layers)
        # how many layers route tokens to experts: sizes the per-layer inboxes of the expert-parallel workspace
        ex.extras["moe_layer_count"] = sum(1 for layer in layers if getattr(layer, "is_moe", False))
        self.norm = RMSNorm(H, spec.norm_epsilon)
        self.lm_head = None if spec.tied_embeddings else nn.Parameter(
            torch.empty(self.vocab_local, H, dtype=torch.float32))
        self.compute_dtype = torch.float32
        # called with a layer index once every kernel of that layer's backward pass has been issued (the parameter
        # store starts that layer's gradient reduction from it); set per forward pass by the training step
        self.layer_backward_hook = None
        # called with a layer index right before that layer runs forward (weights sharded at rest are fetched by it)
        self.layer_prepare = None

    # ---- helpers ---------------------------------------------------------------------------------
    def head_weight(self) -> torch.Tensor:
        return self.embed if self.lm_head is None else self.lm_head

    def make_inputs(self, input_ids: torch.Tensor, token_doc_ids: torch.Tensor | None) -> ForwardInputs:
        B, S = input_ids.shape
        dev = input_ids.device
        chunks: tuple[tuple[int, int], ...] = ()
        if self.ex.cp_size > 1:
            from research_b200.steps.train import context_positions

            glob = context_positions(S * self.ex.cp_size, self.ex.cp_size, self.ex.cp_rank)
            cols = torch.as_tensor(glob, device=dev, dtype=torch.long)
            positions = cols.to(torch.int32).repeat(B)
            # contiguous runs of global positions (one for the contiguous split, two for zig-zag)
            breaks = [0] + [i for i in range(1, len(glob)) if glob[i] != glob[i - 1] + 1] + [len(glob)]
            chunks = tuple((int(glob[a]), b - a) for a, b in zip(breaks[:-1], breaks[1:]))
        else:
            cols = None
            positions = torch.arange(S, device=dev, dtype=torch.int32).repeat(B)
        lo = hi = None
        if token_doc_ids is not None and self.spec.attention_doc_mask:
            d = token_doc_ids.to(dev)                      # document ids of the WHOLE sequence, [B, S_full]
            full = d.shape[1]
            change = torch.ones(B, full, dtype=torch.bool, device=dev)
            change[:, 1:] = d[:, 1:] != d[:, :-1]
            idx = torch.arange(full, device=dev, dtype=torch.int32).expand(B, full)
            lo = torch.cummax(torch.where(change, idx, torch.zeros_like(idx)), dim=1).values.to(torch.int32)
            if cols is not None:
                lo = lo.index_select(1, cols).contiguous()  # this rank's rows, global kv positions
        return ForwardInputs(positions=positions, B=B, S=S, chunks=chunks, lo_causal=lo, hi_causal=hi)

    def hidden_states(self, input_ids: torch.Tensor, token_doc_ids: torch.Tensor | None = None):
        """Returns the final-normed hidden states ``[B, S(/tp), H]`` plus aux losses and router stats."""

        ex = self.ex
        inp = self.make_inputs(input_ids, token_doc_ids)
        x = Fn.embedding(input_ids, self.embed, self.embed_scale, self.compute_dtype)
        x = ex.scatter_sequence(x)
        delta = None
        aux_all: list[AuxLoss] = []
        stats_all: list[RouterStats] = []
        remat = self.spec.remat == "block" and torch.is_grad_enabled()
        hook = self.layer_backward_hook if torch.is_grad_enabled() else None
        for index, layer in enumerate(self.layers):
            if hook is not None and x.requires_grad:
                # the gradient of a layer's input is the last thing its backward pass produces
                x.register_hook(lambda grad, index=index, hook=hook: hook(index))
            if self.layer_prepare is not None:
                self.layer_prepare(index)
            if remat:
                x, delta, aux, stats = checkpoint(layer, x, delta, inp, ex, use_reentrant=False)
            else:
                x, delta, aux, stats = layer(x, delta, inp, ex)
            aux_all.extend(aux)
            stats_all.extend(stats)
        if hook is not None and x.requires_grad:
            # fires before the last layer's backward pass starts ("every layer from len(layers) up is done")
            x.register_hook(lambda grad, n=len(self.layers), hook=hook: hook(n))
        h, _ = self.norm.add_forward(x, delta)
        return h, tuple(aux_all), tuple(stats_all)

    def forward(self, input_ids: torch.Tensor, token_doc_ids: torch.Tensor | None = None) -> ModelOutput:
        h, aux, stats = self.hidden_states(input_ids, token_doc_ids)
        h = self.ex.gather_sequence(h)
        logits = self.full_logits(Fn.linear(h, self.head_weight()))
        return ModelOutput(logits=logits, aux_losses=aux, router_stats=stats)

    def full_logits(self, logits: torch.Tensor) -> torch.Tensor:
        """Logits over the whole vocabulary: with a vocabulary-parallel lm_head the ranks' slices are concatenated."""

        if not self.vocab_parallel:
            return logits
        from research_b200.models.execution import all_gather_dim

        return all_gather_dim(logits, self.ex.tp_group, logits.dim() - 1)

    # ---- inference with a dense functional KV cache --------------------------------------------
    def _infer_block(self, layer, x, delta, positions, attend):
        if isinstance(layer, DecoderBlock):
            h, x = layer.pre_norm.add_forward(x, delta)
            a = attend(layer.attn, h)
            h, x = layer.post_norm.add_forward(x, a)
            return x, layer.mlp(h, self.ex)
        h, x = layer.attn_pre_norm.add_forward(x, delta)
        a = layer.attn_post_norm(attend(layer.attn, h))
        h, x = layer.ffn_pre_norm.add_forward(x, a)
        if layer.is_moe:
            m = layer.mlp(h, self.ex, name="", layer_index=layer.layer_index)[0]
        else:
            m = layer.mlp(h, self.ex)
        return x, layer.ffn_post_norm(m)

    def run_with_cache(self, token_ids: torch.Tensor, positions: torch.Tensor, cache: Any, *,
                       last_only: bool = False) -> torch.Tensor:
        """token_ids, positions: [B,T].  Writes K/V for those positions into ``cache`` and returns logits [B,T,V]
        (``[B,1,V]`` for the last position only when ``last_only``: a prefill needs no other row)."""

        with self.ex.replicated_activations():
            x = Fn.embedding(token_ids, self.embed, self.embed_scale, self.compute_dtype)
            delta = None
            for li, layer in enumerate(self.layers):
                if self.layer_prepare is not None:
                    self.layer_prepare(li)
                def attend(attn: Attention, h, li=li):
                    q, k, v, x2 = attn.project_qkv(h, positions)
                    window = attn.cfg.local_window if attn.cfg.mask == "sliding_window" else None
                    o = cache.update_and_attend(li, q, k, v, positions, window)
                    return attn.finish(o, x2, self.ex)
                x, delta = self._infer_block(layer, x, delta, positions, attend)
            h, _ = self.norm.add_forward(x, delta)
            if last_only:
                h = h[:, -1:].contiguous()
            return self.full_logits(Fn.linear(h, self.head_weight()))
