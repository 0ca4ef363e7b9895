"""Model construction, deterministic initialisation, and the logical parameter table.

``build_model`` returns the module plus one :class:`ParamMeta` per *logical* parameter using the reference's
path and tag scheme (src/jaxtitan/models/decoder.py:297-365) and layout policy (decoder.py:414-452): logical
kernels are ``[in, out]`` and expert stacks ``[E, in, out]``.  Each entry says where the values live in this
framework's fused ``[out, in]`` storage, so optimizers can route by tag and checkpoints can be written with the
reference's names and shapes.
"""

from __future__ import annotations

import hashlib
import math
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.nn as nn

from research_b200.config.specs import ModelSpec
from research_b200.errors import ContractError
from research_b200.models.execution import ExecutionContext
from research_b200.models.transformer import DecoderBlock, TransformerLM, TrinityBlock

ROUTED_EXPERT_TAGS = frozenset({"moe_gate", "moe_up", "moe_down"})
NORM_TAGS = frozenset({
    "attention_q_norm", "attention_k_norm", "attention_pre_norm", "attention_post_norm", "block_pre_norm",
    "block_post_norm", "ffn_pre_norm", "ffn_post_norm", "final_norm",
})


@dataclass(frozen=True)
class ParamMeta:
    """One logical parameter: reference path/tag/shape + where it is stored here."""

    path: tuple[str, ...]
    tag: str
    shape: tuple[int, ...]                 # logical (global) shape, reference layout
    storage: str                           # attribute path of the nn.Parameter holding the values
    rows: tuple[int, int] | None = None    # slice of the storage's "out" dimension (local indices)
    transposed: bool = False               # logical = storage^T over the last two dims
    logical_axes: tuple[str, ...] = ()
    fsdp_axis: int | None = None           # axis of the logical shape sharded by fsdp (reference policy)
    tp_axis: int | None = None             # axis of the logical shape sharded by tensor parallelism
    trainable: bool = True

    @property
    def name(self) -> str:
        return ".".join(self.path)

    @property
    def is_matrix(self) -> bool:
        return len(self.shape) >= 2 and self.tag not in ("embedding",)


@dataclass
class ModelBuildResult:
    model: TransformerLM
    metadata: tuple[ParamMeta, ...]
    execution: ExecutionContext
    spec: ModelSpec
    extras: dict[str, Any] = field(default_factory=dict)

    def storage_param(self, meta: ParamMeta) -> nn.Parameter:
        obj: Any = self.model
        for part in meta.storage.split("."):
            obj = obj[int(part)] if part.isdigit() else getattr(obj, part)
        return obj

    def storage_view(self, meta: ParamMeta, tensor: torch.Tensor | None = None) -> torch.Tensor:
        """The slice of ``tensor`` (default: the master parameter) that holds this logical parameter, in
        storage orientation (``[out, in]`` / ``[E, out, in]``)."""

        t = self.storage_param(meta).data if tensor is None else tensor
        if meta.rows is not None:
            a, b = meta.rows
            t = t[:, a:b] if t.dim() == 3 else t[a:b]
        return t

    def logical_view(self, meta: ParamMeta, tensor: torch.Tensor | None = None) -> torch.Tensor:
        t = self.storage_view(meta, tensor)
        return t.transpose(-1, -2) if meta.transposed else t

    def parameter_count(self) -> int:
        return sum(math.prod(m.shape) for m in self.metadata)


_LAYOUT = {
    "embedding": (("vocab", "hidden"), None, None),
    "lm_head": (("hidden", "vocab"), 0, None),
    "attention_q": (("hidden_in", "hidden_out"), 1, 1),
    "attention_k": (("hidden_in", "hidden_out"), 1, 1),
    "attention_v": (("hidden_in", "hidden_out"), 1, 1),
    "attention_gate": (("hidden_in", "hidden_out"), 1, 1),
    "attention_o": (("hidden_in", "hidden_out"), 0, 0),
    "mlp_gate": (("hidden", "intermediate"), 1, 1),
    "mlp_up": (("hidden", "intermediate"), 1, 1),
    "mlp_down": (("intermediate", "hidden"), 0, 0),
    "moe_router": (("hidden", "expert"), None, None),
    "moe_expert_bias": (("expert",), None, None),
    "moe_gate": (("expert", "hidden", "intermediate"), None, None),
    "moe_up": (("expert", "hidden", "intermediate"), None, None),
    "moe_down": (("expert", "intermediate", "hidden"), None, None),
    "moe_shared_gate": (("hidden", "intermediate"), 1, 1),
    "moe_shared_up": (("hidden", "intermediate"), 1, 1),
    "moe_shared_down": (("intermediate", "hidden"), 0, 0),
}


# axis of the logical shape that the ``expert_fsdp`` mesh axis splits (reference: mesh/sharding.py:524-538)
EXPERT_FSDP_AXIS = {"moe_gate": 2, "moe_up": 2, "moe_down": 1}


def layout_policy(tag: str, rank: int):
    if tag in _LAYOUT:
        return _LAYOUT[tag]
    if tag in NORM_TAGS:
        return tuple("norm" for _ in range(rank)), None, None
    return tuple("replicated" for _ in range(rank)), None, None


def _meta(path: str, tag: str, shape, storage: str, rows=None, transposed=False, trainable=True) -> ParamMeta:
    axes, fsdp_axis, tp_axis = layout_policy(tag, len(shape))
    return ParamMeta(tuple(path.split(".")), tag, tuple(int(s) for s in shape), storage, rows, transposed, axes,
                     fsdp_axis, tp_axis, trainable)


def _attention_entries(prefix: str, attn, spec: ModelSpec, tp: int) -> list[ParamMeta]:
    D, H = spec.head_dim, spec.hidden_size
    hq, hkv = attn.hq, attn.hkv
    out = [
        _meta(f"{prefix}.attn.q.kernel", "attention_q", (H, spec.num_heads * D), f"{prefix}.attn.wqkv", (0, hq * D), True),
        _meta(f"{prefix}.attn.k.kernel", "attention_k", (H, spec.n_kv_heads * D), f"{prefix}.attn.wqkv",
              (hq * D, (hq + hkv) * D), True),
        _meta(f"{prefix}.attn.v.kernel", "attention_v", (H, spec.n_kv_heads * D), f"{prefix}.attn.wqkv",
              ((hq + hkv) * D, (hq + 2 * hkv) * D), True),
        _meta(f"{prefix}.attn.o.kernel", "attention_o", (spec.num_heads * D, H), f"{prefix}.attn.wo", None, True),
    ]
    if attn.q_norm is not None:
        out.append(_meta(f"{prefix}.attn.q_norm.scale", "attention_q_norm", (D,), f"{prefix}.attn.q_norm"))
        out.append(_meta(f"{prefix}.attn.k_norm.scale", "attention_k_norm", (D,), f"{prefix}.attn.k_norm"))
    if attn.wgate is not None:
        out.append(_meta(f"{prefix}.attn.gate.kernel", "attention_gate", (H, spec.num_heads * D),
                         f"{prefix}.attn.wgate", None, True))
    return out


def _swiglu_entries(prefix: str, mlp, hidden: int, inter_total: int, tags: tuple[str, str, str],
                    names=("gate", "up", "down")) -> list[ParamMeta]:
    i_local = mlp.w_gate_up.shape[0] // 2
    return [
        _meta(f"{prefix}.{names[0]}.kernel", tags[0], (hidden, inter_total), f"{prefix}.w_gate_up", (0, i_local), True),
        _meta(f"{prefix}.{names[1]}.kernel", tags[1], (hidden, inter_total), f"{prefix}.w_gate_up",
              (i_local, 2 * i_local), True),
        _meta(f"{prefix}.{names[2]}.kernel", tags[2], (inter_total, hidden), f"{prefix}.w_down", None, True),
    ]


def logical_parameters(model: TransformerLM) -> tuple[ParamMeta, ...]:
    spec, ex = model.spec, model.ex
    H, V = spec.hidden_size, spec.vocab_size
    entries: list[ParamMeta] = [_meta("embed.embedding", "embedding", (V, H), "embed")]
    for i, layer in enumerate(model.layers):
        pre = f"layers.{i}"
        if isinstance(layer, DecoderBlock):
            entries.append(_meta(f"{pre}.pre_norm.scale", "block_pre_norm", (H,), f"{pre}.pre_norm.scale"))
            entries += _attention_entries(pre, layer.attn, spec, ex.tp_size)
            entries.append(_meta(f"{pre}.post_norm.scale", "block_post_norm", (H,), f"{pre}.post_norm.scale"))
            entries += _swiglu_entries(f"{pre}.mlp", layer.mlp, H, spec.intermediate_size,
                                       ("mlp_gate", "mlp_up", "mlp_down"))
        elif isinstance(layer, TrinityBlock):
            entries.append(_meta(f"{pre}.attn_pre_norm.scale", "attention_pre_norm", (H,), f"{pre}.attn_pre_norm.scale"))
            entries += _attention_entries(pre, layer.attn, spec, ex.tp_size)
            entries.append(_meta(f"{pre}.attn_post_norm.scale", "attention_post_norm", (H,), f"{pre}.attn_post_norm.scale"))
            entries.append(_meta(f"{pre}.ffn_pre_norm.scale", "ffn_pre_norm", (H,), f"{pre}.ffn_pre_norm.scale"))
            if layer.is_moe:
                moe = layer.mlp
                E, I_local = moe.num_experts, moe.experts.inter
                I = I_local * ex.efsdp_size                        # logical (global) intermediate size
                entries.append(_meta(f"{pre}.mlp.router.proj.kernel", "moe_router", (H, E), f"{pre}.mlp.router.proj",
                                     None, True))
                entries.append(_meta(f"{pre}.mlp.expert_bias", "moe_expert_bias", (E,), f"{pre}.mlp.expert_bias",
                                     trainable=False))
                entries.append(_meta(f"{pre}.mlp.experts.gate", "moe_gate", (E, H, I), f"{pre}.mlp.experts.w_gate_up",
                                     (0, I_local), True))
                entries.append(_meta(f"{pre}.mlp.experts.up", "moe_up", (E, H, I), f"{pre}.mlp.experts.w_gate_up",
                                     (I_local, 2 * I_local), True))
                entries.append(_meta(f"{pre}.mlp.experts.down", "moe_down", (E, I, H), f"{pre}.mlp.experts.w_down",
                                     None, True))
                if moe.shared_experts is not None:
                    shared_inter = moe.moe.expert_intermediate_size * moe.moe.num_shared_experts
                    entries += _swiglu_entries(f"{pre}.mlp.shared_experts", moe.shared_experts, H, shared_inter,
                                               ("moe_shared_gate", "moe_shared_up", "moe_shared_down"))
            else:
                entries += _swiglu_entries(f"{pre}.mlp", layer.mlp, H, spec.intermediate_size,
                                           ("mlp_gate", "mlp_up", "mlp_down"))
            entries.append(_meta(f"{pre}.ffn_post_norm.scale", "ffn_post_norm", (H,), f"{pre}.ffn_post_norm.scale"))
        else:
            raise ContractError(f"unrecognized layer type {type(layer).__name__}")
    entries.append(_meta("norm.scale", "final_norm", (H,), "norm.scale"))
    if model.lm_head is not None:
        head = _meta("lm_head.kernel", "lm_head", (H, V), "lm_head", None, True)
        if model.vocab_parallel:      # split over the vocabulary (logical axis 1) across the tensor-parallel group
            import dataclasses

            head = dataclasses.replace(head, tp_axis=1)
        entries.append(head)
    return tuple(entries)


# --------------------------------------------------------------------------------------------------
# initialisation
# --------------------------------------------------------------------------------------------------
def _seed_for(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 62) - 1)


def _normal(shape, std: float, seed: int, device, trunc: float | None) -> torch.Tensor:
    gen = torch.Generator(device=device).manual_seed(seed)
    t = torch.empty(shape, dtype=torch.float32, device=device)
    if trunc is None:
        t.normal_(0.0, std, generator=gen)
    else:
        nn.init.trunc_normal_(t, mean=0.0, std=std, a=-trunc * std, b=trunc * std, generator=gen)
    return t


def _shard(full: torch.Tensor, axis: int | None, size: int, rank: int) -> torch.Tensor:
    if axis is None or size == 1:
        return full
    return full.chunk(size, dim=axis)[rank]


@torch.no_grad()
def initialize_parameters(result: ModelBuildResult, seed: int) -> None:
    """Fill every logical parameter from a per-path seed, so all ranks and all layouts see the same values.

    ``nnx_default``: kernels ~ N(0, 1/fan_in), embedding ~ N(0, 1/hidden) (Flax NNX defaults of the reference
    decoder); ``normal_0.02``: N(0, 0.02) for every matrix; Trinity: truncated normal (+-3 sigma) with
    ``init_std`` (default 0.5/sqrt(hidden)) (reference: models/trinity.py:35-36, components/init.py:10-17).
    Norm scales keep their constructor value; ``expert_bias`` starts at zero.
    """

    spec, ex = result.spec, result.execution
    trinity = spec.name == "trinity"
    tr_std = None
    if trinity:
        tr_std = spec.trinity.init_std if spec.trinity.init_std is not None else 0.5 / math.sqrt(spec.hidden_size)
    for meta in result.metadata:
        if meta.tag in NORM_TAGS or meta.tag == "moe_expert_bias":
            continue
        dest = result.logical_view(meta)
        device = dest.device
        fan_in = meta.shape[-2] if len(meta.shape) >= 2 else meta.shape[0]
        if trinity:
            std, trunc = tr_std, 3.0
        elif spec.init == "normal_0.02":
            std, trunc = 0.02, None
        elif meta.tag == "embedding":
            std, trunc = 1.0 / math.sqrt(meta.shape[1]), None
        else:
            std, trunc = 1.0 / math.sqrt(fan_in), None
        full = _normal(meta.shape, std, _seed_for(seed, meta.name), device, trunc)
        local = _shard(full, meta.tp_axis, ex.tp_size, ex.tp_rank)
        if meta.tag in ROUTED_EXPERT_TAGS:
            local = _shard(local, 0, ex.ep_size, ex.ep_rank)
            local = _shard(local, EXPERT_FSDP_AXIS[meta.tag], ex.efsdp_size, ex.efsdp_rank)
        dest.copy_(local)


def build_model(spec: ModelSpec, *, seed: int = 0, execution: ExecutionContext | None = None,
                device: torch.device | str = "cpu", initialize: bool = True) -> ModelBuildResult:
    ex = execution or ExecutionContext()
    with torch.device(device):
        model = TransformerLM(spec, ex)
    result = ModelBuildResult(model=model, metadata=logical_parameters(model), execution=ex, spec=spec)
    if initialize:
        initialize_parameters(result, seed)
    return result


def count_parameters(metadata) -> int:
    """Number of scalar parameters described by a parameter table."""

    total = 0
    for meta in metadata:
        n = 1
        for d in meta.shape:
            n *= int(d)
        total += n
    return total


def dtype_from_name(name: str):
    """``"float32" | "bfloat16" | "float16"`` -> the torch dtype (the names the run contract uses)."""

    import torch

    table = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}
    if name not in table:
        raise ContractError(f"unsupported dtype name {name!r}; expected one of {sorted(table)}")
    return table[name]


def apply_model(model, input_ids, token_doc_ids=None):
    """Forward pass returning the :class:`ModelOutput` (logits, auxiliary losses, router statistics)."""

    return model(input_ids, token_doc_ids)
