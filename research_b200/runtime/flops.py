"""FLOP accounting and peak tables for MFU.

``estimate_flops_per_token`` is the reference's dense formula, kept for comparability
(src/jaxtitan/runtime/diagnostics.py:118-131): ``6 * matmul_params + 12 * L * heads * head_dim * seq_len``; it
ignores routed and shared expert work for MoE models.  ``estimate_flops_per_token_exact`` counts the parameters a
token actually visits (top-k routed experts + shared experts + router) and halves the attention term for the
causal mask.
"""

from __future__ import annotations

from research_b200.config.specs import ModelSpec

BF16_PEAK_FLOPS_TABLE = (
    (("gb200",), 2.5e15), (("grace blackwell",), 2.5e15), (("b200",), 2.25e15), (("b100",), 1.8e15),
    (("h200", "nvl"), 836e12), (("h200",), 989e12), (("h100", "nvl"), 835e12), (("h100", "pcie"), 756e12),
    (("h100",), 989e12), (("a100",), 312e12), (("l40s",), 362e12), (("gb10",), 125e12),
)


def peak_flops_for_device(device_name: str | None) -> float | None:
    if not device_name:
        return None
    name = device_name.lower().replace("nvidia", "").strip()
    for patterns, flops in BF16_PEAK_FLOPS_TABLE:
        if all(p in name for p in patterns):
            return flops
    return None


def estimate_flops_per_token(spec: ModelSpec, seq_len: int) -> int:
    head_dim = spec.hidden_size // spec.num_heads
    kv_width = spec.n_kv_heads * head_dim
    per_layer = (2 * spec.hidden_size * spec.hidden_size + 2 * spec.hidden_size * kv_width +
                 3 * spec.hidden_size * spec.intermediate_size)
    lm_head = 0 if spec.tied_embeddings else spec.hidden_size * spec.vocab_size
    matmul_params = spec.num_layers * per_layer + lm_head
    return int(6 * matmul_params + spec.num_layers * 12 * spec.num_heads * head_dim * seq_len)


def estimate_flops_per_token_exact(spec: ModelSpec, seq_len: int) -> int:
    H = spec.hidden_size
    head_dim = H // spec.num_heads
    kv_width = spec.n_kv_heads * head_dim
    attn = 2 * H * H + 2 * H * kv_width
    tr = spec.trinity
    total = 0
    for layer in range(spec.num_layers):
        layer_params = attn
        if tr is not None and tr.attention_gate:
            layer_params += H * H
        moe = tr.moe if (tr is not None and tr.moe is not None and layer >= tr.initial_dense_layers) else None
        if moe is None:
            layer_params += 3 * H * spec.intermediate_size
        else:
            inter = moe.expert_intermediate_size or spec.intermediate_size
            layer_params += 3 * H * inter * (moe.top_k + moe.num_shared_experts) + H * moe.num_experts
        total += layer_params
    total += H * spec.vocab_size  # lm_head (tied or not, the projection is computed)
    window = seq_len
    attention = 0
    for layer in range(spec.num_layers):
        local = tr is not None and (layer + 1) % (tr.local_layers_per_global + 1) != 0
        span = min(tr.local_window, seq_len) if local else seq_len
        attention += 12 * spec.num_heads * head_dim * span // 2
    del window
    return int(6 * total + attention)
