"""Decode attention over the KV cache (one query token per sequence) on the native split-KV kernel.

The kernel reads only rows ``[lo[b], lengths[b])`` of each sequence's cache, for all query heads of a GQA group at
once; see ``csrc/decode.cu``.  The reference attends over the whole padded cache every step
(src/jaxtitan/infer/generation.py:302, models/components/attention.py:213-218).
"""

from __future__ import annotations

import torch

from research_b200.errors import KernelError
from research_b200.ops import native


def decode_attention_reference(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, lengths: torch.Tensor,
                               lo: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 restatement: q ``[B,Hq,D]``, caches ``[B,rows,Hkv,D]`` -> ``[B, Hq*D]`` in q's dtype."""

    B, Hq, D = q.shape
    rows, Hkv = k_cache.shape[1], k_cache.shape[2]
    g = Hq // Hkv
    kf = k_cache.float().repeat_interleave(g, dim=2)
    vf = v_cache.float().repeat_interleave(g, dim=2)
    s = torch.einsum("bhd,bkhd->bhk", q.float(), kf) * (D ** -0.5)
    pos = torch.arange(rows, device=q.device)[None, :]
    allowed = pos < lengths[:, None]
    if lo is not None:
        allowed = allowed & (pos >= lo[:, None])
    s = s.masked_fill(~allowed[:, None, :], float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    return torch.einsum("bhk,bkhd->bhd", p, vf).to(q.dtype).reshape(B, Hq * D)


def decode_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, lengths: torch.Tensor,
                     lo: torch.Tensor | None = None, scale: float | None = None) -> torch.Tensor:
    """q ``[B,Hq,D]`` bf16, caches ``[B,rows,Hkv,D]`` bf16 views (dense last dim, heads D apart), ``lengths`` int32
    ``[B]``, ``lo`` int32 ``[B]`` or None.  Returns ``[B, Hq*D]`` bf16."""

    if not q.is_cuda:
        return decode_attention_reference(q, k_cache, v_cache, lengths, lo)
    lib = native.load()
    B, Hq, D = q.shape
    rows, Hkv = k_cache.shape[1], k_cache.shape[2]
    for t, name in ((k_cache, "k_cache"), (v_cache, "v_cache")):
        if t.dim() != 4 or t.stride(3) != 1 or t.stride(2) != D or t.dtype != torch.bfloat16:
            raise KernelError(f"{name} must be a bf16 [B,rows,Hkv,D] view with heads D elements apart")
    if q.dtype != torch.bfloat16 or D not in (64, 128) or Hq % Hkv or Hq // Hkv not in (1, 2, 4, 8):
        raise KernelError(f"decode_attention supports bf16, head_dim 64/128 and GQA groups 1/2/4/8; got {q.dtype}, "
                          f"D={D}, Hq={Hq}, Hkv={Hkv}")
    q = q.contiguous()
    lengths = lengths.to(torch.int32).contiguous()
    lo = None if lo is None else lo.to(torch.int32).contiguous()
    splits = lib.b200_decode_attn_splits(B, Hkv, rows)
    part_o = native.scratch("decode_part_o", B * Hq * splits * D, torch.float32, q.device)
    part_ml = native.scratch("decode_part_ml", B * Hq * splits * 2, torch.float32, q.device)
    out = torch.empty((B, Hq, D), dtype=torch.bfloat16, device=q.device)
    rc = lib.b200_decode_attn(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                              lengths.data_ptr(), None if lo is None else lo.data_ptr(), part_o.data_ptr(),
                              part_ml.data_ptr(), B, Hq, Hkv, D, k_cache.stride(1), k_cache.stride(0),
                              v_cache.stride(1), v_cache.stride(0), float(D ** -0.5 if scale is None else scale),
                              splits, native._stream())
    native._check(rc, "b200_decode_attn")
    native.LAUNCHES += 1  # _check counts one launch; the merge kernel is the second
    return out.view(B, Hq * D)
