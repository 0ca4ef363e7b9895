"""Decode attention over the KV cache (one query token per sequence) on the native split-KV kernel.

The kernel reads only rows ``[lo[b], lengths[b])`` of each sequence's cache, for all query heads of a GQA group at
once; see ``csrc/decode.cu``.  The reference attends over the whole padded cache every step
(src/jaxtitan/infer/generation.py:302, models/components/attention.py:213-218).
"""

from __future__ import annotations

import os

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


def _launch(q, k_base, v_base, lengths, lo, *, B, Hq, Hkv, D, rows, strides, page_rows, scale, kernel="auto"):
    """``kernel``: "stream" (tiles through shared memory with bulk asynchronous copies; needs rows that are
    contiguous inside a page and pages of a multiple of 64 rows), "registers" (16-byte loads into registers, any
    strides) or "auto" (stream where the layout allows it)."""

    lib = native.load()
    # the streaming kernel takes the queries where the projection left them (rows of a packed q|k buffer)
    strided_q = q.dim() == 3 and q.stride(2) == 1 and q.stride(1) == D and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
    if not strided_q:
        q = q.contiguous()
    lengths = lengths.to(torch.int32).contiguous()
    lo = None if lo is None else lo.to(torch.int32).contiguous()
    k_row, k_batch, k_head, k_page = strides
    can_stream = k_row == D and page_rows % 64 == 0 and k_batch % 8 == 0 and k_head % 8 == 0 and k_page % 8 == 0
    if kernel == "stream" and not can_stream:
        raise KernelError("the streaming decode kernel needs head-major pages of a multiple of 64 rows")
    stream = can_stream and kernel != "registers" and os.environ.get("RESEARCH_B200_DECODE_STREAM", "1") != "0"
    splits = (lib.b200_decode_attn_paged_splits if stream else lib.b200_decode_attn_splits)(B, Hq, Hkv, rows)
    part_o = native.scratch("decode_part_o", B * Hq * splits * D, torch.float32, q.device)
    part_ml = native.scratch("decode_part_ml", B * Hq * splits * 2, torch.float32, q.device)
    out = torch.empty((B, Hq, D), dtype=torch.bfloat16, device=q.device)
    lo_ptr = None if lo is None else lo.data_ptr()
    sm_scale = float(D ** -0.5 if scale is None else scale)
    if stream:
        rc = lib.b200_decode_attn_paged(q.data_ptr(), k_base.data_ptr(), v_base.data_ptr(), out.data_ptr(),
                                        lengths.data_ptr(), lo_ptr, part_o.data_ptr(), part_ml.data_ptr(), B, Hq, Hkv,
                                        D, k_batch, k_head, k_page, page_rows, sm_scale, splits, q.stride(0),
                                        native.status_word(q.device).data_ptr(), native._stream())
        native._check(rc, "b200_decode_attn_paged")
    else:
        q = q.contiguous()
        rc = lib.b200_decode_attn(q.data_ptr(), k_base.data_ptr(), v_base.data_ptr(), out.data_ptr(),
                                  lengths.data_ptr(), lo_ptr, part_o.data_ptr(), part_ml.data_ptr(), B, Hq, Hkv, D,
                                  k_row, k_batch, k_row, k_batch, k_head, k_head, k_page, k_page, page_rows, sm_scale,
                                  splits, native._stream())
        native._check(rc, "b200_decode_attn")
    native.LAUNCHES += 1  # _check counts one launch; the merge kernel is the second
    return out.view(B, Hq * D)


def _check_q(q, Hkv):
    B, Hq, D = q.shape
    if q.dtype != torch.bfloat16 or D not in (64, 128) or Hq % Hkv or Hq // Hkv not in (1, 2, 4, 8):
        raise KernelError(f"decode_attention supports bf16, head_dim 64/128 and GQA groups 1/2/4/8; got {q.dtype}, "
                          f"D={D}, Hq={Hq}, Hkv={Hkv}")


def decode_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, lengths: torch.Tensor,
                     lo: torch.Tensor | None = None, scale: float | None = None) -> torch.Tensor:
    """q ``[B,Hq,D]`` bf16, caches ``[B,rows,Hkv,D]`` bf16 views (dense last dim, heads D apart), ``lengths`` int32
    ``[B]``, ``lo`` int32 ``[B]`` or None.  Returns ``[B, Hq*D]`` bf16."""

    if not q.is_cuda:
        return decode_attention_reference(q, k_cache, v_cache, lengths, lo)
    B, Hq, D = q.shape
    rows, Hkv = k_cache.shape[1], k_cache.shape[2]
    for t, name in ((k_cache, "k_cache"), (v_cache, "v_cache")):
        if t.dim() != 4 or t.stride(3) != 1 or t.stride(2) != D or t.dtype != torch.bfloat16:
            raise KernelError(f"{name} must be a bf16 [B,rows,Hkv,D] view with heads D elements apart")
    if k_cache.stride() != v_cache.stride():
        raise KernelError("k_cache and v_cache must share their strides")
    _check_q(q, Hkv)
    return _launch(q, k_cache, v_cache, lengths, lo, B=B, Hq=Hq, Hkv=Hkv, D=D, rows=rows,
                   strides=(k_cache.stride(1), k_cache.stride(0), D, 0), page_rows=max(rows, 1), scale=scale)


def decode_attention_paged(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, lengths: torch.Tensor,
                           lo: torch.Tensor | None = None, scale: float | None = None,
                           kernel: str = "auto") -> torch.Tensor:
    """Head-major paged caches ``[B, pages, Hkv, page_rows, D]`` (contiguous): every (page, head) is one dense
    ``page_rows x D`` block, so a CTA streams contiguous memory.  Returns ``[B, Hq*D]`` bf16."""

    B, Hq, D = q.shape
    _, pages, Hkv, page_rows, _ = k_pool.shape
    if not (k_pool.is_contiguous() and v_pool.is_contiguous()) or k_pool.dtype != torch.bfloat16:
        raise KernelError("paged caches must be contiguous bf16 [B, pages, Hkv, page_rows, D]")
    _check_q(q, Hkv)
    return _launch(q, k_pool, v_pool, lengths, lo, B=B, Hq=Hq, Hkv=Hkv, D=D, rows=pages * page_rows,
                   strides=(D, k_pool.stride(0), k_pool.stride(2), k_pool.stride(1)), page_rows=page_rows, scale=scale,
                   kernel=kernel)


def kv_append_paged(k_new: torch.Tensor, v_new: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                    positions: torch.Tensor) -> None:
    """Write one new token per sequence (``k_new`` / ``v_new``: ``[B, Hkv, D]`` views with dense heads) at row
    ``positions[b]`` of head-major paged caches ``[B, pages, Hkv, page_rows, D]``."""

    lib = native.load()
    B, Hkv, D = k_new.shape
    if k_new.stride(2) != 1 or k_new.stride(1) != D or v_new.stride(2) != 1 or v_new.stride(1) != D:
        raise KernelError("k_new / v_new must be [B,Hkv,D] views with heads D elements apart")
    positions = positions.to(torch.int32).contiguous()
    rc = lib.b200_kv_append(k_new.data_ptr(), v_new.data_ptr(), k_new.stride(0), v_new.stride(0), k_pool.data_ptr(),
                            v_pool.data_ptr(), positions.data_ptr(), k_pool.stride(0), k_pool.stride(2),
                            k_pool.stride(1), D, k_pool.shape[3], B, Hkv, D, native._stream())
    native._check(rc, "b200_kv_append")
