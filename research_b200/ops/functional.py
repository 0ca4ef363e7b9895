"""Differentiable building blocks of the models, each with two implementations behind one signature:

* the sm_100a kernels of :mod:`research_b200.ops.native` (bf16 tensors on a CUDA device), wrapped in
  ``torch.autograd.Function`` s whose backward passes call the matching backward kernels, and
* a plain PyTorch restatement (any device / dtype) that is the CPU path and the numerics oracle.

Weights are fp32 master ``nn.Parameter`` s.  On the native path the forward reads the parameter's bf16
``shadow`` and the backward adds the weight gradient straight into its fp32 ``main_grad`` (GEMM epilogue
TMA reduce-add), returning no autograd gradient for the parameter - so no per-parameter ``.grad`` tensors
exist on the GPU path.  On the reference path ordinary autograd populates ``.grad``.
"""

from __future__ import annotations

import math
import os
from contextlib import contextmanager

import torch
import torch.nn.functional as F

from research_b200.ops import native

# RESEARCH_B200_LIBRARY=1 runs the whole stack on stock PyTorch operators (cuBLAS matmuls, the library's
# scaled_dot_product_attention, plain tensor ops in the optimizer, NCCL collectives): the comparison arm of the
# benchmark.  None of this package's kernels runs in that mode.
_LIBRARY = os.environ.get("RESEARCH_B200_LIBRARY", "0") == "1"
_FORCE_REFERENCE = _LIBRARY


def library_mode() -> bool:
    return _LIBRARY


def set_library_mode(enabled: bool) -> None:
    """Switch library mode for objects built after this call (the benchmark's comparison arm)."""

    global _LIBRARY, _FORCE_REFERENCE
    _LIBRARY = bool(enabled)
    _FORCE_REFERENCE = bool(enabled)


def native_enabled() -> bool:
    """False while the plain PyTorch implementations are forced (library mode, ``reference_mode``)."""

    return not _FORCE_REFERENCE


@contextmanager
def reference_mode(enabled: bool = True):
    """Run the plain PyTorch implementations even on CUDA bf16 tensors (used by parity tests)."""

    global _FORCE_REFERENCE
    old = _FORCE_REFERENCE
    _FORCE_REFERENCE = enabled
    try:
        yield
    finally:
        _FORCE_REFERENCE = old


def use_native(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and not _FORCE_REFERENCE


def _ordered_sums_only() -> bool:
    """True in the deterministic debugging mode: kernels that add partial sums in arrival order (fp32 atomics for
    the gradients of norm scales and of the embedding table) give way to the PyTorch forms, whose reductions have a
    fixed order."""

    return native.deterministic()


def compute_weight(p: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    """The tensor a kernel multiplies with: the bf16 shadow on the native path, a cast view otherwise."""

    shadow = getattr(p, "shadow", None)
    if shadow is not None and shadow.dtype == like.dtype and shadow.device == like.device:
        return shadow
    return p.to(like.dtype)


def _main_grad(p: torch.Tensor) -> torch.Tensor:
    mg = getattr(p, "main_grad", None)
    if mg is None:
        mg = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
        p.main_grad = mg
    return mg


# --------------------------------------------------------------------------------------------------
# linear
# --------------------------------------------------------------------------------------------------
class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p):
        w = compute_weight(p, x)
        x2 = x.reshape(-1, x.shape[-1])
        y = native.gemm(x2, w, trans_b=True)
        ctx.save_for_backward(x2)
        ctx.p = p
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        p = ctx.p
        w = compute_weight(p, x2)
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = native.gemm(dy2, w, trans_b=False).view(ctx.x_shape)
        if p.requires_grad:
            native.gemm_wgrad(dy2, x2, _main_grad(p))
        return dx, None


def linear(x: torch.Tensor, p: torch.Tensor) -> torch.Tensor:
    """``y = x @ W^T`` with ``W`` stored ``[out, in]``."""

    if use_native(x):
        if not torch.is_grad_enabled() and x.numel() // x.shape[-1] <= 64:
            # decode-sized input: stream the weight with the whole device (split-K), no autograd bookkeeping
            w = compute_weight(p, x)
            y = native.gemm_skinny(x.reshape(-1, x.shape[-1]), w)
            return y.view(*x.shape[:-1], w.shape[0])
        return _LinearFn.apply(x, p)
    return F.linear(x, p.to(x.dtype))


# --------------------------------------------------------------------------------------------------
# RMSNorm (+ residual add)
# --------------------------------------------------------------------------------------------------
class _RmsNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, delta, p, eps):
        y, rstd, res = native.rmsnorm_fwd(x.contiguous(), p, eps, None if delta is None else delta.contiguous())
        ctx.save_for_backward(res, rstd)
        ctx.p = p
        ctx.has_delta = delta is not None
        ctx.set_materialize_grads(False)
        if delta is None:
            dummy = y.new_empty(0)
            ctx.mark_non_differentiable(dummy)
            return y, dummy
        return y, res

    @staticmethod
    def backward(ctx, dy, dres):
        res, rstd = ctx.saved_tensors
        p = ctx.p
        if dy is None:
            return dres, (dres if ctx.has_delta else None), None, None
        dx = native.rmsnorm_bwd(res, p, rstd, dy.contiguous(), _main_grad(p),
                                None if dres is None else dres.contiguous())
        return dx, (dx if ctx.has_delta else None), None, None


def _rmsnorm_ref(x, w, eps):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return y.to(x.dtype)


def rmsnorm(x: torch.Tensor, p: torch.Tensor, eps: float) -> torch.Tensor:
    if use_native(x) and not (_ordered_sums_only() and p.requires_grad and torch.is_grad_enabled()):
        return _RmsNormFn.apply(x, None, p, eps)[0]
    return _rmsnorm_ref(x, p, eps)


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor, p: torch.Tensor, eps: float):
    """``res = x + delta; y = rmsnorm(res)``; returns ``(y, res)`` from one pass over the data."""

    if use_native(x) and not (_ordered_sums_only() and p.requires_grad and torch.is_grad_enabled()):
        return _RmsNormFn.apply(x, delta, p, eps)
    res = x + delta
    return _rmsnorm_ref(res, p, eps), res


# --------------------------------------------------------------------------------------------------
# QK-RMSNorm + RoPE (interleaved pairs) on a packed [tokens, (Hq + 2 Hkv) * D] projection
# --------------------------------------------------------------------------------------------------
def rope_reference(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """x: [..., T, H, D]; positions: [..., T].  Rotates (even, odd) pairs (reference: position.py:23-26)."""

    D = x.shape[-1]
    inv = theta ** (-torch.arange(0, D, 2, device=x.device, dtype=torch.float32) / D)
    ang = positions.float()[..., None, None] * inv
    c, s = ang.cos(), ang.sin()
    a, b = x[..., 0::2].float(), x[..., 1::2].float()
    return torch.stack([a * c - b * s, a * s + b * c], dim=-1).flatten(-2).to(x.dtype)


class _QkNormRopeFn(torch.autograd.Function):
    """in: packed qkv [T, (Hq+2Hkv)*D]; out: q|k part [T, (Hq+Hkv)*D] normalised and rotated."""

    @staticmethod
    def forward(ctx, qkv, wq, wk, positions, hq, hkv, D, eps, theta, rope):
        T = qkv.shape[0]
        out = torch.empty(T, (hq + hkv) * D, dtype=qkv.dtype, device=qkv.device)
        rq = native.qknorm_rope_fwd_qk(qkv, out, wq, wk, positions, hq, hkv, D, eps, theta, rope)
        rk = None
        ctx.save_for_backward(qkv, positions, rq, rk)
        ctx.params = (wq, wk)
        ctx.cfg = (hq, hkv, D, theta, rope)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, positions, rq, rk = ctx.saved_tensors
        wq, wk = ctx.params
        hq, hkv, D, theta, rope = ctx.cfg
        dout = dout.contiguous()
        dqkv = torch.empty_like(qkv)
        dqkv[:, (hq + hkv) * D:].zero_()  # the V columns get no gradient through this op; the kernel writes the rest
        native.qknorm_rope_bwd_qk(qkv, dout, dqkv, wq, wk, positions, rq, None if wq is None else _main_grad(wq),
                                  None if wk is None else _main_grad(wk), hq, hkv, D, theta, rope)
        return dqkv, None, None, None, None, None, None, None, None, None


def qk_norm_rope(qkv: torch.Tensor, wq, wk, positions: torch.Tensor, hq: int, hkv: int, D: int, eps: float,
                 theta: float, rope: bool) -> torch.Tensor:
    """Normalise (if weights given) and rotate (if ``rope``) the q and k heads of a packed projection.

    qkv: ``[T, (hq + 2 hkv) * D]``; positions: int32 ``[T]``.  Returns ``[T, (hq + hkv) * D]``.
    """

    if use_native(qkv) and not (_ordered_sums_only() and wq is not None and torch.is_grad_enabled()):
        return _QkNormRopeFn.apply(qkv, wq, wk, positions, hq, hkv, D, eps, theta, rope)
    T = qkv.shape[0]
    q = qkv[:, : hq * D].reshape(T, hq, D)
    k = qkv[:, hq * D:(hq + hkv) * D].reshape(T, hkv, D)
    if wq is not None:
        q = _rmsnorm_ref(q, wq, eps)
        k = _rmsnorm_ref(k, wk, eps)
    if rope:
        q = rope_reference(q, positions, theta)
        k = rope_reference(k, positions, theta)
    return torch.cat([q.reshape(T, hq * D), k.reshape(T, hkv * D)], dim=1)


# --------------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------------
def attention_reference(q, k, v, *, causal: bool, lo: torch.Tensor | None, scale: float) -> torch.Tensor:
    """softmax(QK^T * scale) V with fp32 logits; q: [B,S,Hq,D], k/v: [B,Sk,Hkv,D]; row r sees kv in [lo[r], r]."""

    B, S, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    qf = q.permute(0, 2, 1, 3).float()
    kf = k.permute(0, 2, 1, 3).repeat_interleave(g, dim=1).float()
    vf = v.permute(0, 2, 1, 3).repeat_interleave(g, dim=1).float()
    s = torch.einsum("bhqd,bhkd->bhqk", qf, kf) * scale
    qi = torch.arange(S, device=q.device) + (Sk - S)
    ki = torch.arange(Sk, device=q.device)
    allowed = torch.ones(B, 1, S, Sk, dtype=torch.bool, device=q.device)
    if causal:
        allowed = allowed & (qi[None, None, :, None] >= ki[None, None, None, :])
    if lo is not None:
        allowed = allowed & (ki[None, None, None, :] >= lo.long()[:, None, :, None])
    s = s.masked_fill(~allowed, float("-inf"))
    p = torch.softmax(s, dim=-1).to(q.dtype).float()
    o = torch.einsum("bhqk,bhkd->bhqd", p, vf)
    return o.permute(0, 2, 1, 3).to(q.dtype)


class _AttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, lo, hi, causal, scale):
        o, lse = native.attn_fwd(q, k, v, causal=causal, lo=lo, scale=scale)
        ctx.save_for_backward(q, k, v, o, lse, lo, hi)
        ctx.cfg = (causal, scale)
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse, lo, hi = ctx.saved_tensors
        causal, scale = ctx.cfg
        if d_o.stride(3) != 1 or d_o.stride(2) != d_o.shape[3]:
            d_o = d_o.contiguous()
        dq, dk, dv = native.attn_bwd(q, k, v, o, d_o, lse, causal=causal, lo=lo, hi=hi, scale=scale)
        return dq, dk, dv, None, None, None, None


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = True,
              lo: torch.Tensor | None = None, hi: torch.Tensor | None = None,
              scale: float | None = None) -> torch.Tensor:
    """GQA attention over ``[B,S,H,D]`` views.  ``lo`` int32 ``[B,S]`` = first visible kv position per row."""

    D = q.shape[-1]
    if scale is None:
        scale = D ** -0.5
    if use_native(q) and D in (64, 128):
        if lo is not None and hi is None:
            hi = native.kv_visibility_upper_bound(lo)
        return _AttentionFn.apply(q, k, v, lo, hi, causal, scale)
    if _LIBRARY and q.is_cuda:
        return attention_library(q, k, v, causal=causal, lo=lo, scale=scale)
    return attention_reference(q, k, v, causal=causal, lo=lo, scale=scale)


def attention_library(q, k, v, *, causal: bool, lo: torch.Tensor | None, scale: float) -> torch.Tensor:
    """The same attention through ``torch.nn.functional.scaled_dot_product_attention`` (grouped-query form): causal
    flag when there is no document mask, else a boolean ``[B, 1, S, Sk]`` mask built from the per-row bounds."""

    B, S, Hq, D = q.shape
    Sk = k.shape[1]
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if lo is None:
        o = F.scaled_dot_product_attention(qt, kt, vt, is_causal=causal and S == Sk, scale=scale, enable_gqa=True)
        return o.transpose(1, 2)
    qi = torch.arange(S, device=q.device) + (Sk - S)
    ki = torch.arange(Sk, device=q.device)
    allowed = ki[None, None, None, :] >= lo.long()[:, None, :, None]
    if causal:
        allowed = allowed & (qi[None, None, :, None] >= ki[None, None, None, :])
    o = F.scaled_dot_product_attention(qt, kt, vt, attn_mask=allowed, scale=scale, enable_gqa=True)
    return o.transpose(1, 2)


class _AttentionBlockFn(torch.autograd.Function):
    """packed qkv -> QK-norm + RoPE -> flash attention, with one packed gradient buffer in backward."""

    @staticmethod
    def forward(ctx, qkv, wq, wk, positions, lo, hi, B, S, hq, hkv, D, eps, theta, rope, causal, scale):
        T = B * S
        qk = torch.empty(T, (hq + hkv) * D, dtype=qkv.dtype, device=qkv.device)
        rq = rk = None
        if wq is not None or rope:
            rq = native.qknorm_rope_fwd_qk(qkv, qk, wq, wk, positions, hq, hkv, D, eps, theta, rope)
            q4 = qk[:, : hq * D].view(B, S, hq, D)
            k4 = qk[:, hq * D:].view(B, S, hkv, D)
        else:
            q4 = qkv[:, : hq * D].view(B, S, hq, D)
            k4 = qkv[:, hq * D:(hq + hkv) * D].view(B, S, hkv, D)
        v4 = qkv[:, (hq + hkv) * D:].view(B, S, hkv, D)
        o, lse = native.attn_fwd(q4, k4, v4, causal=causal, lo=lo, scale=scale)
        ctx.save_for_backward(qkv, qk, o, lse, positions, lo, hi, rq, rk)
        ctx.params = (wq, wk)
        ctx.cfg = (B, S, hq, hkv, D, theta, rope, causal, scale)
        return o.view(B, S, hq * D)

    @staticmethod
    def backward(ctx, d_o):
        qkv, qk, o, lse, positions, lo, hi, rq, rk = ctx.saved_tensors
        wq, wk = ctx.params
        B, S, hq, hkv, D, theta, rope, causal, scale = ctx.cfg
        T = B * S
        transformed = rq is not None or rope
        if transformed:
            q4 = qk[:, : hq * D].view(B, S, hq, D)
            k4 = qk[:, hq * D:].view(B, S, hkv, D)
        else:
            q4 = qkv[:, : hq * D].view(B, S, hq, D)
            k4 = qkv[:, hq * D:(hq + hkv) * D].view(B, S, hkv, D)
        v4 = qkv[:, (hq + hkv) * D:].view(B, S, hkv, D)
        dqkv = torch.empty_like(qkv)
        outs = (dqkv[:, : hq * D].view(B, S, hq, D), dqkv[:, hq * D:(hq + hkv) * D].view(B, S, hkv, D),
                dqkv[:, (hq + hkv) * D:].view(B, S, hkv, D))
        d_o4 = d_o.reshape(B, S, hq, D)
        if not d_o4.is_contiguous():
            d_o4 = d_o4.contiguous()
        native.attn_bwd(q4, k4, v4, o, d_o4, lse, causal=causal, lo=lo, hi=hi, scale=scale, out=outs)
        if transformed:  # in place: every (token, head) vector is read and rewritten by one warp
            native.qknorm_rope_bwd_qk(qkv, dqkv, dqkv, wq, wk, positions, rq, None if wq is None else _main_grad(wq),
                                      None if wk is None else _main_grad(wk), hq, hkv, D, theta, rope)
        return (dqkv,) + (None,) * 15


def attention_block(qkv: torch.Tensor, wq, wk, positions: torch.Tensor, *, B: int, S: int, hq: int, hkv: int,
                    D: int, eps: float, theta: float, rope: bool, causal: bool = True,
                    lo: torch.Tensor | None = None, hi: torch.Tensor | None = None,
                    scale: float | None = None) -> torch.Tensor:
    """Packed projection ``[B*S, (hq + 2 hkv) * D]`` -> attention output ``[B, S, hq * D]``.

    QK-RMSNorm (when ``wq``/``wk`` are given) then interleaved RoPE (when ``rope``) then GQA attention.
    """

    if scale is None:
        scale = D ** -0.5
    if use_native(qkv) and D in (64, 128) and not (_ordered_sums_only() and wq is not None
                                                   and torch.is_grad_enabled()):
        if lo is not None and hi is None:
            hi = native.kv_visibility_upper_bound(lo)
        return _AttentionBlockFn.apply(qkv, wq, wk, positions, lo, hi, B, S, hq, hkv, D, eps, theta, rope, causal,
                                       scale)
    qk = qk_norm_rope(qkv, wq, wk, positions, hq, hkv, D, eps, theta, rope)
    q4 = qk[:, : hq * D].reshape(B, S, hq, D)
    k4 = qk[:, hq * D:].reshape(B, S, hkv, D)
    v4 = qkv[:, (hq + hkv) * D:].reshape(B, S, hkv, D)
    return attention(q4, k4, v4, causal=causal, lo=lo, hi=hi, scale=scale).reshape(B, S, hq * D)


# --------------------------------------------------------------------------------------------------
# SwiGLU / sigmoid gate
# --------------------------------------------------------------------------------------------------
class _SwigluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        gu = gu.contiguous()
        ctx.save_for_backward(gu)
        return native.swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, dh):
        (gu,) = ctx.saved_tensors
        return native.swiglu_bwd(gu, dh.contiguous())


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` over a fused ``[..., 2I]`` tensor whose first half is the gate."""

    if use_native(gu) and (gu.shape[-1] // 2) % 8 == 0:
        return _SwigluFn.apply(gu)
    inter = gu.shape[-1] // 2
    return F.silu(gu[..., :inter]) * gu[..., inter:]


class _SigmoidGateFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, gate):
        a, gate = a.contiguous(), gate.contiguous()
        ctx.save_for_backward(a, gate)
        return native.sigmoid_gate_fwd(a, gate)

    @staticmethod
    def backward(ctx, dout):
        a, gate = ctx.saved_tensors
        return native.sigmoid_gate_bwd(a, gate, dout.contiguous())


def sigmoid_gate(a: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    if use_native(a) and a.numel() % 8 == 0:
        return _SigmoidGateFn.apply(a, gate)
    return a * torch.sigmoid(gate)


# --------------------------------------------------------------------------------------------------
# embedding
# --------------------------------------------------------------------------------------------------
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, p, scale, like):
        table = compute_weight(p, like)
        ids32 = ids.to(torch.int32).contiguous()
        ctx.save_for_backward(ids32)
        ctx.p = p
        ctx.scale = scale
        return native.embedding_fwd(ids32, table, scale)

    @staticmethod
    def backward(ctx, dout):
        (ids32,) = ctx.saved_tensors
        if ctx.p.requires_grad:
            native.embedding_bwd(ids32, dout.contiguous(), _main_grad(ctx.p), ctx.scale)
        return None, None, None, None


def embedding(ids: torch.Tensor, p: torch.Tensor, scale: float = 1.0, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    if (p.is_cuda and dtype == torch.bfloat16 and not _FORCE_REFERENCE and p.shape[1] % 8 == 0
            and not (_ordered_sums_only() and p.requires_grad and torch.is_grad_enabled())):
        like = torch.empty(0, dtype=dtype, device=p.device)
        return _EmbeddingFn.apply(ids, p, scale, like)
    out = F.embedding(ids.long(), p).to(dtype)
    return out * scale if scale != 1.0 else out


# --------------------------------------------------------------------------------------------------
# lm_head + masked cross-entropy (+ z-loss), chunked over tokens so that logits never exist in full
# --------------------------------------------------------------------------------------------------
class _LmHeadCeFn(torch.autograd.Function):
    """Forward computes loss sums AND the gradients (dx saved, dW added to main_grad) chunk by chunk."""

    @staticmethod
    def forward(ctx, x, p, targets, mask, grad_scale, z_weight, chunk_tokens):
        w = compute_weight(p, x)
        T, H = x.shape
        V = w.shape[0]
        need_grad = bool(ctx.needs_input_grad[0] or ctx.needs_input_grad[1])  # grad mode is off inside forward
        dx = torch.empty_like(x) if need_grad else None
        loss_rows = torch.empty(T, dtype=torch.float32, device=x.device)
        z_rows = torch.empty(T, dtype=torch.float32, device=x.device)
        tgt = targets.to(torch.int32).contiguous()
        msk = mask.to(torch.uint8).contiguous()
        ld = (V + 7) // 8 * 8
        logits_buf = native.scratch("ce_logits", chunk_tokens * ld, torch.bfloat16, x.device)
        for t0 in range(0, T, chunk_tokens):
            t1 = min(t0 + chunk_tokens, T)
            n = t1 - t0
            logits = logits_buf[: n * ld].view(n, ld)[:, :V]
            native.gemm(x[t0:t1], w, trans_b=True, out=logits)
            loss, z, _ = native.ce_fwd_bwd(logits, tgt[t0:t1], msk[t0:t1], grad_scale, z_weight, write_grad=need_grad)
            loss_rows[t0:t1] = loss
            z_rows[t0:t1] = z
            if need_grad:
                native.gemm(logits, w, trans_b=False, out=dx[t0:t1])
                if p.requires_grad:
                    native.gemm(logits, x[t0:t1], trans_a=True, trans_b=False, out=_main_grad(p), accumulate=True)
        ctx.save_for_backward(dx)
        ce_sum, z_sum = loss_rows.sum(), z_rows.sum()
        ctx.mark_non_differentiable(z_sum)
        return ce_sum, z_sum

    @staticmethod
    def backward(ctx, g_loss, g_z):
        (dx,) = ctx.saved_tensors
        # gradients were formed with grad_scale already applied; the incoming factor is 1 in training
        return dx, None, None, None, None, None, None


def lm_head_cross_entropy(x: torch.Tensor, p: torch.Tensor, targets: torch.Tensor, mask: torch.Tensor, *,
                          grad_scale: float, z_weight: float = 0.0, chunk_tokens: int = 4096):
    """Masked CE over ``logits = x @ W^T`` (W ``[V, H]``).

    Returns ``(ce_sum, z_sum)`` where ``z_sum = sum(mask * logsumexp^2)``.  The training objective is
    ``grad_scale * (ce_sum + z_weight * z_sum)``: on the native path the gradient of exactly that objective
    is produced inside the forward pass, so callers must backpropagate through ``ce_sum`` with factor 1
    (use :func:`objective_from_sums`).
    """

    x2 = x.reshape(-1, x.shape[-1])
    t1 = targets.reshape(-1)
    m1 = mask.reshape(-1)
    if use_native(x2):
        return _LmHeadCeFn.apply(x2.contiguous(), p, t1, m1, grad_scale, z_weight, chunk_tokens)
    logits = F.linear(x2, p.to(x2.dtype)).float()
    lse = torch.logsumexp(logits, dim=-1)
    tl = logits.gather(1, t1.long()[:, None])[:, 0]
    mf = m1.float()
    return ((lse - tl) * mf).sum(), (lse.pow(2) * mf).sum()


class _VocabParallelCeFn(torch.autograd.Function):
    """Cross-entropy over a vocabulary that is split across ``group``: this rank holds rows ``[rank * Vl, (rank + 1)
    * Vl)`` of the lm_head and scores them for all tokens; the row maximum, the sum of exponentials and the target
    logit are reduced over the group (one MAX and one SUM reduction per token chunk).  Like :class:`_LmHeadCeFn` the
    forward also produces the gradients of ``grad_scale * (ce + z_weight * z)``: ``dx`` holds this rank's partial
    input gradient (the caller's gather of the activations sums the partials in its backward) and the weight
    gradient goes to ``main_grad`` (native path) or is returned (reference path)."""

    @staticmethod
    def forward(ctx, x, p, targets, mask, grad_scale, z_weight, group, chunk_tokens, native_path):
        import torch.distributed as dist

        w = compute_weight(p, x) if native_path else p.to(x.dtype)
        T, H = x.shape
        Vl = w.shape[0]
        first = dist.get_rank(group) * Vl
        need_grad = bool(ctx.needs_input_grad[0] or ctx.needs_input_grad[1])
        dx = torch.zeros_like(x) if need_grad else None
        dw = None if native_path or not need_grad else torch.zeros(w.shape, dtype=torch.float32, device=x.device)
        ce_sum = torch.zeros((), dtype=torch.float32, device=x.device)
        z_sum = torch.zeros((), dtype=torch.float32, device=x.device)
        for t0 in range(0, T, chunk_tokens):
            t1 = min(t0 + chunk_tokens, T)
            xc = x[t0:t1]
            if native_path:
                logits = native.gemm(xc, w, trans_b=True, out_dtype=torch.float32)
            else:
                logits = (xc @ w.t()).float()
            m = logits.max(dim=1).values
            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
            local = targets[t0:t1].long() - first
            mine = (local >= 0) & (local < Vl)
            picked = logits.gather(1, local.clamp(0, Vl - 1)[:, None])[:, 0] * mine
            packed = torch.stack([torch.exp(logits - m[:, None]).sum(dim=1), picked])
            dist.all_reduce(packed, group=group)
            lse = m + packed[0].log()
            mf = mask[t0:t1].float()
            ce_sum += ((lse - packed[1]) * mf).sum()
            z_sum += (lse.pow(2) * mf).sum()
            if need_grad:
                # d/dlogits of grad_scale * (ce + zw * lse^2) = grad_scale * mask * ((1 + 2 zw lse) softmax - onehot)
                probs = torch.exp(logits - lse[:, None])
                g = probs * ((1.0 + 2.0 * z_weight * lse) * mf * grad_scale)[:, None]
                rows = torch.nonzero(mine, as_tuple=True)[0]
                g[rows, local[rows]] -= (mf * grad_scale)[rows]
                g = g.to(x.dtype)
                if native_path:
                    native.gemm(g, w, trans_b=False, out=dx[t0:t1])
                    if p.requires_grad:
                        native.gemm(g, xc, trans_a=True, trans_b=False, out=_main_grad(p), accumulate=True)
                else:
                    dx[t0:t1] = g @ w
                    dw += (g.t() @ xc).float()
        ctx.save_for_backward(dx, dw)
        ctx.mark_non_differentiable(z_sum)
        return ce_sum, z_sum

    @staticmethod
    def backward(ctx, g_loss, g_z):
        dx, dw = ctx.saved_tensors
        return dx, (None if dw is None else dw.to(dx.dtype)), None, None, None, None, None, None, None


def vocab_parallel_cross_entropy(x: torch.Tensor, p: torch.Tensor, targets: torch.Tensor, mask: torch.Tensor, group, *,
                                 grad_scale: float, z_weight: float = 0.0, chunk_tokens: int = 4096):
    """Masked CE (and z-loss sum) with the lm_head ``p`` (``[V / n, H]``: this rank's rows) split over ``group``.

    ``x``: the activations of ALL tokens (the same on every rank of the group).  Returns ``(ce_sum, z_sum)``, the
    same on every rank; the gradient of ``grad_scale * (ce_sum + z_weight * z_sum)`` is formed inside the forward
    pass as in :func:`lm_head_cross_entropy`, so callers backpropagate through ``ce_sum`` with factor 1.
    Reference: src/jaxtitan/models/execution.py:209-219, src/jaxtitan/steps/eval.py:40-51."""

    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    return _VocabParallelCeFn.apply(x2, p, targets.reshape(-1), mask.reshape(-1), grad_scale, z_weight, group,
                                    chunk_tokens, use_native(x2))


def objective_from_sums(ce_sum: torch.Tensor, z_sum: torch.Tensor, *, grad_scale: float, z_weight: float,
                        native_path: bool) -> torch.Tensor:
    """The scalar to call ``backward()`` on so that both paths give ``d[grad_scale*(ce + zw*z)]``."""

    if native_path:
        return ce_sum  # gradient already scaled inside the fused op
    return grad_scale * (ce_sum + z_weight * z_sum)


def logits(x: torch.Tensor, p: torch.Tensor) -> torch.Tensor:
    """Plain lm_head projection (inference)."""

    return linear(x, p)


def softmax_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
