"""Matrix orthogonalisation used by Muon and Dion2: quintic Newton-Schulz and Polar Express.

Same iterations and constants as the reference (src/jaxtitan/optim/muon.py:18-25, 482-506;
optim/dion2.py:13-24, 151-169).  On CUDA bf16 every product is a tcgen05 GEMM from this package's kernel
library and no transposed copy is ever made: a tall matrix uses the right Gram ``X^T X`` through the
transposed-operand GEMM forms.  Rank-3 inputs are stacks of expert matrices (batched GEMM).
"""

from __future__ import annotations

import torch

from research_b200.ops import native

MUON_MOMENTUM = 0.95
MUON_NESTEROV = True
MUON_NS_STEPS = 5
MUON_NS_EPS = 1e-7
MUON_NS_COEFFICIENTS = (3.4445, -4.7750, 2.0315)
MUON_NS_PRECISION = "bfloat16"
MUON_RMS_MATCH_SCALE = 0.2

DION2_FRACTION = 0.25
DION2_EF_DECAY = 0.95
DION2_EPSILON = 1e-8
DION2_POLAR_EXPRESS_COEFFICIENTS = (
    (8.156554524902461, -22.48329292557795, 15.878769915207462),
    (4.042929935166739, -2.808917465908714, 0.5000178451051316),
    (3.8916678022926607, -2.772484153217685, 0.5060648178503393),
    (3.285753657755655, -2.3681294933425376, 0.46449024233003106),
    (2.3465413258596377, -1.7097828382687081, 0.42323551169305323),
)


def _native_ok(x: torch.Tensor) -> bool:
    from research_b200.ops import functional as Fn

    return (x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.shape[-2] % 8 == 0 and
            Fn.native_enabled())


def _iterate(x: torch.Tensor, coefficients) -> torch.Tensor:
    """``x <- a x + (b G + c G^2) x`` with the Gram on the short side; x: [..., m, n] bf16 or fp32."""

    tall = x.shape[-2] > x.shape[-1]
    if _native_ok(x):
        x = x.contiguous()
        for a, b, c in coefficients:
            if tall:
                gram = native.gemm(x, x, trans_a=True, trans_b=False)          # X^T X  [n, n]
            else:
                gram = native.gemm(x, x, trans_b=True)                          # X X^T  [m, m]
            gram2 = native.gemm(gram, gram, trans_b=True)                       # symmetric: G G^T = G^2
            poly = (b * gram.float() + c * gram2.float()).to(x.dtype)
            out = (a * x.float()).to(x.dtype)
            if tall:
                native.gemm(x, poly, trans_b=False, out=out, accumulate=True)  # + X P
            else:
                native.gemm(poly, x, trans_b=False, out=out, accumulate=True)  # + P X
            x = out
        return x
    for a, b, c in coefficients:
        if tall:
            gram = x.transpose(-1, -2) @ x
            x = a * x + x @ (b * gram + c * (gram @ gram))
        else:
            gram = x @ x.transpose(-1, -2)
            x = a * x + (b * gram + c * (gram @ gram)) @ x
    return x


def newton_schulz_stack_(x: torch.Tensor, coefficients=None) -> torch.Tensor:
    """Newton-Schulz on an already normalised bf16 stack ``[batch, m, n]`` with three batched tcgen05 GEMMs per step.

    Uses ``a X + (b G + c G^2) X = ((b I + c G) G + a I) X`` so that no step needs an accumulate pass:
    ``G = X X^T`` (or ``X^T X`` when tall), ``Q = (b I + c G) G``, ``X <- (Q + a I) X``.
    """

    coefficients = coefficients or (MUON_NS_COEFFICIENTS,) * MUON_NS_STEPS
    tall = x.shape[-2] > x.shape[-1]
    for a, b, c in coefficients:
        if tall:
            gram = native.gemm(x, x, trans_a=True, trans_b=False)
        else:
            gram = native.gemm(x, x, trans_b=True)
        lhs = native.affine_identity(gram, b, c)                  # b I + c G
        q = native.gemm(lhs, gram, trans_b=True)                  # G symmetric: (bI + cG) G^T = bG + cG^2
        native.affine_identity(q, a, 1.0, out=q)                  # + a I
        if tall:
            x = native.gemm(x, q, trans_b=True)                   # X Q   (Q symmetric)
        else:
            x = native.gemm(q, x, trans_b=False)                  # Q X
    return x


def zeropower_via_newton_schulz(value: torch.Tensor, *, precision: str = MUON_NS_PRECISION) -> torch.Tensor:
    """Approximate ``U V^T`` of ``value = U S V^T`` (rank 2, or rank 3 = one matrix per expert)."""

    if value.dim() not in (2, 3):
        raise ValueError(f"Muon Newton-Schulz expects rank-2 or expert-axis rank-3 arrays, got shape {tuple(value.shape)}")
    dtype = torch.bfloat16 if precision == "bfloat16" else torch.float32
    x = value.to(dtype)
    if x.dim() == 3:
        norm = torch.linalg.matrix_norm(x.float(), keepdim=True).to(dtype)
    else:
        norm = torch.linalg.matrix_norm(x.float()).to(dtype)
    x = x / torch.clamp(norm, min=MUON_NS_EPS)
    coeffs = (MUON_NS_COEFFICIENTS,) * MUON_NS_STEPS
    return _iterate(x, coeffs).to(value.dtype)


def polar_express(value: torch.Tensor, *, epsilon: float = DION2_EPSILON) -> torch.Tensor:
    if value.dim() != 2:
        raise ValueError(f"Polar Express expects rank-2 arrays, got shape {tuple(value.shape)}")
    x = value.to(torch.bfloat16)
    norm = torch.linalg.matrix_norm(x.float()).to(torch.bfloat16)
    x = x / (norm * 1.02 + epsilon)
    return _iterate(x, DION2_POLAR_EXPRESS_COEFFICIENTS).to(value.dtype)


def rms_match_scale(shape) -> float:
    m, n = shape[-2], shape[-1]
    return MUON_RMS_MATCH_SCALE * float(max(m, n)) ** 0.5


def select_dion2_slices(value: torch.Tensor, *, select_axis: int, fraction: float = DION2_FRACTION):
    """Top-``ceil(fraction * dim)`` rows (axis 0) or columns (axis 1) by L1 norm; returns (slices, indices)."""

    if value.dim() != 2:
        raise ValueError(f"Dion2 expects rank-2 arrays, got shape {tuple(value.shape)}")
    if select_axis not in (0, 1):
        raise ValueError(f"Dion2 select_axis must be 0 or 1, got {select_axis}")
    if not 0.0 < fraction <= 1.0:
        raise ValueError(f"Dion2 fraction must be in (0, 1], got {fraction}")
    import math

    k = max(1, math.ceil(fraction * value.shape[select_axis]))
    norms = value.float().abs().sum(dim=1 if select_axis == 0 else 0)
    indices = torch.topk(norms, k).indices
    selected = value.index_select(select_axis, indices)
    return selected, indices


def muon_policy_constants() -> dict:
    return {"momentum": MUON_MOMENTUM, "nesterov": MUON_NESTEROV, "newton_schulz_steps": MUON_NS_STEPS,
            "newton_schulz_eps": MUON_NS_EPS, "newton_schulz_coefficients": list(MUON_NS_COEFFICIENTS),
            "newton_schulz_precision": MUON_NS_PRECISION, "scale_mode": "match_rms_adamw",
            "rms_match_scale": MUON_RMS_MATCH_SCALE}


def dion2_policy_constants() -> dict:
    return {"fraction": DION2_FRACTION, "ef_decay": DION2_EF_DECAY, "epsilon": DION2_EPSILON,
            "adjust_lr": "spectral_norm", "orthogonalizer": "polar_express",
            "polar_express_coefficients": [list(c) for c in DION2_POLAR_EXPRESS_COEFFICIENTS]}
