"""Where did the non-finite values come from?  Scans parameters and gradients leaf by leaf.

The training loop aborts when the loss or a global norm stops being finite; the event it writes names the
metric, not the culprit.  :func:`find_nonfinite_leaves` names the parameters whose values or gradients hold
NaN / Inf, with counts, using one device reduction per leaf and a single device-to-host read for all of them.

Reference: src/research/train_debug.py (non-finite leaf finder of the legacy training loop).
"""

from __future__ import annotations

from typing import Any

import torch


def _counts(t: torch.Tensor) -> torch.Tensor:
    f = t.detach().float().reshape(-1)
    return torch.stack([torch.isnan(f).sum(), torch.isinf(f).sum()])


@torch.no_grad()
def find_nonfinite_leaves(trainer, limit: int = 32) -> list[dict[str, Any]]:
    """``[{"name", "kind" ("param" | "grad"), "nan", "inf", "numel"}]`` for this rank's storage parameters, at
    most ``limit`` entries, parameters before gradients.  Sharded arenas are scanned as this rank holds them."""

    names, kinds, tensors = [], [], []
    for e in trainer.store.entries:
        names.append(e.name)
        kinds.append("param")
        tensors.append(e.param.data)
        grad = getattr(e.param, "main_grad", None)
        if grad is None:
            grad = e.param.grad
        if grad is not None:
            names.append(e.name)
            kinds.append("grad")
            tensors.append(grad)
    if not tensors:
        return []
    table = torch.stack([_counts(t) for t in tensors]).cpu().tolist()        # one read for every leaf
    found = [{"name": n, "kind": k, "nan": int(c[0]), "inf": int(c[1]), "numel": int(t.numel())}
             for n, k, t, c in zip(names, kinds, tensors, table) if c[0] or c[1]]
    found.sort(key=lambda d: d["kind"] != "param")
    return found[:limit]
