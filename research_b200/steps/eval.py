"""Masked cross-entropy evaluation (reference: src/jaxtitan/steps/eval.py:27-105: fp32 log-softmax, sum / count)."""

from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from research_b200.contracts import Batch, EvalMetrics
from research_b200.ops import functional as Fn
from research_b200.steps.train import BatchStager, local_batch_slices


def causal_lm_loss(logits: torch.Tensor, targets: torch.Tensor, mask: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Sum of masked token losses and the masked token count, from full logits."""

    logp = torch.log_softmax(logits.float(), dim=-1)
    tok = -logp.gather(-1, targets.long().unsqueeze(-1)).squeeze(-1)
    m = mask.float()
    return (tok * m).sum(), m.sum()


class EvalStep:
    def __init__(self, result, store, mesh):
        self.result, self.store, self.mesh = result, store, mesh
        self.model = result.model
        self.device = store.device
        self.stager = BatchStager(self.device, [0])
        self.loss_axes = [a for a in ("data", "fsdp", "cp") if mesh.size(a) > 1]
        if result.execution.sp and not result.model.vocab_parallel:
            self.loss_axes.append("tp")

    @torch.no_grad()
    def run(self, batch: Batch) -> EvalMetrics:
        B, S = batch.input_ids.shape
        rows, cols = local_batch_slices(self.mesh, B, S)
        db = self.stager.stage(batch, rows, cols, 0)
        self.stager.wait()
        h, _, _ = self.model.hidden_states(db.input_ids, db.token_doc_ids)
        targets, mask = db.target_ids, db.loss_mask
        ex = self.result.execution
        if self.model.vocab_parallel:
            ce_sum, _ = Fn.vocab_parallel_cross_entropy(ex.gather_sequence(h), self.model.head_weight(), targets, mask,
                                                        ex.tp_group, grad_scale=1.0, z_weight=0.0)
        else:
            if ex.sp:
                targets = targets.chunk(ex.tp_size, dim=1)[ex.tp_rank].contiguous()
                mask = mask.chunk(ex.tp_size, dim=1)[ex.tp_rank].contiguous()
            ce_sum, _ = Fn.lm_head_cross_entropy(h, self.model.head_weight(), targets, mask, grad_scale=1.0,
                                                 z_weight=0.0)
        total = ce_sum.detach().float().reshape(1)
        for axis in self.loss_axes:
            group = self.mesh.group(axis)
            if group is not None:
                dist.all_reduce(total, group=group)
        return EvalMetrics(loss_sum=float(total.item()), token_count=float(np.asarray(batch.loss_mask).sum()))
