"""One optimizer step: gradient accumulation over microbatches, token-sum loss, z-loss, aux losses,
data-parallel gradient reduction, optimizer update, SMEBU bias update, metrics.

Loss semantics follow the reference step (src/jaxtitan/steps/train.py:98-283): the objective of a microbatch is
``ce_sum + z_weight * z_sum + aux * token_count`` and the accumulated gradient is divided by the **global**
masked-token count of the whole optimizer step (train.py:120, 204-205).  Here the division is folded into the
backward pass (``grad_scale = 1 / global_count``), which is known up front because every rank derives the
global batch from the same deterministic data pipeline.

Each microbatch's tokens are copied from pinned host memory on a side stream while the previous microbatch
computes; loss scalars stay on the device until the step's single device-to-host read.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import numpy as np
import torch
import torch.distributed as dist

from research_b200.config.specs import RunSpec
from research_b200.contracts import Batch, StepMetrics
from research_b200.models.build import ModelBuildResult
from research_b200.ops import functional as Fn
from research_b200.ops import native
from research_b200.optim.optimizer import Optimizer
from research_b200.parallel.mesh import MeshContext
from research_b200.parallel.sharding import ParamStore
from research_b200.steps.moe_balance import MoeBalanceState, apply_moe_balance_update, router_diagnostics


@dataclass
class DeviceBatch:
    input_ids: torch.Tensor
    target_ids: torch.Tensor
    loss_mask: torch.Tensor
    token_doc_ids: torch.Tensor | None
    local_token_count: float


def context_positions(seq_len: int, cp: int, cp_rank: int) -> np.ndarray:
    """Global sequence positions that context-parallel rank ``cp_rank`` works on.

    Zig-zag split: the sequence is cut into ``2 cp`` chunks and rank ``r`` takes chunks ``r`` and ``2 cp - 1 - r``,
    so that under a causal mask every rank attends to the same number of (query, key) pairs.  (The reference splits
    contiguously and leaves the balance to XLA's partitioner: mesh/sharding.py:165-167.)  Odd chunkings fall back to
    the contiguous split."""

    if cp == 1:
        return np.arange(seq_len)
    if seq_len % (2 * cp):
        seq = seq_len // cp
        return np.arange(cp_rank * seq, (cp_rank + 1) * seq)
    c = seq_len // (2 * cp)
    return np.concatenate([np.arange(cp_rank * c, (cp_rank + 1) * c),
                           np.arange((2 * cp - 1 - cp_rank) * c, (2 * cp - cp_rank) * c)])


def local_batch_slices(mesh: MeshContext, batch_rows: int, seq_len: int):
    """Rows of the global microbatch (a slice) and the sequence positions (a slice, or an index array under
    context parallelism) this rank works on.

    The batch is split over the ``data`` and ``fsdp`` axes (``data`` major), the sequence over ``cp``.
    """

    dp = mesh.size("data") * mesh.size("fsdp")
    dp_rank = mesh.coord("data") * mesh.size("fsdp") + mesh.coord("fsdp")
    rows = batch_rows // dp
    cp, cp_rank = mesh.size("cp"), mesh.coord("cp")
    cols = slice(0, seq_len) if cp == 1 else context_positions(seq_len, cp, cp_rank)
    return slice(dp_rank * rows, (dp_rank + 1) * rows), cols


class BatchStager:
    """Pinned host buffers + a copy stream: host->device copies of microbatch k+1 overlap compute of k."""

    def __init__(self, device: torch.device, bytes_counter: list[int]):
        self.device = device
        self.cuda = device.type == "cuda"
        self.stream = torch.cuda.Stream(device) if self.cuda else None
        self.pinned: dict[tuple, torch.Tensor] = {}
        self.bytes_counter = bytes_counter

    def _to_device(self, key: str, array: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
        host = torch.from_numpy(np.ascontiguousarray(array)).to(dtype)
        if not self.cuda:
            return host
        k = (key, tuple(host.shape), dtype)
        buf = self.pinned.get(k)
        if buf is None:
            buf = torch.empty(host.shape, dtype=dtype, pin_memory=True)
            self.pinned[k] = buf
        buf.copy_(host)
        self.bytes_counter[0] += buf.numel() * buf.element_size()
        return buf.to(self.device, non_blocking=True)

    def stage(self, batch: Batch, rows: slice, cols: slice, slot: int) -> DeviceBatch:
        ids = np.ascontiguousarray(np.asarray(batch.input_ids)[rows][:, cols])
        tgt = np.ascontiguousarray(np.asarray(batch.target_ids)[rows][:, cols])
        msk = np.ascontiguousarray(np.asarray(batch.loss_mask)[rows][:, cols])
        docs = None if batch.token_doc_ids is None else np.asarray(batch.token_doc_ids)[rows]
        ctx = torch.cuda.stream(self.stream) if self.cuda else _NullCtx()
        with ctx:
            out = DeviceBatch(
                input_ids=self._to_device(f"ids{slot}", ids, torch.int32),
                target_ids=self._to_device(f"tgt{slot}", tgt, torch.int32),
                loss_mask=self._to_device(f"msk{slot}", msk, torch.uint8),
                token_doc_ids=None if docs is None else self._to_device(f"doc{slot}", docs, torch.int32),
                local_token_count=float(msk.sum()),
            )
        return out

    def wait(self) -> None:
        if self.cuda:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)


class _NullCtx:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


class TrainStep:
    def __init__(self, spec: RunSpec, result: ModelBuildResult, store: ParamStore, optimizer: Optimizer,
                 mesh: MeshContext, moe_balance: MoeBalanceState | None = None):
        self.spec = spec
        self.result = result
        self.model = result.model
        self.store = store
        self.optimizer = optimizer
        self.mesh = mesh
        self.moe_balance = moe_balance
        self.device = store.device
        self.h2d_bytes = [0]
        self.d2h_bytes = [0]
        self.stager = BatchStager(self.device, self.h2d_bytes)
        self.z_weight = float(spec.training.loss.z_loss_weight)
        self.native = (self.device.type == "cuda" and store.compute_dtype == torch.bfloat16 and Fn.native_enabled())
        self.loss_axes = [a for a in ("data", "fsdp", "cp") if mesh.size(a) > 1]
        if result.execution.sp and not result.model.vocab_parallel:
            self.loss_axes.append("tp")       # token-parallel loss: every tensor-parallel rank scored other tokens

    # ------------------------------------------------------------------------------------------------
    def _microbatch(self, db: DeviceBatch, grad_scale: float, global_mb_tokens: float, dp_world: int):
        model, ex = self.model, self.result.execution
        h, aux_losses, stats = model.hidden_states(db.input_ids, db.token_doc_ids)
        targets, mask = db.target_ids, db.loss_mask
        head = self._head_weight()
        if model.vocab_parallel:
            # every tensor-parallel rank scores its slice of the vocabulary for all tokens; the loss sums come out
            # the same on every rank of the group and the gradient is formed inside the op on both paths
            h = ex.gather_sequence(h)
            ce_sum, z_sum = Fn.vocab_parallel_cross_entropy(h, head, targets, mask, ex.tp_group,
                                                            grad_scale=grad_scale, z_weight=self.z_weight)
            native_path = True
        else:
            if ex.sp:  # the final hidden states are sequence-sharded over tp: shard targets the same way
                n, r = ex.tp_size, ex.tp_rank
                targets = targets.chunk(n, dim=1)[r].contiguous()
                mask = mask.chunk(n, dim=1)[r].contiguous()
            ce_sum, z_sum = Fn.lm_head_cross_entropy(h, head, targets, mask, grad_scale=grad_scale,
                                                     z_weight=self.z_weight)
            native_path = Fn.use_native(h)
        objective = Fn.objective_from_sums(ce_sum, z_sum, grad_scale=grad_scale, z_weight=self.z_weight,
                                           native_path=native_path)
        aux_total = None
        for aux in aux_losses:
            term = aux.value.float() * aux.weight
            aux_total = term if aux_total is None else aux_total + term
        if aux_total is not None:
            objective = objective + aux_total * (global_mb_tokens / dp_world) * grad_scale
        objective.backward()
        return ce_sum.detach(), z_sum.detach(), (None if aux_total is None else aux_total.detach()), stats

    def _backward_hook(self, last_microbatch: bool):
        """What the model calls when the backward pass of layer ``i`` has been issued: start the reduction of that
        layer's gradients (last microbatch, native path) and, with weights sharded at rest, fetch layer ``i - 1``."""

        store = self.store
        reduce = last_microbatch and self.native
        if store.resident and not reduce:
            return None

        def hook(layer: int) -> None:
            if reduce:
                store.on_layer_backward(layer)
            if not store.resident and layer >= 1:
                store.acquire_layer(layer - 1, -1)

        return hook

    def _head_weight(self):
        return self.model.head_weight()

    def run(self, batches: list[Batch], *, diagnostics: bool = False) -> StepMetrics:
        """``batches``: the step's microbatches as **global** host batches (every rank passes the same ones)."""

        mesh = self.mesh
        B, S = batches[0].input_ids.shape
        rows, cols = local_batch_slices(mesh, B, S)
        # a pipeline that materialises only this rank's rows says how many targets the whole batch leaves unmasked
        global_counts = [float(np.asarray(b.loss_mask).sum()) if getattr(b, "mask_count", None) is None
                         else float(b.mask_count) for b in batches]
        global_count = max(sum(global_counts), 1.0)
        grad_scale = 1.0 / global_count
        dp_world = mesh.size("data") * mesh.size("fsdp") * mesh.size("cp")
        self.store.zero_grads()
        if self.device.type == "cuda":
            from research_b200.parallel.symmetric import align_ranks

            align_ranks()      # absorbs host skew between ranks before the first peer-memory kernel of the step
        staged = self.stager.stage(batches[0], rows, cols, 0)
        ce_sums, z_sums, aux_vals = [], [], []
        all_stats = []
        for k in range(len(batches)):
            self.stager.wait()
            current = staged
            if k + 1 < len(batches):
                staged = self.stager.stage(batches[k + 1], rows, cols, (k + 1) % 2)
            last = k + 1 == len(batches)
            if last and self.native:
                self.store.begin_backward_overlap()
            self.model.layer_backward_hook = self._backward_hook(last)
            ce, z, aux, stats = self._microbatch(current, grad_scale, global_counts[k], dp_world)
            ce_sums.append(ce)
            z_sums.append(z)
            aux_vals.append(aux)
            all_stats.append(stats)
        if not self.native or native.deterministic():   # deterministic mode sends a few operators through autograd
            self.store.collect_autograd_grads()
        self.store.reduce_gradients()
        opt = self.optimizer.step(diagnostics=diagnostics)
        # ---- metrics: one small device vector, one reduction, one device-to-host read ------------
        mb = len(batches)
        vec = [torch.stack(ce_sums).float(), torch.stack(z_sums).float()]
        has_aux = aux_vals[0] is not None
        if has_aux:
            vec.append(torch.stack(aux_vals).float())
        packed = torch.cat(vec)
        for axis in self.loss_axes:
            group = mesh.group(axis)
            if group is not None:
                dist.all_reduce(packed, group=group)
        extras = [opt["grad_norm"].reshape(1).float(), opt["clip_scale"].reshape(1).float()]
        n_groups = 0
        if diagnostics:
            extras += [opt["param_norm"].reshape(1).float(), opt["update_norm"].reshape(1).float()]
            n_groups = len(self.optimizer.group_templates)
            extras.append(opt["group_squares"].reshape(-1).float())
        router_payload = self._router_metrics(all_stats) if all_stats and all_stats[0] else {}
        router_keys = sorted(k for k, v in router_payload.items() if torch.is_tensor(v) and v.dim() == 0)
        extras += [router_payload[k].reshape(1).float() for k in router_keys]
        # the kernels' status word (a bounded wait that gave up) rides along: max over all ranks, checked every step
        status = None
        if self.device.type == "cuda":
            status = native.status_code_tensor(self.device).float()
            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                status = status.clone()
                dist.all_reduce(status, op=dist.ReduceOp.MAX)
            extras.append(status)
        flat = torch.cat([packed] + extras)
        host = flat.detach().cpu().tolist()
        self.d2h_bytes[0] += flat.numel() * 4
        if status is not None:
            native.raise_for_status_code(int(host.pop()), self.device)
        ce_host, z_host = host[:mb], host[mb:2 * mb]
        pos = 2 * mb
        aux_host = None
        if has_aux:
            n_aux_ranks = 1
            for axis in self.loss_axes:          # the ranks whose values the packed reduction added up
                n_aux_ranks *= mesh.size(axis)
            aux_host = [v / n_aux_ranks for v in host[pos:pos + mb]]
            pos += mb
        grad_norm, clip_scale = host[pos], host[pos + 1]
        pos += 2
        param_norm = update_norm = None
        group_squares = None
        if diagnostics:
            param_norm, update_norm = host[pos], host[pos + 1]
            pos += 2
            group_squares = host[pos:pos + 3 * n_groups]
            pos += 3 * n_groups
        router_host = {k: host[pos + i] for i, k in enumerate(router_keys)}
        metrics = StepMetrics(
            loss_sum=float(sum(ce_host)), token_count=float(sum(global_counts)), lr=opt["lr"], grad_norm=grad_norm,
            param_norm=param_norm, update_norm=update_norm, z_loss_sum=float(sum(z_host)),
            microbatch_loss_sums=[float(v) for v in ce_host], microbatch_token_counts=global_counts,
        )
        if aux_host is not None:
            weights = [c / global_count for c in global_counts]
            metrics.aux_loss = float(sum(a * w for a, w in zip(aux_host, weights)))
            metrics.moe_aux_loss = metrics.aux_loss
        metrics.router = router_host
        metrics.router_layers = router_payload.get("layers", [])
        metrics.smebu = {k: v for k, v in router_host.items() if k.startswith("smebu_")}
        if group_squares is not None:
            from research_b200.optim.diagnostics import groups_payload

            metrics.optimizer_groups = groups_payload(self.optimizer.group_templates, group_squares)
        metrics.router["clip_scale"] = clip_scale
        return metrics

    # ------------------------------------------------------------------------------------------------
    def _router_metrics(self, all_stats) -> dict[str, Any]:
        """Sum per-layer expert counts over microbatches and replicas; apply the SMEBU update."""

        layers: dict[int, list] = {}
        for stats in all_stats:
            for st in stats:
                layers.setdefault(st.layer_index, []).append(st)
        if not layers:
            return {}
        order = sorted(layers)
        counts = torch.stack([torch.stack([s.expert_counts for s in layers[i]]).sum(0) for i in order])
        importance = torch.stack([torch.stack([s.importance for s in layers[i]]).sum(0) for i in order])
        both = torch.stack([counts, importance])
        for axis in self.loss_axes:
            group = self.mesh.group(axis)
            if group is not None:
                dist.all_reduce(both, group=group)
        counts, importance = both[0], both[1]
        out = router_diagnostics(counts, importance)
        out.update(apply_moe_balance_update(self.moe_balance, counts))
        out["layers"] = [{"layer_index": i, "counts": counts[k], "importance": importance[k]}
                         for k, i in enumerate(order)]
        return out
