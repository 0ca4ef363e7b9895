"""``run preflight``: prove a config can train before a run directory exists.

Loads the config, refuses if the run directory exists, builds data / mesh / model / optimizer exactly as training
does, runs ONE real optimizer step on the first batch and, when evals are configured, one validation pass, then
reports devices, mesh, data pipeline, first-batch provenance, model and optimizer policy, first-step loss / tokens
per second / MFU and the placement - writing nothing (reference: src/jaxtitan/runtime/preflight.py:58-307).
"""

from __future__ import annotations

import time
from pathlib import Path
from typing import Any

from research_b200.config import load_config, resolved_config_sha256
from research_b200.config.canonical import normalize
from research_b200.errors import ContractError
from research_b200.optim.build import optimizer_policy_summary
from research_b200.runtime.diagnostics import build_runtime_diagnostics
from research_b200.runtime.trainer import Trainer


def run_preflight(config_path: str | Path) -> dict[str, Any]:
    config_path = Path(config_path)
    spec = load_config(config_path)
    if spec.dirs.run_dir.exists():
        raise ContractError(f"run directory already exists: {spec.dirs.run_dir}")
    from research_b200.parallel.mesh import init_distributed

    init_distributed()
    trainer = Trainer(spec)
    spec = trainer.spec
    policy = optimizer_policy_summary(trainer.optimizer_build)
    pipeline = trainer.data.describe()
    runtime = build_runtime_diagnostics(spec, trainer, optimizer_policy=policy, data_pipeline=pipeline)
    batches = trainer.next_accumulated_batch()
    prov = trainer.last_provenance
    start = time.perf_counter()
    metrics = trainer.train_on(batches, diagnostics=True)
    step_sec = time.perf_counter() - start
    tokens = sum(p.target_tokens for p in prov)
    perf = runtime["performance"]
    tps = tokens / step_sec if step_sec > 0 else None
    mfu = None
    if tps and perf["peak_flops_total"]:
        mfu = 100.0 * perf["flops_per_token"] * tps / perf["peak_flops_total"]
    eval_report = None
    if spec.evals:
        ev = spec.evals[0]
        t0 = time.perf_counter()
        result = trainer.evaluate(ev.num_batches)
        eval_report = {"name": ev.name, "loss": result["loss"], "token_count": int(result["token_count"]),
                       "num_batches": result["num_batches"], "eval_sec": time.perf_counter() - t0}
    return normalize({
        "schema_version": 1, "status": "ok", "config_path": config_path.as_posix(), "run_id": spec.run_id,
        "run_dir": spec.dirs.run_dir.as_posix(), "resolved_config_sha256": resolved_config_sha256(spec),
        "devices": {"kind": runtime["runtime"]["device_kind"], "count": trainer.mesh.world_size,
                    "backend": trainer.device.type},
        "mesh": runtime["mesh"], "parallelism": runtime["parallelism"], "data_pipeline": pipeline,
        "first_batch": {"token_start": min(p.token_start for p in prov), "token_end": max(p.token_end for p in prov),
                        "examples": sum(p.examples for p in prov), "target_tokens": tokens,
                        "row_start_offsets": list(prov[0].row_start_offsets),
                        "row_doc_ids": None if prov[0].row_doc_ids is None else list(prov[0].row_doc_ids)},
        "model": runtime["model"], "optimizer": {"description": trainer.optimizer_build.description,
                                                 "backend_parameter_counts": policy["backend_parameter_counts"]},
        "first_step": {"loss": metrics.loss, "token_count": int(metrics.token_count), "grad_norm": metrics.grad_norm,
                       "param_norm": metrics.param_norm, "update_norm": metrics.update_norm, "lr": metrics.lr,
                       "step_sec": step_sec, "train_tokens_per_sec": tps, "mfu": mfu},
        "eval": eval_report, "compile": runtime["compile"], "sharding": runtime["sharding"],
        "kernels": runtime["kernels"], "performance": perf,
    })
