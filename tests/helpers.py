"""Shared builders for the CPU tests: tiny configs, synthetic datasets, multi-process gloo launches."""

from __future__ import annotations

import os
import socket
import tempfile
import traceback
from pathlib import Path

import numpy as np
import torch


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def tiny_dataset(root: Path, *, vocab: int = 256, documents: int = 300, mean: float = 120.0, seed: int = 0) -> Path:
    from research_b200.data import generate_synthetic_dataset

    return generate_synthetic_dataset(root / "ds", seed=seed, num_documents=documents, mean_length=mean, min_length=8,
                                      max_length=600, vocab_size=vocab, eos_id=vocab - 1, val_fraction=0.1)


def tiny_raw_config(manifest: Path, *, kind: str = "decoder", optimizer: str = "adamw", mesh=None, parallelism=None,
                    seq_len: int = 32, batch: int = 4, accum: int = 1, steps: int = 4, run_id: str = "tiny",
                    output_dir: str = "runs", order: str = "document_buffer", extra_model=None, evals: bool = False,
                    checkpoint_every: int = 1000, clip: float | None = 1.0) -> dict:
    model = dict(name="decoder", variant="tiny", vocab_size=256, hidden_size=64, intermediate_size=128, num_layers=2,
                 num_heads=4, n_kv_heads=2, max_seq_len=max(seq_len, 64), rope_theta=10000.0, compute_dtype="float32",
                 attention_doc_mask=True)
    if kind == "trinity":
        model.update(name="trinity", trinity=dict(
            initial_dense_layers=1, local_window=8, local_layers_per_global=1,
            moe=dict(num_experts=4, top_k=2, expert_intermediate_size=32, num_shared_experts=1,
                     balance=dict(name="smebu"))))
    if extra_model:
        model.update(extra_model)
    data = dict(train_manifest=str(manifest), order=order)
    if order == "document_buffer":
        data.update(shuffle_seed=1, document_buffer_size=8, document_refill_size=8)
    elif order == "shuffle":
        data.update(shuffle_seed=1)
    opt = dict(name=optimizer, weight_decay=0.01, schedule=dict(peak_lr=3e-3, name="constant", warmup_steps=2))
    if clip is not None:
        opt["grad_clip_norm"] = clip
    raw = dict(
        run=dict(id=run_id, seed=0, output_dir=output_dir), model=model, optimizer=opt, data=data,
        training=dict(seq_len=seq_len, global_batch_size=batch, target_tokens=seq_len * batch * accum * steps,
                      precision="fp32", gradient_accumulation_steps=accum, log_every_steps=1,
                      checkpoint_every_steps=checkpoint_every))
    if mesh:
        raw["mesh"] = dict(axis_names=list(mesh), axis_sizes=list(mesh.values()))
    if parallelism:
        raw["parallelism"] = parallelism
    if evals:
        raw["evals"] = [dict(name="validation", every_steps=2, num_batches=2)]
    return raw


def write_toml(raw: dict, path: Path) -> Path:
    def fmt(v):
        if isinstance(v, bool):
            return "true" if v else "false"
        if isinstance(v, str):
            return '"' + v.replace("\\", "\\\\") + '"'
        if isinstance(v, (list, tuple)):
            return "[" + ", ".join(fmt(x) for x in v) + "]"
        return repr(v)

    lines: list[str] = []

    def emit(table: dict, prefix: str):
        scalars = {k: v for k, v in table.items() if not isinstance(v, dict) and not (
            isinstance(v, list) and v and isinstance(v[0], dict))}
        if prefix:
            lines.append(f"[{prefix}]")
        for k, v in scalars.items():
            if v is not None:
                lines.append(f"{k} = {fmt(v)}")
        lines.append("")
        for k, v in table.items():
            if isinstance(v, dict):
                emit(v, f"{prefix}.{k}" if prefix else k)
            elif isinstance(v, list) and v and isinstance(v[0], dict):
                for item in v:
                    lines.append(f"[[{prefix + '.' if prefix else ''}{k}]]")
                    for kk, vv in item.items():
                        lines.append(f"{kk} = {fmt(vv)}")
                    lines.append("")

    emit(raw, "")
    path.write_text("\n".join(lines))
    return path


GLOO_COLLECTIVE_TIMEOUT_S = 180
GLOO_RUN_DEADLINE_S = 420
GLOO_HANG_DUMP_S = 150


def _worker(rank: int, world: int, port: int, fn, args, out_dir: str):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(world),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      RESEARCH_B200_GROUP_TIMEOUT_S=str(GLOO_COLLECTIVE_TIMEOUT_S))
    torch.set_num_threads(1)
    # a rank that is still running shortly before the deadline writes the stack of every thread next to its result
    import faulthandler

    hang_file = open(os.path.join(out_dir, f"rank{rank}.hang"), "w")
    faulthandler.dump_traceback_later(GLOO_HANG_DUMP_S, file=hang_file, exit=False)
    try:
        import datetime

        import torch.distributed as dist

        # a short collective timeout: a rank that waits for a peer that never comes fails in minutes, not in half an hour
        dist.init_process_group("gloo", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=GLOO_COLLECTIVE_TIMEOUT_S))
        result = fn(rank, world, *args)
        torch.save(result, os.path.join(out_dir, f"rank{rank}.pt"))
        dist.barrier()
        dist.destroy_process_group()
        faulthandler.cancel_dump_traceback_later()
    except Exception:
        with open(os.path.join(out_dir, f"rank{rank}.err"), "w") as handle:
            handle.write(traceback.format_exc())
        raise


def _run_gloo_once(world: int, fn, args, hash_seeds=None):
    import time

    import torch.multiprocessing as mp

    out_dir = tempfile.mkdtemp(prefix="gloo_")
    port = free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, args, out_dir)) for r in range(world)]
    saved_seed = os.environ.get("PYTHONHASHSEED")
    try:
        for r, p in enumerate(procs):
            if hash_seeds is not None:
                os.environ["PYTHONHASHSEED"] = str(hash_seeds[r])     # read by the child interpreter when it starts
            p.start()
    finally:
        if hash_seeds is not None:
            if saved_seed is None:
                os.environ.pop("PYTHONHASHSEED", None)
            else:
                os.environ["PYTHONHASHSEED"] = saved_seed
    deadline = time.monotonic() + GLOO_RUN_DEADLINE_S
    for p in procs:
        p.join(timeout=max(deadline - time.monotonic(), 0.0))
    stuck = [r for r, p in enumerate(procs) if p.is_alive()]
    for r in stuck:
        procs[r].terminate()                      # our own children, by handle
        procs[r].join(timeout=10)
    errors = []
    for r, p in enumerate(procs):
        err = Path(out_dir) / f"rank{r}.err"
        if err.exists():
            errors.append(f"rank {r}:\n{err.read_text()}")
        elif r in stuck:
            hang = Path(out_dir) / f"rank{r}.hang"
            stacks = hang.read_text() if hang.exists() else ""
            errors.append(f"rank {r} was still running after {GLOO_RUN_DEADLINE_S} s\n{stacks}")
        elif p.exitcode != 0:
            errors.append(f"rank {r} exited with code {p.exitcode}")
    if errors:
        _keep_hang_stacks(out_dir, world, fn)
        return None, errors, bool(stuck) or all("Timed out" in e or "timed out" in e for e in errors)
    return [torch.load(os.path.join(out_dir, f"rank{r}.pt"), weights_only=False) for r in range(world)], [], False


def _keep_hang_stacks(out_dir: str, world: int, fn) -> None:
    """Copy the stack dumps of a failed run into the temporary directory, where they outlive a retry that passes."""

    import time

    stacks = []
    for r in range(world):
        hang = Path(out_dir) / f"rank{r}.hang"
        if hang.exists() and hang.stat().st_size:
            stacks.append(f"==== rank {r}\n{hang.read_text()}")
    if stacks:
        keep = Path(tempfile.gettempdir()) / "research_b200_gloo_hangs"
        keep.mkdir(exist_ok=True)
        (keep / f"{int(time.time())}_{getattr(fn, '__name__', 'fn')}_{world}.txt").write_text("\n".join(stacks))


def run_gloo(world: int, fn, *args, hash_seeds=None):
    """Run ``fn(rank, world, *args)`` in ``world`` CPU processes over gloo; returns the per-rank results.
    ``hash_seeds`` gives every rank its own string-hash seed (the order in which a process iterates a set of strings).

    A run in which the ranks only timed out on one another (no rank raised anything else) is tried once more: on a
    loaded host the gloo rendezvous of a fresh group occasionally loses a connection."""

    results, errors, only_timeouts = _run_gloo_once(world, fn, args, hash_seeds)
    if errors and only_timeouts and hash_seeds is None:
        results, errors, _ = _run_gloo_once(world, fn, args)
    if errors:
        raise AssertionError("\n".join(errors))
    return results


def train_and_collect(rank: int, world: int, raw: dict, steps: int):
    """Build a trainer from a raw config mapping, run ``steps`` optimizer steps, return losses and logical params."""

    from research_b200.config import run_spec_from_mapping
    from research_b200.runtime.state_io import collect_state_tensors
    from research_b200.runtime.trainer import Trainer

    spec = run_spec_from_mapping(raw)
    trainer = Trainer(spec, device="cpu")
    losses, counts, norms = [], [], []
    for _ in range(steps):
        m = trainer.train_step(diagnostics=True)
        losses.append(m.loss_sum)
        counts.append(m.token_count)
        norms.append(m.grad_norm)
    tensors = collect_state_tensors(trainer)
    model = {k: torch.from_numpy(np.array(v)) for k, v in tensors.items() if k.startswith("model.")}
    return {"loss_sum": losses, "token_count": counts, "grad_norm": norms, "model": model}
