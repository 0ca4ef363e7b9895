"""The ``jaxtitan`` command line (same grammar as the reference: src/jaxtitan/cli.py:16-148).

``config check``, ``data prepare|check|inspect``, ``kernels list|check|compile|bench``, ``profile analyze|bench``,
``run init|preflight|train [--resume] [--overwrite]|inspect``, ``eval checkpoint``, ``sample checkpoint``; ``--json``
prints canonical JSON; a :class:`JaxtitanError` becomes ``error: ...`` on stderr and exit code 2.
"""

from __future__ import annotations

import argparse
import json
import shutil
import sys
import time
from pathlib import Path
from typing import Any

from research_b200 import __version__
from research_b200.config import load_config, run_spec_to_json
from research_b200.config.canonical import canonical_json
from research_b200.errors import ContractError, JaxtitanError


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="jaxtitan", description="Blackwell-native LM training contracts and tools.")
    parser.add_argument("--version", action="version", version=f"jaxtitan {__version__} (research_b200)")
    commands = parser.add_subparsers(dest="command")

    config = commands.add_parser("config", help="Inspect and validate TOML configs.").add_subparsers(
        dest="config_command", required=True)
    p = config.add_parser("check", help="Validate a TOML config against the run contract.")
    p.add_argument("path")
    p.add_argument("--json", action="store_true")

    data = commands.add_parser("data", help="Prepare, validate and inspect prepared data.").add_subparsers(
        dest="data_command", required=True)
    p = data.add_parser("prepare", help="Prepare a text dataset for training.")
    p.add_argument("path")
    p.add_argument("--overwrite", action="store_true")
    p.add_argument("--json", action="store_true")
    p = data.add_parser("check", help="Validate a prepared-token manifest.")
    p.add_argument("path")
    p.add_argument("--tokenizer", required=True)
    p.add_argument("--verify-checksums", action="store_true")
    p.add_argument("--json", action="store_true")
    p = data.add_parser("inspect", help="Inspect a prepared-token manifest.")
    p.add_argument("path")
    p.add_argument("--tokenizer")
    p.add_argument("--verify-checksums", action="store_true")
    p.add_argument("--seq-len", type=int)
    p.add_argument("--json", action="store_true")
    p = data.add_parser("synth", help="Generate a seed-defined synthetic prepared dataset.")
    p.add_argument("out_dir")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--documents", type=int, default=2000)
    p.add_argument("--mean-length", type=float, default=300.0)
    p.add_argument("--min-length", type=int, default=16)
    p.add_argument("--max-length", type=int, default=2048)
    p.add_argument("--vocab-size", type=int, default=50257)
    p.add_argument("--eos-id", type=int, default=50256)
    p.add_argument("--val-fraction", type=float, default=0.05)
    p.add_argument("--overwrite", action="store_true")
    p.add_argument("--json", action="store_true")

    kernels = commands.add_parser("kernels", help="Inspect and build the sm_100a kernel library.").add_subparsers(
        dest="kernels_command", required=True)
    p = kernels.add_parser("list")
    p.add_argument("--json", action="store_true")
    p = kernels.add_parser("check")
    p.add_argument("path")
    p.add_argument("--cache-dir")
    p.add_argument("--json", action="store_true")
    p = kernels.add_parser("compile")
    p.add_argument("path")
    p.add_argument("--arch")
    p.add_argument("--cache-dir")
    p.add_argument("--json", action="store_true")
    p = kernels.add_parser("bench")
    p.add_argument("op", choices=["rmsnorm", "gemm", "attention"])
    p.add_argument("path")
    p.add_argument("--cache-dir")
    p.add_argument("--rows", default="1,4,17,64,256")
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--json", action="store_true")

    profile = commands.add_parser("profile", help="Analyze and benchmark performance paths.").add_subparsers(
        dest="profile_command", required=True)
    p = profile.add_parser("analyze")
    p.add_argument("root")
    p.add_argument("--warmup-steps", type=int, default=2)
    p.add_argument("--json", action="store_true")
    p = profile.add_parser("bench")
    p.add_argument("component", choices=["moe", "muon"])
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--artifact-dir")
    p.add_argument("--trace", action="store_true")
    p.add_argument("--json", action="store_true")

    run = commands.add_parser("run", help="Create, train and inspect local runs.").add_subparsers(
        dest="run_command", required=True)
    p = run.add_parser("init")
    p.add_argument("path")
    p = run.add_parser("preflight")
    p.add_argument("path")
    p.add_argument("--json", action="store_true")
    p = run.add_parser("train")
    p.add_argument("path")
    p.add_argument("--resume", action="store_true")
    p.add_argument("--overwrite", action="store_true")
    p = run.add_parser("inspect")
    p.add_argument("run_dir")
    p.add_argument("--json", action="store_true")

    ev = commands.add_parser("eval", help="Run deterministic evals over local artifacts.").add_subparsers(
        dest="eval_command", required=True)
    p = ev.add_parser("checkpoint")
    p.add_argument("run_dir")
    p.add_argument("--checkpoint", required=True)
    p.add_argument("--json", action="store_true")

    sample = commands.add_parser("sample", help="Generate token samples from local artifacts.").add_subparsers(
        dest="sample_command", required=True)
    p = sample.add_parser("checkpoint")
    p.add_argument("run_dir")
    p.add_argument("--checkpoint", required=True)
    p.add_argument("--prompt-ids", required=True)
    p.add_argument("--max-new-tokens", required=True, type=int)
    p.add_argument("--temperature", type=float, default=1.0)
    p.add_argument("--top-k", type=int, default=None)
    p.add_argument("--json", action="store_true")
    return parser


# ---- formatting helpers (console formats: reference cli.py:391-517) ------------------------------------
def _fmt_int(v) -> str:
    return "n/a" if v is None else f"{int(v):,}"


def _fmt_metric(v) -> str:
    return "n/a" if v is None else f"{float(v):.4f}"


def _fmt_number(v) -> str:
    return "n/a" if v is None else f"{float(v):.3g}"


def _fmt_percent(v) -> str:
    return "n/a" if v is None else f"{float(v):.2f}%"


def _fmt_tps(v) -> str:
    return "n/a" if v is None else f"{float(v):,.0f}"


def _fmt_count(n) -> str:
    n = float(n)
    for unit, div in (("B", 1e9), ("M", 1e6), ("K", 1e3)):
        if n >= div:
            return f"{n / div:.1f}{unit}"
    return str(int(n))


def _fmt_runtime(sec: float) -> str:
    m, s = divmod(int(sec), 60)
    h, m = divmod(m, 60)
    return f"{h:d}:{m:02d}:{s:02d}"


def _is_rank0() -> bool:
    import os

    return int(os.environ.get("RANK", "0")) == 0


def training_progress_printer():
    state: dict[str, Any] = {}

    def emit(event: str, payload: dict[str, Any]) -> None:
        if not _is_rank0():
            return
        if event == "start":
            spec = payload["spec"]
            state["t0"] = time.perf_counter()
            print("=========================")
            print("JAX TITAN TRAINING")
            print("=========================")
            print(f"run: {spec.run_id}")
            print(f"config: {Path(payload['config_path']).as_posix()}")
            print(f"resume: {str(payload['resume']).lower()}")
            print("initializing runtime...")
        elif event == "initialized":
            spec, d = payload["spec"], payload["diagnostics"]
            mesh, model, data, rt = d["mesh"], d["model"], d["data_pipeline"] or {}, d["runtime"]
            print("")
            print("config:")
            print(f"  model   | {spec.model.name}/{spec.model.variant} | params {_fmt_count(model['parameters'])} | "
                  f"seq {spec.training.seq_len} | dtype {spec.model.compute_dtype}/{spec.model.param_dtype} | "
                  f"remat {spec.model.remat}")
            print(f"  train   | target {_fmt_int(spec.training.target_tokens)} | batch {spec.training.global_batch_size} "
                  f"x accum {spec.training.gradient_accumulation_steps} = {mesh['effective_global_batch_size']} | "
                  f"tokens/step {_fmt_int(mesh['effective_tokens_per_step'])}")
            print(f"  optim   | {spec.optimizer.name} | schedule {spec.optimizer.schedule.name} | "
                  f"peak_lr {_fmt_number(spec.optimizer.schedule.peak_lr)}")
            print(f"  data    | {data.get('backend')} | order {data.get('order')} | docs "
                  f"{'yes' if data.get('document_aware') else 'no'} | records {_fmt_int(data.get('num_records'))} | "
                  f"{data.get('manifest_path')}")
            axes = ",".join(f"{n}={s}" for n, s in zip(mesh["axis_names"], mesh["axis_sizes"]))
            print(f"  mesh    | {rt['backend']} | devices {rt['selected_device_count']} | axes {axes}")
            print(f"  run_dir | {payload['run_dir']}")
            print("-------------------------")
        elif event == "resumed":
            print(f"resumed: checkpoint_step={payload['checkpoint_step']} step={payload['step']} "
                  f"tokens={_fmt_int(payload['tokens_seen'])} path={payload['checkpoint_path']}")
        elif event == "compile_start":
            if payload["phase"] == "train":
                print(f"step: {0:<6} | first train step (kernel library load)...")
        elif event == "train":
            row = payload["row"]
            total = time.perf_counter() - float(state.get("t0", time.perf_counter()))
            print(f"step: {row['step']:<6} | loss: {_fmt_metric(row['loss']):>9} | grad_norm: "
                  f"{_fmt_metric(row.get('grad_norm')):>9} | mfu: {_fmt_percent(row.get('mfu')):>7} | lr: "
                  f"{_fmt_number(row['lr']):>9} | tps: {_fmt_tps(row.get('train_tokens_per_sec')):>9} | total_time: "
                  f"{_fmt_runtime(total):>9}")
        elif event == "eval":
            row = payload["row"]
            print(f"eval step {row['step']}: loss={_fmt_metric(row['loss'])} tokens={_fmt_int(row['token_count'])} "
                  f"batches={row['num_batches']} tps={_fmt_metric(row.get('eval_tokens_per_sec'))} "
                  f"sec={_fmt_metric(row.get('eval_sec'))}")
        elif event == "checkpoint":
            ev = payload.get("eval_loss")
            tail = "" if ev is None else f" eval_loss={_fmt_metric(ev)}"
            print(f"checkpoint step {payload['step']}: {payload['checkpoint_path']} reason={payload['reason']} "
                  f"sec={_fmt_metric(payload['checkpoint_sec'])}{tail}")
        elif event == "failed":
            row = payload.get("row", {})
            groups = ", ".join(payload.get("optimizer_nonfinite_groups") or [])
            print(f"failed at step {row.get('step')}: non-finite optimizer groups: {groups}")
        elif event == "completed":
            s = payload["summary"]
            tail = "" if s.final_eval_loss is None else f" final_eval={_fmt_metric(s.final_eval_loss)}"
            print("-------------------------")
            print(f"completed: step={s.steps} tokens={_fmt_int(s.tokens_seen)}/{_fmt_int(s.target_tokens)} "
                  f"loss={_fmt_metric(s.final_loss)}{tail} steady_tps={_fmt_metric(s.steady_train_tokens_per_sec)} "
                  f"mfu={_fmt_percent(s.final_mfu)}")
            print(f"run_dir: {s.run_dir}")

    return emit


def _prepare_fresh_train_run(path: str, overwrite: bool) -> None:
    run_dir = load_config(path).dirs.run_dir
    if not run_dir.exists() or not _is_rank0():
        return
    if overwrite:
        shutil.rmtree(run_dir)
        return
    if not sys.stdin.isatty():
        raise ContractError(f"run directory already exists: {run_dir}; rerun with --overwrite to replace it")
    print(f"run directory already exists: {run_dir}", file=sys.stderr)
    if input("Overwrite this run directory? [y/N] ").strip().lower() not in ("y", "yes"):
        raise ContractError(f"run directory already exists: {run_dir}")
    shutil.rmtree(run_dir)


def _print_json(payload: Any) -> None:
    print(canonical_json(payload))


def _dispatch(args: argparse.Namespace) -> int:
    if args.command == "config":
        spec = load_config(args.path)
        print(run_spec_to_json(spec) if args.json else f"ok: {args.path} (run {spec.run_id})")
    elif args.command == "data":
        return _data(args)
    elif args.command == "kernels":
        return _kernels(args)
    elif args.command == "profile":
        return _profile(args)
    elif args.command == "run":
        if args.run_command == "init":
            from research_b200.services.artifacts import initialize_run

            manifest = initialize_run(args.path)
            print(f"initialized run {manifest.run_id} at {manifest.run_dir}")
        elif args.run_command == "preflight":
            from research_b200.runtime.preflight import (format_preflight_report, preflight_report_to_json,
                                                         run_preflight)

            report = run_preflight(args.path)
            if _is_rank0():
                print(preflight_report_to_json(report) if args.json else format_preflight_report(report))
        elif args.run_command == "train":
            from research_b200.runtime.training import run_training

            if not args.resume:
                _prepare_fresh_train_run(args.path, args.overwrite)
            run_training(args.path, resume=args.resume, progress=training_progress_printer())
        elif args.run_command == "inspect":
            from research_b200.runtime.inspect import format_run_inspection, inspect_run, run_inspection_to_json

            report = inspect_run(args.run_dir)
            print(run_inspection_to_json(report) if args.json else format_run_inspection(report))
    elif args.command == "eval":
        from research_b200.runtime.checkpoint_eval import evaluate_checkpoint

        payload = evaluate_checkpoint(args.run_dir, args.checkpoint)
        if _is_rank0():
            if args.json:
                _print_json(payload)
            else:
                from research_b200.runtime.checkpoint_eval import format_checkpoint_eval

                print(format_checkpoint_eval(payload))
    elif args.command == "sample":
        from research_b200.runtime.sampling import sample_checkpoint

        row = sample_checkpoint(args.run_dir, args.checkpoint, prompt_ids=args.prompt_ids,
                                max_new_tokens=args.max_new_tokens, temperature=args.temperature, top_k=args.top_k)
        if _is_rank0():
            if args.json:
                _print_json(row)
            else:
                from research_b200.runtime.sampling import format_checkpoint_sample

                print(format_checkpoint_sample(row))
    else:
        build_parser().print_help()
    return 0


def _data(args: argparse.Namespace) -> int:
    if args.data_command == "prepare":
        from research_b200.data.prepare import prepare_dataset

        summary = prepare_dataset(args.path, overwrite=args.overwrite)
        print(canonical_json(summary) if args.json else f"prepared {summary['num_tokens']:,} tokens at {summary['manifest_path']}")
    elif args.data_command == "check":
        from research_b200.data.manifest import prepared_dataset_manifest_to_json, validate_dataset_manifest

        manifest = validate_dataset_manifest(args.path, tokenizer_id=args.tokenizer, verify_checksums=args.verify_checksums)
        print(prepared_dataset_manifest_to_json(manifest) if args.json else
              f"ok: {args.path} ({manifest.num_tokens:,} tokens, {manifest.shard_count} shards)")
    elif args.data_command == "inspect":
        from research_b200.data.inspect import inspect_dataset, format_inspection

        report = inspect_dataset(args.path, tokenizer_id=args.tokenizer, verify_checksums=args.verify_checksums,
                                 seq_len=args.seq_len)
        print(canonical_json(report) if args.json else format_inspection(report))
    elif args.data_command == "synth":
        from research_b200.data.synthetic import generate_synthetic_dataset

        path = generate_synthetic_dataset(args.out_dir, seed=args.seed, num_documents=args.documents,
                                          mean_length=args.mean_length, min_length=args.min_length,
                                          max_length=args.max_length, vocab_size=args.vocab_size, eos_id=args.eos_id,
                                          val_fraction=args.val_fraction, overwrite=args.overwrite)
        print(canonical_json({"manifest_path": path.as_posix()}) if args.json else f"wrote {path}")
    return 0


def _kernels(args: argparse.Namespace) -> int:
    from research_b200.kernels import registry

    if args.kernels_command == "list":
        print(canonical_json(registry.kernel_registry_payload()) if args.json else registry.format_kernel_registry())
    elif args.kernels_command == "check":
        plan = registry.enrich_kernel_plan_with_cache(registry.kernel_plan(load_config(args.path)))
        print(registry.kernel_plan_to_json(plan) if args.json else registry.format_kernel_plan(plan))
    elif args.kernels_command == "compile":
        if args.arch and args.arch.upper() not in ("SM100", "SM_100A", "SM100A"):
            raise ContractError(f"unsupported kernel architecture {args.arch!r}; this build targets SM100 (sm_100a) only")
        payload = registry.compile_kernel_plan(load_config(args.path))
        _print_json(payload) if args.json else print(registry.format_compile_result(payload))
    elif args.kernels_command == "bench":
        from research_b200.kernels.bench import benchmark_kernel

        report = benchmark_kernel(args.op, load_config(args.path), rows=[int(r) for r in args.rows.split(",")],
                                  warmup=args.warmup, iters=args.iters)
        _print_json(report) if args.json else print(json.dumps(report, indent=1))
    return 0


def _profile(args: argparse.Namespace) -> int:
    if args.profile_command == "analyze":
        from research_b200.runtime.profile_analysis import (analyze_profile_root, format_profile_analysis,
                                                            profile_analysis_to_json)

        report = analyze_profile_root(args.root, warmup_steps=args.warmup_steps)
        print(profile_analysis_to_json(report) if args.json else format_profile_analysis(report))
    else:
        from research_b200.runtime.profile_bench import benchmark_component, benchmark_to_json, format_benchmark

        report = benchmark_component(args.component, warmup=args.warmup, iters=args.iters,
                                     artifact_dir=args.artifact_dir, trace=args.trace)
        if _is_rank0():
            print(benchmark_to_json(report) if args.json else format_benchmark(report))
    return 0


def main(argv: list[str] | None = None) -> int:
    parser = build_parser()
    args = parser.parse_args(argv)
    if args.command is None:
        parser.print_help()
        return 0
    try:
        return _dispatch(args)
    except JaxtitanError as exc:
        print(f"error: {exc}", file=sys.stderr)
        return 2


if __name__ == "__main__":
    raise SystemExit(main())
