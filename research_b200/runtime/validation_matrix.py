"""Validation matrices: fixed sets of short training runs over layouts and optimizers on the GPUs of one box, an
archive of their run directories, and analyzers that gate a candidate archive (alone, or against a baseline archive).

The reference validates its multi-GPU paths with cloud matrices and analyzers
(scripts/jaxtitan/cloud_moe_m1_h100_matrix.sh, cloud_dist_muon_m2_matrix.sh, cloud_dist_muon_leaf_bench.sh: 17-step
correctness runs and 64-step profile runs per layout and optimizer, bundled as a ``.tgz``;
scripts/jaxtitan/analyze_moe_m1_h100_results.py:78-118, analyze_dist_muon_m2_results.py and
analyze_dist_muon_leaf_bench.py: per-run steady medians, a speed-up gate against a baseline bundle, an overall
gate as the exit code).  Here the runner is local - one ``torch.distributed.run`` launch of ``jaxtitan run train`` per
case on the GPUs of this box - and the gates are the ones this stack can state about itself:

* the run completed, every loss is finite and the loss fell;
* no ``*_failed``, ``optimizer_nonfinite`` or ``rank_lost`` event;
* the optimizer-health and router-health roll-ups of ``run inspect`` are clean;
* paired cases (peer-memory kernels against NCCL, distributed against duplicated Muon) stay inside a step-time
  envelope; with a baseline archive, every shared case keeps at least ``min_speedup`` of the baseline's step time.

``python -m research_b200.runtime.validation_matrix run correctness17 --gpus 4 --out runs/matrix`` runs a matrix,
``... analyze runs/matrix/correctness17.tgz [--baseline old.tgz]`` prints the table and exits 1 when a gate fails,
``... analyze-muon runs/muon-bench`` gates the artifact of ``jaxtitan profile bench muon``.
"""

from __future__ import annotations

import argparse
import json
import math
import shutil
import subprocess
import sys
import tarfile
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Mapping

from research_b200.errors import ContractError

SCHEMA_VERSION = 1
FAILURE_EVENTS = ("training_failed", "checkpoint_restore_failed", "eval_failed", "optimizer_nonfinite", "rank_lost",
                  "rank_heartbeat_lost")
REPO = Path(__file__).resolve().parents[2]


# ---------------------------------------------------------------------------------------------------
# cases
# ---------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class MatrixCase:
    """One run of a matrix: a base config from ``configs/``, re-meshed and shortened."""

    run_id: str
    base: str                                    # file name under configs/
    axis_names: tuple[str, ...]
    axis_sizes: tuple[int, ...]
    steps: int
    optimizer: str | None = None
    parallelism: Mapping[str, Any] = field(default_factory=dict)
    model: Mapping[str, Any] = field(default_factory=dict)
    env: Mapping[str, str] = field(default_factory=dict)
    optimizer_options: Mapping[str, Any] = field(default_factory=dict)
    per_replica_batch: int = 2
    seq_len: int | None = None
    profile_steps: tuple[int, int] | None = None      # (first step, number of steps) of a profiler trace window

    @property
    def gpus(self) -> int:
        return math.prod(self.axis_sizes)


_SMALL_DENSE = {"hidden_size": 1024, "intermediate_size": 2816, "num_layers": 4, "num_heads": 8, "n_kv_heads": 4}
_SMALL_MOE = {"hidden_size": 1024, "num_layers": 4, "num_heads": 8, "n_kv_heads": 4}


def _family(prefix: str, steps: int, profile: tuple[int, int] | None) -> list[MatrixCase]:
    dense, moe, ctx = "dense_1p3b_fsdp8_muon.toml", "moe_7b_ep8_dion.toml", "dense_1p3b_cp4_fsdp2_32k.toml"
    nccl = {"RESEARCH_B200_PEER_COLLECTIVES": "0"}
    mk = lambda rid, *a, **k: MatrixCase(f"{prefix}_{rid}", *a, steps=steps, profile_steps=profile, **k)   # noqa: E731
    return [
        mk("dense_fsdp4_muon_fused", dense, ("fsdp",), (4,), optimizer="muon", model=_SMALL_DENSE),
        mk("dense_fsdp4_muon_nccl", dense, ("fsdp",), (4,), optimizer="muon", model=_SMALL_DENSE, env=nccl),
        mk("dense_fsdp4_adamw_fused", dense, ("fsdp",), (4,), optimizer="adamw", model=_SMALL_DENSE),
        mk("dense_tp2_muon_distributed", dense, ("data", "tensor"), (2, 2), optimizer="muon", model=_SMALL_DENSE,
           parallelism={"mode": "ddp", "tensor_parallel": True}, optimizer_options={"muon_tp_mode": "distributed"}),
        mk("dense_tp2_muon_duplicated", dense, ("data", "tensor"), (2, 2), optimizer="muon", model=_SMALL_DENSE,
           parallelism={"mode": "ddp", "tensor_parallel": True}, optimizer_options={"muon_tp_mode": "duplicated"}),
        mk("dense_fsdp4_sharded_weights_muon_fused", dense, ("fsdp",), (4,), optimizer="muon", model=_SMALL_DENSE,
           parallelism={"fsdp_resident": False}),
        mk("moe_ep4_adamw_fused", moe, ("fsdp",), (4,), optimizer="adamw", model=_SMALL_MOE,
           parallelism={"expert_parallel": True}),
        mk("moe_ep4_adamw_nccl", moe, ("fsdp",), (4,), optimizer="adamw", model=_SMALL_MOE,
           parallelism={"expert_parallel": True}, env=nccl),
        mk("moe_ep4_dion_fused", moe, ("fsdp",), (4,), optimizer="dion", model=_SMALL_MOE,
           parallelism={"expert_parallel": True}),
        mk("dense_cp4_muon_fused", ctx, ("context",), (4,), optimizer="muon", model=_SMALL_DENSE, seq_len=8192,
           per_replica_batch=1, parallelism={"mode": "ddp", "context_parallel": True}),
        mk("dense_cp4_muon_nccl", ctx, ("context",), (4,), optimizer="muon", model=_SMALL_DENSE, seq_len=8192,
           per_replica_batch=1, parallelism={"mode": "ddp", "context_parallel": True}, env=nccl),
    ]


MATRICES: dict[str, list[MatrixCase]] = {
    "correctness17": _family("local_4gpu_correctness17", 17, None),
    "profile64": _family("local_4gpu_profile64", 64, (24, 2)),
}


# ---------------------------------------------------------------------------------------------------
# configs
# ---------------------------------------------------------------------------------------------------
def _toml_value(value: Any) -> str:
    if isinstance(value, bool):
        return "true" if value else "false"
    if isinstance(value, (int, float)):
        return repr(value)
    if isinstance(value, str):
        return json.dumps(value)
    if isinstance(value, (list, tuple)):
        return "[" + ", ".join(_toml_value(v) for v in value) + "]"
    raise ContractError(f"cannot write {type(value).__name__} to TOML")


def write_toml(raw: Mapping[str, Any]) -> str:
    """Tables of scalars, lists and nested tables (all that a run config holds) as TOML text."""

    lines: list[str] = []

    def emit(table: Mapping[str, Any], path: tuple[str, ...]) -> None:
        scalars = {k: v for k, v in table.items() if not isinstance(v, Mapping)}
        if path and (scalars or not table):
            lines.append(f"[{'.'.join(path)}]")
        for k, v in scalars.items():
            lines.append(f"{k} = {_toml_value(v)}")
        if scalars or path:
            lines.append("")
        for k, v in table.items():
            if isinstance(v, Mapping):
                emit(v, path + (k,))

    emit(raw, ())
    return "\n".join(lines).rstrip() + "\n"


def derive_config(case: MatrixCase, manifest: str | Path, output_dir: str | Path) -> dict[str, Any]:
    """The base config of ``case`` re-meshed, shortened and pointed at ``manifest``."""

    import tomllib

    raw = tomllib.loads((REPO / "configs" / case.base).read_text())
    seq = case.seq_len or raw["training"]["seq_len"]
    raw["model"].update(case.model)
    raw["model"]["max_seq_len"] = max(seq, raw["model"].get("max_seq_len", seq)) if case.seq_len is None else seq
    replicas = math.prod(s for n, s in zip(case.axis_names, case.axis_sizes) if n in ("data", "fsdp"))
    gb = case.per_replica_batch * max(replicas, 1)
    raw["mesh"] = {"axis_names": list(case.axis_names), "axis_sizes": list(case.axis_sizes)}
    par = dict(raw.get("parallelism", {}))
    for key in ("tensor_parallel", "context_parallel", "expert_parallel"):
        par[key] = False
    par.update(case.parallelism)
    raw["parallelism"] = par
    if case.optimizer:
        raw["optimizer"]["name"] = case.optimizer
    raw["optimizer"].update(case.optimizer_options)
    raw["optimizer"]["schedule"] = {"name": "constant", "peak_lr": 3e-4, "warmup_steps": 4}
    raw["run"] = {**raw.get("run", {}), "id": case.run_id, "output_dir": str(output_dir)}
    raw["data"]["train_manifest"] = str(manifest)
    raw["training"].update(seq_len=seq, global_batch_size=gb, gradient_accumulation_steps=1,
                           target_tokens=gb * seq * case.steps, log_every_steps=1)   # every step is a row: the gates
    #                                                                                  and the steady medians read them
    raw.pop("evals", None)
    if case.profile_steps:
        raw["profiling"] = {"enabled": True, "trace_start_step": case.profile_steps[0],
                            "trace_steps": case.profile_steps[1]}
    return raw


# ---------------------------------------------------------------------------------------------------
# runner
# ---------------------------------------------------------------------------------------------------
def case_command(case: MatrixCase, config_path: Path, port: int) -> list[str]:
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={case.gpus}",
            "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "research_b200", "run", "train",
            str(config_path)]


def run_matrix(name: str, out_root: str | Path, *, gpus: int, manifest: str | Path, dry_run: bool = False,
               timeout_s: float = 1800.0, runner=subprocess.run, only: tuple[str, ...] = ()) -> dict[str, Any]:
    """Run (or, with ``dry_run``, only plan) every case of matrix ``name`` that fits ``gpus`` GPUs; returns and writes
    ``matrix.json`` (cases, commands, exit codes) and bundles the run directories as ``<name>.tgz``."""

    if name not in MATRICES:
        raise ContractError(f"unknown validation matrix {name!r}; known: {sorted(MATRICES)}")
    out_root = Path(out_root)
    runs_dir = out_root / name
    runs_dir.mkdir(parents=True, exist_ok=True)
    records = []
    for i, case in enumerate(MATRICES[name]):
        if only and not any(part in case.run_id for part in only):
            continue
        record: dict[str, Any] = {"case": asdict(case), "gpus": case.gpus}
        if case.gpus > gpus:
            record.update(status="skipped", reason=f"needs {case.gpus} GPUs, {gpus} given")
            records.append(record)
            continue
        cfg = derive_config(case, manifest, runs_dir)
        cfg_path = runs_dir / f"{case.run_id}.toml"
        cfg_path.write_text(write_toml(cfg))
        cmd = case_command(case, cfg_path, 29800 + i)
        record.update(config=cfg_path.as_posix(), command=cmd, env=dict(case.env))
        if dry_run:
            record["status"] = "planned"
        else:
            import os

            t0 = time.time()
            try:
                proc = runner(cmd, env={**os.environ, **case.env}, capture_output=True, text=True, timeout=timeout_s)
                record.update(status="ok" if proc.returncode == 0 else "failed", returncode=proc.returncode,
                              stderr_tail=(proc.stderr or "")[-2000:])
            except subprocess.TimeoutExpired:
                record.update(status="timeout", returncode=None)
            record["wall_s"] = round(time.time() - t0, 1)
        records.append(record)
    payload = {"schema_version": SCHEMA_VERSION, "matrix": name, "gpus": gpus, "cases": records}
    (runs_dir / "matrix.json").write_text(json.dumps(payload, indent=2, sort_keys=True, default=str))
    if not dry_run:
        # the bundle carries what the analyzers read (metrics, events, diagnostics, summaries, traces, configs); the
        # checkpoints stay in the run directories: gigabytes of weights would turn bundling into the longest step
        def without_checkpoints(info: tarfile.TarInfo) -> tarfile.TarInfo | None:
            return None if "/checkpoints/" in f"/{info.name}/" and not info.name.endswith("/checkpoints") else info

        with tarfile.open(out_root / f"{name}.tgz", "w:gz") as archive:
            archive.add(runs_dir, arcname=name, filter=without_checkpoints)
    return payload


# ---------------------------------------------------------------------------------------------------
# analyzers
# ---------------------------------------------------------------------------------------------------
def materialize(source: str | Path, work_dir: str | Path) -> Path:
    """A capture directory as it is, or a ``.tgz`` / ``.tar.gz`` bundle extracted below ``work_dir``."""

    source, work_dir = Path(source), Path(work_dir)
    if source.is_dir():
        return source
    if not source.is_file():
        raise ContractError(f"missing artifact: {source}")
    if not (source.suffix == ".tgz" or source.name.endswith(".tar.gz")):
        raise ContractError(f"unsupported artifact type: {source}")
    if work_dir.exists():
        shutil.rmtree(work_dir)
    work_dir.mkdir(parents=True)
    with tarfile.open(source, "r:gz") as archive:
        archive.extractall(work_dir, filter="data")
    return work_dir


def _jsonl(path: Path) -> list[dict[str, Any]]:
    if not path.is_file():
        return []
    return [json.loads(line) for line in path.read_text().splitlines() if line.strip()]


def gate_run(run_dir: Path) -> dict[str, Any]:
    """The per-run gates (see the module docstring) from the artifacts of one run directory."""

    from research_b200.runtime.inspect import optimizer_health, router_health

    train = _jsonl(run_dir / "metrics" / "train.jsonl")
    events = _jsonl(run_dir / "events.jsonl")
    summary_path = run_dir / "summaries" / "final.json"
    summary = json.loads(summary_path.read_text()) if summary_path.is_file() else {}
    types = [e.get("type") for e in events]
    losses = [float(r["loss"]) for r in train if r.get("loss") is not None]
    problems: list[str] = []
    if "training_completed" not in types:
        problems.append("no training_completed event")
    bad = sorted({t for t in types if t in FAILURE_EVENTS or str(t).endswith("_failed")})
    if bad:
        problems.append(f"failure events: {bad}")
    if not losses:
        problems.append("no training rows")
    elif not all(math.isfinite(x) for x in losses):
        problems.append("non-finite loss")
    elif len(losses) >= 4 and not min(losses[len(losses) // 2:]) < losses[0]:
        problems.append(f"loss did not fall: first {losses[0]:.4f}, best of the second half "
                        f"{min(losses[len(losses) // 2:]):.4f}")
    # Non-finite optimizer groups fail the run.  Groups without a gradient or an update (a router bias that the
    # balance policy moves instead of the optimizer, an expert that no token reached) and dead experts are reported
    # next to the verdict, as the reference's roll-ups report them, but do not fail it.
    notes: list[str] = []
    opt = optimizer_health(summary, train[-8:])
    if opt:
        if opt.get("nonfinite_groups"):
            problems.append(f"optimizer health: nonfinite_groups = {opt['nonfinite_groups']}")
        for key in ("groups_with_zero_grad", "groups_with_zero_update"):
            if opt.get(key):
                notes.append(f"{key} = {opt[key]}")
    rtr = router_health(summary, train[-8:])
    if rtr and rtr.get("dead_experts_count"):
        notes.append(f"dead experts = {rtr['dead_experts_count']}")
    return {"run_id": run_dir.name, "rows": len(train), "first_loss": losses[0] if losses else None,
            "final_loss": losses[-1] if losses else None, "problems": problems, "notes": notes,
            "gate": not problems}


PAIRS = (("fused", "nccl", "transport", 1.10), ("distributed", "duplicated", "muon_tp_mode", 1.25))


def analyze_matrix(candidate: str | Path, *, baseline: str | Path | None = None, min_speedup: float = 0.95,
                   warmup_steps: int = 2, work_dir: str | Path = "matrix_analysis_extract") -> dict[str, Any]:
    """Gates of every run below ``candidate``; pair envelopes; with ``baseline``, a step-time gate per shared run."""

    from research_b200.runtime.profile_analysis import analyze_profile_root

    cand_root = materialize(candidate, Path(work_dir) / "candidate")
    cand = analyze_profile_root(cand_root, warmup_steps=warmup_steps)
    step = {r["run_id"]: r["steady"]["medians"].get("train_step_sec") for r in cand["runs"]}
    runs = [dict(gate_run(Path(r["path"])), train_step_sec=step[r["run_id"]]) for r in cand["runs"]]
    pairs = []
    for cand_tag, base_tag, kind, envelope in PAIRS:
        for rid, sec in sorted(step.items()):
            other = rid.replace(cand_tag, base_tag)
            if cand_tag not in rid or other == rid or other not in step or not sec or not step[other]:
                continue
            ratio = sec / step[other]
            pairs.append({"kind": kind, "candidate": rid, "reference": other, "step_time_ratio": ratio,
                          "envelope": envelope, "gate": ratio <= envelope})
    against = []
    if baseline is not None:
        base_root = materialize(baseline, Path(work_dir) / "baseline")
        base = analyze_profile_root(base_root, warmup_steps=warmup_steps)
        base_step = {r["run_id"]: r["steady"]["medians"].get("train_step_sec") for r in base["runs"]}
        for rid, sec in sorted(step.items()):
            if rid in base_step and sec and base_step[rid]:
                speedup = base_step[rid] / sec
                against.append({"run_id": rid, "baseline_train_step_sec": base_step[rid], "candidate_train_step_sec": sec,
                                "speedup": speedup, "gate": speedup >= min_speedup})
        if not against:
            raise ContractError("candidate and baseline share no run with a steady step time")
    overall = all(r["gate"] for r in runs) and all(p["gate"] for p in pairs) and all(a["gate"] for a in against)
    return {"schema_version": SCHEMA_VERSION, "candidate_source": cand["source"], "runs": runs, "pairs": pairs,
            "baseline": against, "min_speedup": min_speedup, "overall_gate": overall}


def format_matrix_analysis(payload: Mapping[str, Any]) -> str:
    ms = lambda v: "-" if not v else f"{v * 1000.0:.1f}"     # noqa: E731
    lines = ["run                                                        rows  first     final     step ms  gate"]
    for r in payload["runs"]:
        first = "-" if r["first_loss"] is None else f"{r['first_loss']:.4f}"
        final = "-" if r["final_loss"] is None else f"{r['final_loss']:.4f}"
        lines.append(f"{r['run_id']:<58} {r['rows']:>4}  {first:<8}  {final:<8}  {ms(r['train_step_sec']):>7}  "
                     f"{'ok' if r['gate'] else 'FAIL: ' + '; '.join(r['problems'])}"
                     f"{'  (' + '; '.join(r['notes']) + ')' if r.get('notes') else ''}")
    for p in payload["pairs"]:
        lines.append(f"pair {p['kind']}: {p['candidate']} / {p['reference']} = {p['step_time_ratio']:.3f} "
                     f"(envelope {p['envelope']:.2f}) {'ok' if p['gate'] else 'FAIL'}")
    for a in payload["baseline"]:
        lines.append(f"baseline {a['run_id']}: {ms(a['baseline_train_step_sec'])} -> {ms(a['candidate_train_step_sec'])} ms, "
                     f"{a['speedup']:.2f}x {'ok' if a['gate'] else 'FAIL'}")
    lines.append(f"overall_gate={payload['overall_gate']}")
    return "\n".join(lines)


def analyze_muon_bench(artifact_dir: str | Path) -> dict[str, Any]:
    """Gate the artifact of the distributed-Muon selector: every selected candidate passed its correctness gate, ran
    twice to the same bits and left replicas equal; lists what each leaf class selected and by how much it won."""

    root = Path(artifact_dir)
    manifests = sorted(root.rglob("manifest.json")) if root.is_dir() else []
    if not manifests:
        raise ContractError(f"no Muon benchmark manifest below {root}")
    raw = json.loads(manifests[-1].read_text())
    rows, problems = [], []
    for case in raw.get("cases", []):
        if "skipped" in case:
            continue
        by_exec = {c["execution"]: c for c in case.get("candidates", [])}
        chosen = by_exec.get(case.get("selected"))
        if chosen is None:
            problems.append(f"{case.get('case')}: selected execution {case.get('selected')!r} is not a candidate")
            continue
        ok = bool(chosen.get("correctness_gate", False)) and bool(chosen.get("deterministic", False)) and \
            float(chosen.get("replica_max_abs_error", 1.0)) == 0.0
        if not ok:
            shown = {k: chosen.get(k) for k in ("correctness_gate", "deterministic", "replica_max_abs_error",
                                                "max_update_abs_error", "max_parameter_abs_error")}
            problems.append(f"{case.get('case')}: selected {case.get('selected')} fails its gate {shown}")
        dup = by_exec.get("duplicated", {}).get("timing_ms", {}).get("median")
        sel = chosen.get("timing_ms", {}).get("median")
        rows.append({"case": case.get("case"), "selected": case.get("selected"), "median_ms": sel,
                     "duplicated_ms": dup, "speedup_vs_duplicated": (dup / sel) if dup and sel else None, "gate": ok})
    overall = not problems and bool(raw.get("all_selected_pass", True))
    return {"schema_version": SCHEMA_VERSION, "source": manifests[-1].as_posix(), "transport": raw.get("transport"),
            "rows": rows, "problems": problems, "overall_gate": overall}


# ---------------------------------------------------------------------------------------------------
# command line
# ---------------------------------------------------------------------------------------------------
def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description="Validation matrices on the GPUs of one box")
    sub = ap.add_subparsers(dest="command", required=True)
    p = sub.add_parser("run", help="run every case of a matrix and bundle the run directories")
    p.add_argument("matrix", choices=sorted(MATRICES))
    p.add_argument("--gpus", type=int, required=True)
    p.add_argument("--out", default="runs/validation")
    p.add_argument("--manifest", required=True, help="prepared-token manifest (jaxtitan data prepare | synth)")
    p.add_argument("--dry-run", action="store_true", help="write the configs and the plan, launch nothing")
    p.add_argument("--only", action="append", default=[], metavar="TEXT",
                   help="run only the cases whose id contains TEXT (repeatable)")
    p = sub.add_parser("analyze", help="gate a capture directory or bundle, optionally against a baseline")
    p.add_argument("candidate")
    p.add_argument("--baseline")
    p.add_argument("--min-speedup", type=float, default=0.95)
    p.add_argument("--work-dir", default="matrix_analysis_extract")
    p.add_argument("--json-out")
    p = sub.add_parser("analyze-muon", help="gate the artifact of `jaxtitan profile bench muon`")
    p.add_argument("artifact_dir")
    p.add_argument("--json-out")
    args = ap.parse_args(argv)
    try:
        if args.command == "run":
            payload = run_matrix(args.matrix, args.out, gpus=args.gpus, manifest=args.manifest, dry_run=args.dry_run,
                                 only=tuple(args.only))
            for rec in payload["cases"]:
                print(f"{rec['case']['run_id']:<58} {rec['status']}")
            return 0 if all(r["status"] in ("ok", "planned", "skipped") for r in payload["cases"]) else 1
        if args.command == "analyze":
            payload = analyze_matrix(args.candidate, baseline=args.baseline, min_speedup=args.min_speedup,
                                     work_dir=args.work_dir)
            print(format_matrix_analysis(payload))
        else:
            payload = analyze_muon_bench(args.artifact_dir)
            for row in payload["rows"]:
                sp = "-" if row["speedup_vs_duplicated"] is None else f"{row['speedup_vs_duplicated']:.2f}x"
                print(f"{row['case']:<44} {row['selected']:<26} {sp:>7} {'ok' if row['gate'] else 'FAIL'}")
            for problem in payload["problems"]:
                print("problem:", problem)
            print(f"overall_gate={payload['overall_gate']}")
        if args.json_out:
            out = Path(args.json_out)
            out.parent.mkdir(parents=True, exist_ok=True)
            out.write_text(json.dumps(payload, sort_keys=True, indent=2))
        return 0 if payload["overall_gate"] else 1
    except ContractError as exc:
        print(f"error: {exc}", file=sys.stderr)
        return 2


if __name__ == "__main__":
    raise SystemExit(main())
