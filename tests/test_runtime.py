"""End-to-end host loop on a tiny synthetic dataset: artifacts, resume exactness, failure events, CLI."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from research_b200.errors import ContractError
from research_b200.runtime.checkpoint_index import CheckpointIndex, load_checkpoint_index, record_checkpoint
from research_b200.runtime.inspect import inspect_run
from research_b200.runtime.training import run_training
from research_b200.services.checkpoints import LocalCheckpointService, read_array
from tests.helpers import tiny_dataset, tiny_raw_config, write_toml

ROOT = Path(__file__).resolve().parent.parent


def _config(tmp_path, **kw) -> Path:
    manifest = tiny_dataset(tmp_path)
    kw.setdefault("output_dir", (tmp_path / "runs").as_posix())
    return write_toml(tiny_raw_config(manifest, **kw), tmp_path / f"{kw.get('run_id', 'tiny')}.toml")


def _jsonl(path: Path):
    return [json.loads(l) for l in path.read_text().splitlines() if l.strip()]


def test_training_writes_the_full_artifact_set(tmp_path):
    cfg = _config(tmp_path, steps=6, evals=True, checkpoint_every=3, kind="trinity", optimizer="muon")
    summary = run_training(cfg)
    run_dir = tmp_path / "runs" / "tiny"
    assert summary.status == "completed" and summary.steps == 6 and summary.tokens_seen == 6 * 4 * 32
    for rel in ("manifest.json", "config/source.toml", "config/resolved.json", "events.jsonl", "metrics/train.jsonl",
                "metrics/eval.jsonl", "diagnostics/runtime.json", "checkpoints/index.json", "summaries/final.json"):
        assert (run_dir / rel).is_file(), rel
    rows = _jsonl(run_dir / "metrics" / "train.jsonl")
    assert [r["step"] for r in rows] == [1, 2, 3, 4, 5, 6]
    row = rows[-1]
    for key in ("loss", "lm_loss", "lr", "grad_norm", "param_norm", "update_norm", "total_loss", "batch_het",
                "tokens_per_sec", "train_tokens_per_sec", "flops_per_token", "mfu", "router_max_vio",
                "smebu_bias_norm", "document_aware", "documents_touched", "data_order", "moe_router_layers",
                "effective_tokens_per_step", "per_device_batch_size", "step_sec", "data_sec"):
        assert key in row, key
    assert row["document_aware"] is True and row["data_pipeline_backend"] == "blackwell_native"
    types = [e["type"] for e in _jsonl(run_dir / "events.jsonl")]
    assert types[0] == "run_initialized" and types[-1] == "training_completed"
    assert types.count("checkpoint_saved") == 2 and "eval_completed" in types
    eval_rows = _jsonl(run_dir / "metrics" / "eval.jsonl")
    # bits per byte: the synthetic tokenizer gives 3 bytes per token (0 for the end-of-text id)
    assert all(r["bpb"] is not None and 0.0 < r["bpb"] < r["loss"] for r in eval_rows)
    index = json.loads((run_dir / "checkpoints" / "index.json").read_text())
    assert index["latest_step"] == 6 and index["best_eval_step"] in (3, 6)
    ck = run_dir / "checkpoints" / "000006"
    for item in ("dataset", "host", "metadata"):
        assert (ck / item / "metadata").is_file()
    assert (ck / "_CHECKPOINT_METADATA").is_file() and (ck / "train" / "_METADATA").is_file()
    q = read_array(ck / "train" / "model.layers.0.attn.q.kernel")
    assert q.shape == (64, 64) and q.dtype == np.float32           # reference layout [in, out]
    assert read_array(ck / "train" / "tokens_seen").dtype == np.uint32
    runtime = json.loads((run_dir / "diagnostics" / "runtime.json").read_text())
    for key in ("mesh", "model", "training", "optimizer", "performance", "compile", "parallelism", "kernels",
                "sharding", "data_pipeline", "device_telemetry"):
        assert key in runtime, key
    assert runtime["compile"]["train"]["expected_batch_shape"] == [1, 4, 32]
    report = inspect_run(run_dir)
    assert report["status"] == "completed" and report["progress"]["step"] == 6
    with pytest.raises(ContractError, match="run directory already exists"):
        run_training(cfg)


def test_resume_continues_exactly_and_rejects_unsafe_changes(tmp_path):
    full = _config(tmp_path, steps=6, run_id="full", checkpoint_every=100)
    run_training(full)
    want = [r["loss_sum"] for r in _jsonl(tmp_path / "runs" / "full" / "metrics" / "train.jsonl")]
    manifest = tmp_path / "ds" / "manifest.json"
    part_raw = tiny_raw_config(manifest, steps=3, run_id="part", checkpoint_every=100,
                               output_dir=(tmp_path / "runs").as_posix())
    part = write_toml(part_raw, tmp_path / "part.toml")
    run_training(part)
    part_raw["training"]["target_tokens"] = 6 * 4 * 32          # constant schedule: target_tokens may grow
    write_toml(part_raw, part)
    summary = run_training(part, resume=True)
    got = [r["loss_sum"] for r in _jsonl(tmp_path / "runs" / "part" / "metrics" / "train.jsonl")]
    assert summary.steps == 6 and len(got) == 6
    assert np.allclose(got, want, rtol=1e-6, atol=1e-5)
    events = [e["type"] for e in _jsonl(tmp_path / "runs" / "part" / "events.jsonl")]
    assert "training_resumed" in events
    part_raw["training"]["target_tokens"] = 8 * 4 * 32
    part_raw["model"]["hidden_size"] = 128
    write_toml(part_raw, part)
    with pytest.raises(ContractError, match="resume compatibility mismatch at compatibility.model.hidden_size"):
        run_training(part, resume=True)
    events = _jsonl(tmp_path / "runs" / "part" / "events.jsonl")
    assert events[-1]["type"] == "training_failed" and events[-2]["type"] == "checkpoint_restore_failed"


def test_data_exhaustion_and_nonfinite_abort_with_events(tmp_path, monkeypatch):
    cfg = _config(tmp_path, steps=100000, run_id="exhaust", order="sequential")
    with pytest.raises(ContractError, match="training data exhausted"):
        run_training(cfg)
    assert _jsonl(tmp_path / "runs" / "exhaust" / "events.jsonl")[-1]["type"] == "training_failed"

    manifest = tmp_path / "ds" / "manifest.json"
    cfg2 = write_toml(tiny_raw_config(manifest, steps=3, run_id="nan", output_dir=(tmp_path / "runs").as_posix()),
                      tmp_path / "nan.toml")

    def poison(trainer):
        original = trainer.train_step_fn.run

        def run(batches, diagnostics=False):
            metrics = original(batches, diagnostics=diagnostics)
            metrics.grad_norm = float("nan")
            victim = trainer.store.entries[1]
            victim.param.main_grad.view(-1)[:3] = float("inf")      # the event must name this leaf
            return metrics

        trainer.train_step_fn.run = run

    with pytest.raises(ContractError, match="non-finite training metrics"):
        run_training(cfg2, trainer_hook=poison)
    events = _jsonl(tmp_path / "runs" / "nan" / "events.jsonl")
    types = [e["type"] for e in events]
    assert "optimizer_nonfinite" in types and types[-1] == "training_failed"
    leaves = next(e for e in events if e["type"] == "optimizer_nonfinite")["leaves"]
    assert [(leaf["kind"], leaf["inf"], leaf["nan"]) for leaf in leaves] == [("grad", 3, 0)]
    assert not (tmp_path / "runs" / "nan" / "checkpoints" / "000001").exists()


def test_checkpoint_retention_index_and_corruption(tmp_path):
    svc = LocalCheckpointService(tmp_path, max_to_keep=2)
    ds = {"a": 1}
    index = CheckpointIndex()
    for step, ev in ((1, 3.0), (2, 1.0), (3, 2.0), (4, 2.5)):
        path = svc.save(step, {"step": np.asarray(step, dtype=np.int32), "w": np.arange(6, dtype=np.float32).reshape(2, 3)},
                        ds, {"dataset": ds}, {"schema_version": 1})
        index = record_checkpoint(index, tmp_path, step=step, tokens_seen=step * 10, checkpoint_path=path,
                                  reason="cadence", train_loss=1.0, eval_loss=ev)
        svc.set_protected_steps(index.protected_steps())
    assert svc.all_steps() == [2, 3, 4]                      # newest two + the best (step 2)
    (tmp_path / "checkpoints" / "index.json").write_text(json.dumps(index.to_dict()))
    loaded = load_checkpoint_index(tmp_path)
    assert loaded.best_record.step == 2 and loaded.latest_record.step == 4
    assert [r.retained for r in loaded.records] == [False, True, True, True]
    chunk = tmp_path / "checkpoints" / "000004" / "train" / "w" / "0.0"
    chunk.write_bytes(chunk.read_bytes()[:-4])
    with pytest.raises(ContractError, match="missing or has the wrong size"):
        svc.restore(4)
    with pytest.raises(ContractError, match="host_state.dataset must match"):
        svc.save(5, {}, ds, {"dataset": {"a": 2}}, {})
    (tmp_path / "checkpoints" / "index.json").write_text("{not json")
    with pytest.raises(ContractError, match="failed to parse checkpoint index"):
        load_checkpoint_index(tmp_path)


def test_watchdog_reports_lost_and_lagging_ranks(tmp_path):
    from research_b200.runtime.watchdog import HeartbeatWriter, Watchdog

    dog = Watchdog(tmp_path, 3, timeout_s=10.0, max_step_lag=2)
    t0 = dog.started
    HeartbeatWriter(tmp_path, 0).beat(5, now=t0 + 20)
    HeartbeatWriter(tmp_path, 1).beat(5, now=t0 + 1)      # stale
    assert dog.lost_ranks(now=t0 + 5) == []               # rank 2 has not reported yet, still within the limit
    lost = {item["rank"]: item["reason"] for item in dog.lost_ranks(now=t0 + 21)}
    assert lost == {1: "stale_heartbeat", 2: "no_heartbeat"}
    HeartbeatWriter(tmp_path, 1).beat(1, now=t0 + 15)
    HeartbeatWriter(tmp_path, 2).beat(5, now=t0 + 20)
    lost = dog.lost_ranks(now=t0 + 21)
    assert [(i["rank"], i["reason"]) for i in lost] == [(1, "step_lag")]

    class Sink:
        events = []

        def append_event(self, e):
            self.events.append(e)

    with pytest.raises(ContractError, match="lost heartbeat"):
        dog.check(Sink(), "r", now=t0 + 21)
    assert Sink.events[-1]["type"] == "rank_heartbeat_lost"


def test_cli_exit_codes_and_json(tmp_path):
    cfg = _config(tmp_path, steps=2, run_id="cli", checkpoint_every=2, evals=True)
    exe = [sys.executable, str(ROOT / "bin" / "jaxtitan")]
    ok = subprocess.run(exe + ["config", "check", str(cfg), "--json"], capture_output=True, text=True)
    assert ok.returncode == 0 and json.loads(ok.stdout)["run_id"] == "cli"
    bad = subprocess.run(exe + ["config", "check", str(tmp_path / "nope.toml")], capture_output=True, text=True)
    assert bad.returncode == 2 and bad.stderr.startswith("error: failed to read config")
    pre = subprocess.run(exe + ["run", "preflight", str(cfg), "--json"], capture_output=True, text=True)
    assert pre.returncode == 0, pre.stderr
    report = json.loads(pre.stdout)
    assert report["status"] == "ok" and report["first_step"]["loss"] > 0 and not (tmp_path / "runs" / "cli").exists()
    train = subprocess.run(exe + ["run", "train", str(cfg)], capture_output=True, text=True)
    assert train.returncode == 0 and "completed: step=2" in train.stdout, train.stderr
    again = subprocess.run(exe + ["run", "train", str(cfg)], capture_output=True, text=True, stdin=subprocess.DEVNULL)
    assert again.returncode == 2 and "rerun with --overwrite" in again.stderr
    run_dir = tmp_path / "runs" / "cli"
    ev = subprocess.run(exe + ["eval", "checkpoint", str(run_dir), "--checkpoint", "latest", "--json"],
                        capture_output=True, text=True)
    assert ev.returncode == 0 and json.loads(ev.stdout)["checkpoint_step"] == 2, ev.stderr
    assert (run_dir / "evals" / "checkpoints" / "000002.json").is_file()
    sm = subprocess.run(exe + ["sample", "checkpoint", str(run_dir), "--checkpoint", "best", "--prompt-ids", "1,2,3",
                               "--max-new-tokens", "4", "--top-k", "1", "--json"], capture_output=True, text=True)
    assert sm.returncode == 0 and len(json.loads(sm.stdout)["generated_ids"]) == 4, sm.stderr
    assert (run_dir / "samples" / "checkpoints" / "000002.jsonl").is_file()
    bad_prompt = subprocess.run(exe + ["sample", "checkpoint", str(run_dir), "--checkpoint", "latest", "--prompt-ids",
                                       "1,x", "--max-new-tokens", "2"], capture_output=True, text=True)
    assert bad_prompt.returncode == 2 and "invalid token id" in bad_prompt.stderr
    ins = subprocess.run(exe + ["run", "inspect", str(run_dir), "--json"], capture_output=True, text=True)
    inspected = json.loads(ins.stdout)
    assert inspected["checkpoint_index"]["latest_step"] == 2 and inspected["latest_checkpoint"]["exists"]
    assert [c["step"] for c in inspected["checkpoints"]] == [2] and inspected["final"]["step"] == 2
    text = subprocess.run(exe + ["run", "inspect", str(run_dir)], capture_output=True, text=True).stdout
    assert "status: completed" in text and "latest checkpoint: step=2" in text and "kernels: enabled=True" in text
    kl = subprocess.run(exe + ["kernels", "list", "--json"], capture_output=True, text=True)
    assert kl.returncode == 0 and any(k["op"] == "gemm" for k in json.loads(kl.stdout)["kernels"])


def test_batch_prefetcher_hands_out_the_same_batches_and_states(tmp_path):
    """The worker thread runs ahead, but the trainer's data state moves only with the batches handed out, and
    assigning a state (resume) drops what was assembled ahead."""
    import numpy as np

    from research_b200.config.loader import run_spec_from_mapping
    from research_b200.runtime.trainer import Trainer
    from tests.helpers import tiny_dataset, tiny_raw_config

    manifest = tiny_dataset(tmp_path)
    spec = run_spec_from_mapping(tiny_raw_config(manifest, accum=2))
    ahead, plain = Trainer(spec, device="cpu"), Trainer(spec, device="cpu")
    plain.prefetch = False
    for _ in range(3):
        a, b = ahead.next_accumulated_batch(), plain.next_accumulated_batch()
        assert len(a) == len(b) == 2
        for x, y in zip(a, b):
            assert np.array_equal(np.asarray(x.input_ids), np.asarray(y.input_ids))
        assert ahead.data.state_to_json(ahead.data_state) == plain.data.state_to_json(plain.data_state)
        assert ahead.last_provenance == plain.last_provenance
    # resume from the plain trainer's second position: the batches assembled ahead must not be used
    rewind = Trainer(spec, device="cpu")
    first = rewind.next_accumulated_batch()
    second = rewind.next_accumulated_batch()
    state_after_first = Trainer(spec, device="cpu")
    state_after_first.prefetch = False
    state_after_first.next_accumulated_batch()
    rewind.data_state = state_after_first.data_state
    again = rewind.next_accumulated_batch()
    assert np.array_equal(np.asarray(again[0].input_ids), np.asarray(second[0].input_ids))
    assert not np.array_equal(np.asarray(again[0].input_ids), np.asarray(first[0].input_ids))
    for t in (ahead, rewind):
        t.close_prefetcher()
