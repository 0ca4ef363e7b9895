"""Host services that talk to something outside the process, tested against fakes: Hugging Face streaming with a
fake iterable dataset, the W&B mirror with a fake ``wandb`` module, the profiler window with a fake
``torch.profiler.profile``, and the profile analyzer on hand-made runs and traces.  (The reference tests the same
parts the same way: tests/jaxtitan/test_data_pipeline.py:123-182, test_runtime_training.py:300-595,
test_profile_analysis.py.)"""

import json
import sys
import types

import numpy as np
import pytest

from research_b200.config import run_spec_from_mapping
from research_b200.config.specs import DataSpec, HFStreamingSpec
from research_b200.errors import ContractError
from tests.helpers import tiny_dataset, tiny_raw_config, write_toml


# ---- Hugging Face streaming ------------------------------------------------------------------------
class FakeTokenizer:
    eot_id = 255

    def encode(self, text):
        return [ord(c) % 200 for c in text]


class FakeIterableDataset:
    """Rows of text with the ``state_dict`` / ``load_state_dict`` pair of a streaming ``datasets`` dataset."""

    def __init__(self, rows):
        self.rows, self.position = rows, 0

    def __iter__(self):
        while self.position < len(self.rows):
            row = self.rows[self.position]
            self.position += 1
            yield row

    def state_dict(self):
        return {"position": self.position}

    def load_state_dict(self, state):
        self.position = int(state["position"])


def _streaming(rows, seq_len=8, batch=2, loads=None):
    from research_b200.data.streaming import HFStreamingTextPipeline

    spec = DataSpec(mode="hf_streaming", tokenizer_id="fake", hf_streaming=HFStreamingSpec(
        dataset="corp/us", split="train", revision="abc123"))

    def loader(s):
        if loads is not None:
            loads.append((s.dataset, s.split, s.revision))
        return FakeIterableDataset(rows)

    return HFStreamingTextPipeline(spec, seq_len=seq_len, batch_size=batch, dataset_loader=loader,
                                   tokenizer=FakeTokenizer())


ROWS = [{"text": "the quick brown fox"}, {"text": ""}, {"text": "jumps over the lazy dog", "other": 1},
        {"text": "pack my box with five dozen liquor jugs"}, {"text": "sphinx of black quartz judge my vow"}]


def _stream_tokens(rows, eot=255):
    out = []
    for row in rows:
        out.extend([ord(c) % 200 for c in row["text"]] + [eot])
    return out


def test_streaming_records_overlap_by_one_token_so_every_token_is_a_target_once():
    loads = []
    pipe = _streaming(ROWS, loads=loads)
    first = pipe.next_batch(pipe.initial_state())
    assert loads == [("corp/us", "train", "abc123")]                        # the pinned revision reaches the loader
    stream = _stream_tokens(ROWS)
    assert first.batch.input_ids.tolist() == [stream[0:8], stream[8:16]]
    assert first.batch.target_ids.tolist() == [stream[1:9], stream[9:17]]
    assert first.batch.loss_mask.all() and first.batch.input_ids.shape == (2, 8)
    st = first.state.stream_state
    assert st["pending_tokens"] == [stream[16]] and st["tokens_emitted"] == 16 and first.state.next_record_index == 2
    assert st["rows_seen"] == 1 and st["docs_seen"] == 1 and st["current_doc_active"] and st["hf_state"] == {"position": 0}
    assert st["current_doc_token_offset"] == 17                              # of the 20 tokens of the first document
    assert first.provenance.token_start == 0 and first.provenance.token_end == 16
    assert first.provenance.row_start_offsets == (0, 8) and first.provenance.row_doc_ids is None
    second = pipe.next_batch(first.state)
    assert second.batch.input_ids.tolist() == [stream[16:24], stream[24:32]]
    assert second.state.stream_state["rows_seen"] == 3                       # an empty text is a document of one EOT
    assert second.state.stream_state["docs_seen"] == 3
    d = pipe.describe()
    assert d["backend"] == "hf_streaming" and d["revision"] == "abc123" and d["exact_resume"] and d["num_records"] is None
    assert d["tokens_emitted"] == 32 and d["rows_seen"] == 3 and d["source"]["dataset"] == "corp/us"
    assert json.loads(d["source_summary"])["revision"] == "abc123" and d["document_aware"] is False


def test_streaming_never_holds_more_than_one_record_of_pending_tokens():
    long_rows = [{"text": "x" * 1000}, {"text": "y" * 1000}]
    pipe = _streaming(long_rows, seq_len=8, batch=2)
    state = pipe.initial_state()
    for _ in range(20):
        pb = pipe.next_batch(state)
        state = pb.state
        assert len(state.stream_state["pending_tokens"]) == 1


def test_streaming_resumes_with_the_very_next_token():
    pipe = _streaming(ROWS)
    state = pipe.initial_state()
    straight = []
    for _ in range(4):
        pb = pipe.next_batch(state)
        state = pb.state
        straight.append(pb.batch.input_ids.copy())
    for stop in (1, 2, 3):                                                   # mid-document and at a document's end
        pipe2 = _streaming(ROWS)
        state = pipe2.initial_state()
        for _ in range(stop):
            state = pipe2.next_batch(state).state
        saved = json.loads(json.dumps(pipe2.state_to_json(state)))          # what a checkpoint stores
        resumed = _streaming(ROWS)                                           # a new process, a new dataset object
        state = resumed.state_from_json(saved)
        for want in straight[stop:]:
            pb = resumed.next_batch(state)
            state = pb.state
            assert np.array_equal(pb.batch.input_ids, want)
    # going back to an older state of the same pipeline object restores it as well
    again = pipe.next_batch(pipe.state_from_json(saved))
    assert np.array_equal(again.batch.input_ids, straight[3])


def test_streaming_rejects_foreign_state_bad_rows_and_ends_cleanly():
    from research_b200.data.streaming import build_hf_streaming_pipeline, hf_streaming_compat_payload

    pipe = _streaming(ROWS[:1], seq_len=64)
    with pytest.raises(StopIteration, match="ended before one full batch"):
        pipe.next_batch(pipe.initial_state())
    other = _streaming(ROWS, seq_len=4)
    saved = other.state_to_json(other.next_batch(other.initial_state()).state)
    with pytest.raises(ContractError, match="state seq_len mismatch"):
        _streaming(ROWS, seq_len=8).state_from_json(saved)
    with pytest.raises(ContractError, match="token_offset must match"):
        other.state_from_json({**saved, "token_offset": 3})
    with pytest.raises(ContractError, match="only epoch=0"):
        other.state_from_json({**saved, "epoch": 1})
    with pytest.raises(ContractError, match="hf_state must be a JSON object"):
        other.state_from_json({**saved, "stream_state": {**saved["stream_state"], "hf_state": None}})
    broken = other.state_from_json({**saved, "stream_state": {**saved["stream_state"], "current_doc_token_offset": 999}})
    with pytest.raises(ContractError, match="outside current document tokens"):
        other.next_batch(broken)
    for rows, match in (([{"other": 1}], "missing text column"), ([{"text": 5}], "must contain strings"),
                        (["plain"], "rows must be mappings")):
        bad = _streaming(rows)
        with pytest.raises(ContractError, match=match):
            bad.next_batch(bad.initial_state())
    spec = DataSpec(mode="hf_streaming", tokenizer_id="fake", hf_streaming=HFStreamingSpec(
        dataset="corp/us", split="train", revision="abc123"))
    built = build_hf_streaming_pipeline(spec, seq_len=8, batch_size=2, tokenizer=FakeTokenizer(),
                                        dataset_loader=lambda s: FakeIterableDataset(ROWS))
    assert built.next_batch(built.initial_state()).batch.input_ids.shape == (2, 8)
    compat = hf_streaming_compat_payload(spec.hf_streaming, tokenizer_id="fake", seq_len=8, batch_size=2)
    assert compat["exact_resume"] and compat["source"]["revision"] == "abc123" and compat["order"] == "sequential"


# ---- W&B mirror --------------------------------------------------------------------------------------
class FakeWandb(types.ModuleType):
    def __init__(self, fail_on=None):
        super().__init__("wandb")
        self.calls, self.fail_on = [], fail_on
        self.run = types.SimpleNamespace(summary={})

    def _call(self, what, **kw):
        self.calls.append((what, kw))
        hit = self.fail_on(what, kw) if callable(self.fail_on) else self.fail_on == what
        if hit:
            raise RuntimeError(f"fake wandb {what} failure")

    def Table(self, columns, data):
        return {"columns": columns, "data": data}

    def init(self, **kw):
        self._call("init", **kw)
        return self.run

    def log(self, payload, step=None):
        self._call("log", payload=payload, step=step)

    def finish(self):
        self._call("finish")


def _wandb_config(tmp_path, run_id):
    manifest = tmp_path / "ds" / "manifest.json"
    if not manifest.exists():
        manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, steps=3, run_id=run_id, output_dir=(tmp_path / "runs").as_posix(), evals=True)
    raw["artifacts"] = {"wandb_enabled": True, "wandb_project": "proj", "wandb_mode": "offline",
                        "wandb_tags": ["a", "b"]}
    return write_toml(raw, tmp_path / f"{run_id}.toml")


def test_wandb_mirror_logs_namespaced_metrics_after_the_local_files(tmp_path, monkeypatch):
    from research_b200.runtime.training import run_training
    from research_b200.services.wandb import namespaced_metrics

    fake = FakeWandb()
    monkeypatch.setitem(sys.modules, "wandb", fake)
    summary = run_training(_wandb_config(tmp_path, "wb"))
    names = [c[0] for c in fake.calls]
    assert names[0] == "init" and names[-1] == "finish" and names.count("log") >= 4
    init = fake.calls[0][1]
    assert init["project"] == "proj" and init["mode"] == "offline" and init["resume"] == "allow"
    assert init["id"].startswith("wb-") and len(init["id"]) == len("wb-") + 16 and init["tags"] == ["a", "b"]
    train_logs = [c[1] for c in fake.calls if c[0] == "log" and "train/loss" in c[1]["payload"]]
    assert [c["step"] for c in train_logs] == [1, 2, 3]
    assert {"optimizer/grad_norm", "optimizer/lr", "perf/train_tokens_per_sec", "data/token_start"} <= \
        set(train_logs[-1]["payload"])
    assert any("eval/loss" in c[1]["payload"] for c in fake.calls if c[0] == "log")
    assert fake.run.summary["steps"] == summary.steps == 3
    meta = json.loads((tmp_path / "runs" / "wb" / "diagnostics" / "wandb.json").read_text())
    assert meta["enabled"] and meta["run_id"] == init["id"] and meta["project"] == "proj"
    assert meta["wandb_run_id"] == init["id"] and meta["resume"] == "allow" and meta["tags"] == ["a", "b"]
    ns = namespaced_metrics({"loss": 1.0, "router_max_vio": 0.1, "mfu": 0.4, "flag": True, "name": "x", "step": 3,
                             "bad": float("nan"), "worse": float("inf"), "optimizer_groups": [1], "gpu_power_w": 700.0,
                             "tokens_seen": 10, "smebu_bias_norm": 0.5, "optimizer_update_norm_max": 2.0})
    assert ns == {"train/loss": 1.0, "router/router_max_vio": 0.1, "perf/mfu": 0.4, "train/flag": True,
                  "perf/gpu_power_w": 700.0, "data/tokens_seen": 10, "router/smebu_bias_norm": 0.5,
                  "optimizer/optimizer_update_norm_max": 2.0}
    assert namespaced_metrics({"loss": 2.0, "eval_sec": 1.0}, "eval") == {"eval/loss": 2.0, "eval/eval_sec": 1.0}
    # lifecycle events become markers, the runtime diagnostics and the summary land in the W&B summary
    markers = [k for c in fake.calls if c[0] == "log" for k in c[1]["payload"] if k.startswith("event/") and
               k.count("/") == 1]
    assert markers[0] == "event/training_started" and markers[-1] == "event/training_completed"
    assert "event/checkpoint_saved" in markers
    assert fake.run.summary["diagnostics/device_count"] == 1 and fake.run.summary["diagnostics/flops_per_token"] > 0
    assert fake.run.summary["final/final_loss"] == pytest.approx(summary.final_loss)
    tables = [c[1]["payload"] for c in fake.calls if c[0] == "log" and "final/optimizer_groups" in c[1]["payload"]]
    assert len(tables) == 1 and "group" in " ".join(tables[0]["final/optimizer_groups"]["columns"])


def test_wandb_resume_continues_the_recorded_run_and_needs_its_metadata(tmp_path, monkeypatch):
    from research_b200.runtime.training import run_training

    fake = FakeWandb()
    monkeypatch.setitem(sys.modules, "wandb", fake)
    config = _wandb_config(tmp_path, "wbres")
    run_training(config)
    first_id = fake.calls[0][1]["id"]
    raw = config.read_text().replace(f"target_tokens = {32 * 4 * 3}", f"target_tokens = {32 * 4 * 5}")
    assert raw != config.read_text()
    config.write_text(raw)
    again = FakeWandb()
    monkeypatch.setitem(sys.modules, "wandb", again)
    summary = run_training(config, resume=True)
    init = again.calls[0][1]
    assert summary.steps == 5 and init["resume"] == "must" and init["id"] == first_id
    (tmp_path / "runs" / "wbres" / "diagnostics" / "wandb.json").unlink()
    monkeypatch.setitem(sys.modules, "wandb", FakeWandb())
    with pytest.raises(ContractError, match="diagnostics/wandb.json is missing"):
        run_training(config, resume=True)
    events = [json.loads(line) for line in (tmp_path / "runs" / "wbres" / "events.jsonl").read_text().splitlines()]
    assert events[-1]["type"] == "wandb_failed" and events[-1]["operation"] == "init"


def test_wandb_failure_is_an_event_and_aborts_with_local_files_intact(tmp_path, monkeypatch):
    from research_b200.runtime.training import run_training

    fake = FakeWandb(fail_on=lambda what, kw: what == "log" and "train/loss" in kw["payload"])
    monkeypatch.setitem(sys.modules, "wandb", fake)
    with pytest.raises(ContractError, match="wandb log_train failed"):
        run_training(_wandb_config(tmp_path, "wbfail"))
    after = [c for c in fake.calls[[c[0] == "log" and "train/loss" in c[1]["payload"] for c in fake.calls].index(True) + 1:]
             if c[0] == "log"]
    assert after == []                                                      # the mirror is off after its first failure
    run_dir = tmp_path / "runs" / "wbfail"
    events = [json.loads(line) for line in (run_dir / "events.jsonl").read_text().splitlines()]
    failed = next(e for e in events if e["type"] == "wandb_failed")
    assert failed["operation"] == "log_train" and failed["error_type"] == "RuntimeError"
    assert events[-1]["type"] == "training_failed"
    assert len((run_dir / "metrics" / "train.jsonl").read_text().splitlines()) == 1     # local row written first


def test_wandb_enabled_without_the_package_is_a_contract_error(tmp_path, monkeypatch):
    from research_b200.runtime.training import run_training

    monkeypatch.setitem(sys.modules, "wandb", None)                        # import wandb -> ImportError
    with pytest.raises(ContractError, match="wandb package is not importable"):
        run_training(_wandb_config(tmp_path, "wbmissing"))


# ---- profiler window ---------------------------------------------------------------------------------
class FakeProfile:
    instances = []

    def __init__(self, activities=None, fail_export=False):
        self.entered = self.exited = False
        self.exported = None
        FakeProfile.instances.append(self)

    def __enter__(self):
        self.entered = True
        return self

    def __exit__(self, *exc):
        self.exited = True
        return False

    def export_chrome_trace(self, path):
        if FakeProfile.fail_export:
            raise OSError("disk full")
        self.exported = path
        with open(path, "w") as f:
            json.dump({"traceEvents": []}, f)

    fail_export = False


class Sink:
    def __init__(self):
        self.events, self.profiling = [], None

    def append_event(self, e):
        self.events.append(e)

    def write_profiling_diagnostics(self, payload):
        self.profiling = payload


def _profiling_spec(tmp_path, **prof):
    raw = tiny_raw_config(tmp_path / "m.json")
    raw["profiling"] = dict(enabled=True, trace_start_step=2, trace_steps=2, **prof)
    return run_spec_from_mapping(raw)


def test_profiler_traces_exactly_the_configured_window(tmp_path, monkeypatch):
    import torch

    from research_b200.runtime.profiling import ProfilingManager

    FakeProfile.instances, FakeProfile.fail_export = [], False
    monkeypatch.setattr(torch.profiler, "profile", FakeProfile)
    (tmp_path / "profiles").mkdir()
    sink = Sink()
    mgr = ProfilingManager(_profiling_spec(tmp_path), tmp_path, sink)
    running = []
    for step in range(1, 6):
        with mgr.step(step):
            with mgr.annotate("train_step"):
                running.append(bool(FakeProfile.instances and FakeProfile.instances[-1].entered
                                    and not FakeProfile.instances[-1].exited))
    mgr.finish()
    assert running == [False, True, True, False, False]                     # steps 2 and 3 only
    assert len(FakeProfile.instances) == 1
    assert [e["type"] for e in sink.events] == ["profiling_trace_started", "profiling_trace_completed"]
    assert sink.events[0]["step"] == 2 and sink.events[1]["step"] == 3
    assert sink.profiling["status"] == "completed" and sink.profiling["trace_path"] == "profiles/trace_steps_2_3.json"
    assert (tmp_path / sink.profiling["trace_path"]).is_file()
    with pytest.raises(ContractError, match="is not after resumed step 2"):
        mgr.check_resume(2)
    mgr.check_resume(1)


def test_profiler_failure_and_disabled_modes(tmp_path, monkeypatch):
    import torch

    from research_b200.runtime.profiling import ProfilingManager

    FakeProfile.instances, FakeProfile.fail_export = [], True
    monkeypatch.setattr(torch.profiler, "profile", FakeProfile)
    (tmp_path / "profiles").mkdir()
    sink = Sink()
    mgr = ProfilingManager(_profiling_spec(tmp_path), tmp_path, sink)
    for step in range(1, 5):
        with mgr.step(step):
            pass
    assert [e["type"] for e in sink.events] == ["profiling_trace_started", "profiling_trace_failed"]
    assert sink.events[-1]["error_type"] == "OSError" and sink.profiling["status"] == "failed"
    FakeProfile.instances, FakeProfile.fail_export = [], False
    # a rank that is not the writer never starts a trace; a disabled section reports "disabled"
    quiet = ProfilingManager(_profiling_spec(tmp_path), tmp_path, Sink(), enabled=False)
    for step in range(1, 5):
        with quiet.step(step):
            pass
    assert FakeProfile.instances == []
    off = ProfilingManager(run_spec_from_mapping(tiny_raw_config(tmp_path / "m.json")), tmp_path, Sink())
    assert off.payload()["status"] == "disabled" and not off.active


# ---- profile analysis ----------------------------------------------------------------------------------
def _fake_run(root, name, *, step_sec, tps, trace_end=None, exclude=None, trace=None, optimizer="adamw"):
    run = root / name
    (run / "metrics").mkdir(parents=True)
    (run / "diagnostics").mkdir()
    rows = [{"step": i + 1, "train_step_sec": s, "step_sec": s + 0.01, "train_tokens_per_sec": t, "loss": 3.0 - 0.1 * i}
            for i, (s, t) in enumerate(zip(step_sec, tps))]
    (run / "metrics" / "train.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    events = [{"type": "checkpoint_saved", "step": s} for s in (exclude or [])]
    (run / "events.jsonl").write_text("\n".join(json.dumps(e) for e in events))
    (run / "diagnostics" / "runtime.json").write_text(json.dumps({
        "runtime": {"device_kind": "NVIDIA B200"}, "mesh": {"device_count": 8}, "optimizer": {"name": optimizer},
        "parallelism": {"mode": "fsdp"}}))
    if trace_end is not None:
        (run / "diagnostics" / "profiling.json").write_text(json.dumps({"enabled": True, "trace_end_step": trace_end}))
    if trace is not None:
        (run / "profiles").mkdir()
        (run / "profiles" / "trace.json").write_text(json.dumps({"traceEvents": trace}))
    return run


def test_profile_analysis_steady_window_medians_pairs_and_kernel_categories(tmp_path):
    from research_b200.runtime.profile_analysis import analyze_profile_root, categorize_kernel, summarize_trace

    trace = [
        {"ph": "X", "cat": "kernel", "name": "gemm_bf16_kernel<256>", "dur": 700.0},
        {"ph": "X", "cat": "kernel", "name": "attn_fwd_kernel<128>", "dur": 200.0},
        {"ph": "X", "cat": "kernel", "name": "ncclDevKernel_AllGather_RING_LL", "dur": 60.0},
        {"ph": "X", "cat": "kernel", "name": "ncclDevKernel_ReduceScatter_Sum_f32", "dur": 40.0},
        {"ph": "X", "cat": "cpu_op", "name": "aten::mm", "dur": 999.0},             # host op: ignored
        {"ph": "M", "name": "process_name"},
    ]
    _fake_run(tmp_path, "dense_tp_adamw", step_sec=[9.0, 0.5, 0.4, 0.41, 0.39, 5.0, 0.40],
              tps=[1, 100, 110, 108, 112, 10, 111], trace_end=3, exclude=[6], trace=trace)
    _fake_run(tmp_path, "dense_tp_muon", step_sec=[9.0, 0.6, 0.6, 0.62, 0.58, 0.60, 0.61],
              tps=[1, 80, 82, 81, 83, 82, 80], optimizer="muon")
    out = analyze_profile_root(tmp_path, warmup_steps=2)
    assert out["run_count"] == 2 and out["hardware"] == {"8xNVIDIA B200": ["dense_tp_adamw", "dense_tp_muon"]}
    adamw, muon = out["runs"]
    # steady window: after max(warmup + 1, trace_end + 1) = step 4, without the checkpoint step 6
    assert adamw["steady"]["start_step"] == 4 and adamw["steady"]["rows"] == 3 and adamw["steady"]["excluded_steps"] == [6]
    assert adamw["steady"]["medians"]["train_step_sec"] == pytest.approx(0.40)
    assert muon["steady"]["start_step"] == 3 and muon["steady"]["medians"]["train_step_sec"] == pytest.approx(0.60)
    (pair,) = out["comparisons"]
    assert pair["kind"] == "optimizer" and pair["candidate"] == "dense_tp_muon" and pair["baseline"] == "dense_tp_adamw"
    assert pair["train_step_delta"] == pytest.approx(0.5)
    t = adamw["traces"][0]
    assert t["total_gpu_time_us"] == 1000.0 and t["gpu_time_share"]["gemm"] == pytest.approx(0.7)
    assert t["collective_counts"] == {"AllGather": 1, "ReduceScatter": 1} and t["kernel_counts"]["nccl"] == 2
    assert t["top_kernels"][0]["name"].startswith("gemm_bf16_kernel")
    assert categorize_kernel("b200c_reduce_scatter_pull") == "other" and categorize_kernel("adamw_kernel") == "optimizer"
    assert summarize_trace(tmp_path / "dense_tp_adamw" / "profiles" / "trace.json")["trace"] == "trace.json"


def test_profile_analysis_rejects_bad_roots(tmp_path):
    from research_b200.runtime.profile_analysis import analyze_profile_root

    with pytest.raises(ContractError, match="not a directory"):
        analyze_profile_root(tmp_path / "nope")
    with pytest.raises(ContractError, match="no metrics/train.jsonl"):
        analyze_profile_root(tmp_path)
    with pytest.raises(ContractError, match="non-negative"):
        analyze_profile_root(tmp_path, warmup_steps=-1)


def _structured_run(root, name, *, optimizer, parallelism, step=0.5, status="completed", nonfinite=0, hidden=64):
    import gzip

    run = _fake_run(root, name, step_sec=[9.0, step, step, step, step], tps=[1, 100, 100, 100, 100], optimizer=optimizer)
    (run / "config").mkdir()
    (run / "summaries").mkdir()
    (run / "config" / "resolved.json").write_text(json.dumps({
        "model": {"name": "decoder", "hidden_size": hidden, "variant": name, "remat": "none"},
        "optimizer": {"name": optimizer}, "parallelism": parallelism}))
    (run / "summaries" / "final.json").write_text(json.dumps({
        "run_id": name, "status": status, "final_optimizer_nonfinite_group_count": nonfinite}))
    (run / "profiles").mkdir()
    with gzip.open(run / "profiles" / "step.trace.json.gz", "wt") as handle:
        json.dump({"traceEvents": [{"ph": "X", "cat": "kernel", "name": "gemm_bf16_kernel", "dur": 30.0},
                                   {"ph": "X", "cat": "gpu_memcpy", "name": "Memcpy DtoD", "dur": 10.0},
                                   {"ph": "X", "cat": "kernel", "name": "broken", "dur": "x"}]}, handle)
    return run


def test_profile_analysis_pairs_by_structure_and_reports_the_tracing_tax(tmp_path):
    from research_b200.runtime.profile_analysis import (analyze_profile_root, format_profile_analysis, layout_name,
                                                        model_signature, profile_analysis_to_json, relative_delta)

    _structured_run(tmp_path, "a-plain", optimizer="adamw", parallelism={"mode": "ddp"}, step=0.4)
    _structured_run(tmp_path, "b-tensor", optimizer="adamw", parallelism={"mode": "ddp", "tensor_parallel": True}, step=0.5)
    _structured_run(tmp_path, "c-tensor-ns", optimizer="muon", parallelism={"mode": "ddp", "tensor_parallel": True}, step=0.6)
    _structured_run(tmp_path, "d-sharded", optimizer="adamw", parallelism={"mode": "fsdp", "tensor_parallel": True}, step=0.55)
    _structured_run(tmp_path, "e-other-net", optimizer="muon", parallelism={"mode": "ddp", "tensor_parallel": True},
                    hidden=128)
    traced = tmp_path / "a-plain" / "diagnostics" / "profiling.json"
    traced.write_text(json.dumps({"enabled": True, "trace_start_step": 2, "trace_end_step": 3}))
    rows = [json.loads(l) for l in (tmp_path / "a-plain" / "metrics" / "train.jsonl").read_text().splitlines()]
    rows[1]["train_step_sec"] = rows[2]["train_step_sec"] = 0.6                      # the traced steps run slower
    (tmp_path / "a-plain" / "metrics" / "train.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    out = analyze_profile_root(tmp_path, warmup_steps=1)
    pairs = {(p["kind"], p["candidate"], p["baseline"]): p for p in out["comparisons"]}
    assert set(pairs) == {("layout", "b-tensor", "a-plain"), ("layout", "d-sharded", "b-tensor"),
                          ("optimizer", "c-tensor-ns", "b-tensor")}           # the other network pairs with nothing
    assert pairs[("optimizer", "c-tensor-ns", "b-tensor")]["train_step_delta"] == pytest.approx(0.2)
    assert pairs[("layout", "b-tensor", "a-plain")]["train_step_delta"] == pytest.approx(0.25)
    plain = out["runs"][0]
    assert plain["layout"] == "ddp" and out["runs"][3]["layout"] == "fsdp+tp" and plain["status"] == "completed"
    assert plain["trace_window"]["row_count"] == 2 and plain["steady"]["start_step"] == 4
    assert plain["trace_window"]["tax"]["train_step_sec"] == pytest.approx(0.5)
    assert out["runs"][1]["trace_window"]["tax"] is None and plain["hlo"] is None
    trace = plain["trace"]
    assert trace["trace"] == "step.trace.json.gz" and trace["event_count"] == 2       # the malformed event is skipped
    assert trace["gpu_time_us"] == {"gemm": 30.0, "memcpy": 10.0} and trace["max_kernel_us"]["gemm"] == 30.0
    text = format_profile_analysis(out)
    assert "profile analysis: runs=5" in text and "paired deltas:" in text and "traced steps 2-3: train +50.0%" in text
    assert "optimizer c-tensor-ns vs b-tensor: train=+20.0%" in text and "gpu time: gemm=75% memcpy=25%" in text
    assert json.loads(profile_analysis_to_json(out))["run_count"] == 5
    assert model_signature({"a": 1, "variant": "x", "remat": "full"}) == '{"a":1}' and model_signature(None) == "unknown"
    assert layout_name({"parallelism": {"mode": "zero2", "tensor_parallel": True, "expert_parallel": True}}) == "zero2+tp+ep"
    assert layout_name({}) == "ddp"
    assert relative_delta(3.0, 2.0) == pytest.approx(0.5) and relative_delta(1.0, 0) is None and relative_delta(None, 1.0) is None


def test_profile_analysis_refuses_unfinished_or_nonfinite_runs(tmp_path):
    from research_b200.runtime.profile_analysis import analyze_profile_root

    _structured_run(tmp_path / "one", "failed-run", optimizer="adamw", parallelism={"mode": "ddp"}, status="failed")
    with pytest.raises(ContractError, match="is not completed: status='failed'"):
        analyze_profile_root(tmp_path / "one")
    _structured_run(tmp_path / "two", "nan-run", optimizer="adamw", parallelism={"mode": "ddp"}, nonfinite=2)
    with pytest.raises(ContractError, match="contains nonfinite optimizer groups"):
        analyze_profile_root(tmp_path / "two")
    run = _structured_run(tmp_path / "three", "bad-trace", optimizer="adamw", parallelism={"mode": "ddp"})
    (run / "profiles" / "broken.json").write_text("{not json")
    with pytest.raises(ContractError, match="failed to read trace"):
        analyze_profile_root(tmp_path / "three")


def test_streaming_data_through_preflight_training_and_resume(tmp_path, monkeypatch):
    """``data.mode = "hf_streaming"`` end to end with a fake dataset and tokenizer: the dataset state rides in the
    checkpoint and a resumed run sees the rows a straight run sees."""

    import research_b200.data.prepare as prepare
    import research_b200.data.streaming as streaming
    from research_b200.runtime.preflight import run_preflight
    from research_b200.runtime.training import run_training

    rows = [{"text": f"document {i} says hello to the world " * 3} for i in range(400)]
    monkeypatch.setattr(streaming, "load_hf_dataset", lambda source: FakeIterableDataset(rows))
    monkeypatch.setattr(prepare, "load_tokenizer", lambda name: FakeTokenizer())
    manifest = tiny_dataset(tmp_path)

    def config(run_id, steps):
        raw = tiny_raw_config(manifest, run_id=run_id, output_dir=(tmp_path / "runs").as_posix(), steps=steps,
                              checkpoint_every=2)
        raw["data"] = {"mode": "hf_streaming", "tokenizer_id": "fake", "order": "sequential",
                       "hf_streaming": {"dataset": "corp/us", "split": "train", "revision": "abc"}}
        return write_toml(raw, tmp_path / f"{run_id}.toml")

    report = run_preflight(config("pre", 4))
    assert report["data"]["mode"] == "hf_streaming" and report["data"]["train_split_tokens"] is None
    assert report["data"]["pipeline"]["exact_resume"] is True and report["first_batch"]["target_tokens"] == 128
    straight = run_training(config("straight", 6))
    first = run_training(config("halves", 4))
    assert first.data_pipeline_backend == "hf_streaming" and first.data_document_aware is False
    second = run_training(config("halves", 6), resume=True)
    assert second.steps == 6 and second.final_loss == pytest.approx(straight.final_loss, rel=1e-6)

    def rows_of(run_id):
        path = tmp_path / "runs" / run_id / "metrics" / "train.jsonl"
        return [json.loads(line) for line in path.read_text().splitlines()]

    a, b = rows_of("straight"), rows_of("halves")
    assert [(r["step"], r["token_start"], r["token_end"]) for r in b] == [(r["step"], r["token_start"], r["token_end"]) for r in a]
    assert [r["loss"] for r in b] == pytest.approx([r["loss"] for r in a], rel=1e-6)
    ck = LocalCheckpointRestoreProbe(tmp_path / "runs" / "halves")
    assert ck["backend"] == "hf_streaming" and ck["stream_state"]["tokens_emitted"] == 6 * 128


def LocalCheckpointRestoreProbe(run_dir):
    """The dataset state stored with the newest checkpoint of a run."""

    from research_b200.services.checkpoints import LocalCheckpointService

    return LocalCheckpointService(run_dir, is_writer=False).restore_latest().dataset_state
