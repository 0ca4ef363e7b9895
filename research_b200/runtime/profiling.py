"""Programmatic trace capture over a configured step window (reference: src/jaxtitan/runtime/profiling.py:15-166).

``[profiling] enabled`` starts a ``torch.profiler`` (Kineto) trace at ``trace_start_step`` and stops it after
``trace_end_step``; the Chrome / Perfetto JSON lands in ``<run>/profiles``; phase annotations (``data``,
``train_step``, ``eval``, ``checkpoint``...) are NVTX ranges + profiler record functions;
``diagnostics/profiling.json`` and ``profiling_trace_*`` events record the outcome.  Resuming past the window
is an error, as in the reference (profiling.py:37-45).
"""

from __future__ import annotations

from contextlib import contextmanager
from pathlib import Path
from typing import Any

import torch

from research_b200.config.specs import RunSpec
from research_b200.errors import ContractError
from research_b200.services.artifacts import utc_now


class ProfilingManager:
    def __init__(self, spec: RunSpec, run_dir: Path, writer, *, enabled: bool = True):
        self.spec = spec.profiling
        self.run_id = spec.run_id
        self.run_dir = Path(run_dir)
        self.writer = writer
        self.active = bool(self.spec.enabled and enabled)
        self._profiler = None
        self._status = "disabled" if not self.spec.enabled else "pending"
        self._trace_path: str | None = None

    def check_resume(self, step: int) -> None:
        if self.spec.enabled and step >= self.spec.trace_start_step:
            raise ContractError(
                f"profiling.trace_start_step={self.spec.trace_start_step} is not after resumed step {step}"
            )

    @contextmanager
    def annotate(self, name: str):
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(name)
        try:
            with torch.profiler.record_function(name):
                yield
        finally:
            if torch.cuda.is_available():
                torch.cuda.nvtx.range_pop()

    @contextmanager
    def step(self, step: int):
        if self.active and step == self.spec.trace_start_step:
            self._start(step)
        try:
            yield
        finally:
            if self.active and self._profiler is not None and step >= self.spec.trace_end_step:
                self._stop(step)

    def _start(self, step: int) -> None:
        try:
            activities = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                activities.append(torch.profiler.ProfilerActivity.CUDA)
            self._profiler = torch.profiler.profile(activities=activities)
            self._profiler.__enter__()
            self._status = "running"
            self.writer.append_event({"schema_version": 1, "type": "profiling_trace_started", "run_id": self.run_id,
                                      "created_at": utc_now(), "step": step})
        except Exception as exc:
            self._fail(step, exc)

    def _stop(self, step: int) -> None:
        try:
            self._profiler.__exit__(None, None, None)
            out = self.run_dir / "profiles" / f"trace_steps_{self.spec.trace_start_step}_{self.spec.trace_end_step}.json"
            if self.spec.create_perfetto_trace:
                self._profiler.export_chrome_trace(str(out))
                self._trace_path = out.relative_to(self.run_dir).as_posix()
            self._status = "completed"
            self.writer.append_event({"schema_version": 1, "type": "profiling_trace_completed", "run_id": self.run_id,
                                      "created_at": utc_now(), "step": step, "trace_path": self._trace_path})
        except Exception as exc:
            self._fail(step, exc)
        finally:
            self._profiler = None
            self._write()

    def _fail(self, step: int, exc: Exception) -> None:
        self._status = "failed"
        self._profiler = None
        self.writer.append_event({"schema_version": 1, "type": "profiling_trace_failed", "run_id": self.run_id,
                                  "created_at": utc_now(), "step": step, "error_type": type(exc).__name__,
                                  "error_message": str(exc)})
        self._write()

    def _write(self) -> None:
        self.writer.write_profiling_diagnostics(self.payload())

    def payload(self) -> dict[str, Any]:
        return {"schema_version": 1, "enabled": self.spec.enabled, "status": self._status,
                "trace_start_step": self.spec.trace_start_step, "trace_end_step": self.spec.trace_end_step,
                "trace_steps": self.spec.trace_steps, "trace_path": self._trace_path, "backend": "torch.profiler",
                "trace_dir": "profiles", "trace_files": [] if self._trace_path is None else [self._trace_path],
                "traced_step_range": {"start": self.spec.trace_start_step, "end": self.spec.trace_end_step},
                "create_perfetto_trace": self.spec.create_perfetto_trace,
                "create_perfetto_link": self.spec.create_perfetto_link}

    def finish(self) -> None:
        if self._profiler is not None:
            self._stop(self.spec.trace_end_step)
        elif self.spec.enabled and self.active:
            self._write()
