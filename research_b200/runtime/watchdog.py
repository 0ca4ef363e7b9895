"""Rank-level failure detection for one-process-per-GPU runs.

The reference is a single process and detects failure by failing loudly with durable events (``training_failed``,
``checkpoint_restore_failed``, ``optimizer_nonfinite``...; src/jaxtitan/runtime/training.py:258-266, 453-471) and
recovers with ``run train --resume``.  With several processes two more things can go wrong: a rank dies or stops
making progress, and the others would wait in a collective.  Each rank therefore writes a heartbeat file
(step, wall time, phase) from the host between steps, and a watchdog - polled on the host before the next launch,
never from inside a kernel - reports ranks whose heartbeat is older than a limit, so the job stops with a
``rank_heartbeat_lost`` event instead of hanging.  Device-side waits are bounded separately (status word read by
``native.check_status``).
"""

from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass
from pathlib import Path

from research_b200.errors import ContractError


@dataclass(frozen=True)
class Heartbeat:
    rank: int
    step: int
    phase: str
    wall_time: float
    pid: int


class HeartbeatWriter:
    def __init__(self, directory: str | Path, rank: int):
        self.path = Path(directory) / f"heartbeat.rank{rank}.json"
        self.rank = rank
        self.path.parent.mkdir(parents=True, exist_ok=True)

    def beat(self, step: int, phase: str = "step", now: float | None = None) -> None:
        payload = {"rank": self.rank, "step": int(step), "phase": phase,
                   "wall_time": time.time() if now is None else now, "pid": os.getpid()}
        tmp = self.path.with_suffix(".tmp")
        tmp.write_text(json.dumps(payload))
        tmp.replace(self.path)


class Watchdog:
    """Reads every rank's heartbeat; ``check`` raises when one is missing for too long or has fallen behind."""

    def __init__(self, directory: str | Path, world_size: int, *, timeout_s: float = 300.0, max_step_lag: int = 2):
        self.directory = Path(directory)
        self.world_size = world_size
        self.timeout_s = timeout_s
        self.max_step_lag = max_step_lag
        self.started = time.time()

    def read(self) -> dict[int, Heartbeat]:
        out = {}
        for rank in range(self.world_size):
            path = self.directory / f"heartbeat.rank{rank}.json"
            try:
                raw = json.loads(path.read_text())
                out[rank] = Heartbeat(int(raw["rank"]), int(raw["step"]), str(raw["phase"]), float(raw["wall_time"]),
                                      int(raw["pid"]))
            except (OSError, ValueError, KeyError):
                continue
        return out

    def lost_ranks(self, now: float | None = None) -> list[dict]:
        now = time.time() if now is None else now
        beats = self.read()
        newest_step = max((b.step for b in beats.values()), default=0)
        lost = []
        for rank in range(self.world_size):
            b = beats.get(rank)
            if b is None:
                if now - self.started > self.timeout_s:
                    lost.append({"rank": rank, "reason": "no_heartbeat", "age_s": now - self.started})
            elif now - b.wall_time > self.timeout_s:
                lost.append({"rank": rank, "reason": "stale_heartbeat", "age_s": now - b.wall_time, "step": b.step})
            elif newest_step - b.step > self.max_step_lag and now - b.wall_time > self.timeout_s / 2:
                lost.append({"rank": rank, "reason": "step_lag", "lag": newest_step - b.step, "step": b.step})
        return lost

    def check(self, writer=None, run_id: str = "", now: float | None = None) -> None:
        lost = self.lost_ranks(now)
        if not lost:
            return
        if writer is not None:
            from research_b200.services.artifacts import utc_now

            writer.append_event({"schema_version": 1, "type": "rank_heartbeat_lost", "run_id": run_id,
                                 "created_at": utc_now(), "ranks": lost})
        raise ContractError(f"lost heartbeat of rank(s) {[item['rank'] for item in lost]}: {lost}")
