"""Rank-level failure detection for one-process-per-GPU runs.

The reference is a single process and detects failure by failing loudly with durable events (``training_failed``,
``checkpoint_restore_failed``, ``optimizer_nonfinite``...; src/jaxtitan/runtime/training.py:258-266, 453-471) and
recovers with ``run train --resume``.  With several processes two more things can go wrong: a rank dies or stops
making progress, and the others would wait in a collective.  Each rank therefore writes a heartbeat file
(step, wall time, phase) from the host between steps, and a watchdog - polled on the host before the next launch,
never from inside a kernel - reports ranks whose heartbeat is older than a limit, so the job stops with a
``rank_heartbeat_lost`` event instead of hanging.  Device-side waits are bounded separately (status word read by
``native.check_status``).

:class:`RankMonitor` is what the training loop runs: heartbeats go to the process group's key-value store (and to
the heartbeat files, for a post-mortem), a rank that leaves through an exception marks itself failed there, every
rank checks the marks on the host before it launches its next step, and a polling thread covers the case where the
main thread already sits in a collective: it records the ``rank_lost`` event and, after a grace period, ends the
process so that the launcher can tear the job down.
"""

from __future__ import annotations

import json
import os
import time
import sys
import threading
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


class RankMonitor:
    """Heartbeats and failure marks of all ranks in the process group's store.

    ``beat`` after every step; ``check`` on the host before the next launch (raises when a peer has marked itself
    failed or its heartbeat is older than ``timeout_s``); ``mark_failed`` from the exception path of a rank that
    leaves; ``start`` runs the polling thread.  ``abort`` is what the thread calls ``grace_s`` after it saw a lost
    rank if the process is still alive (default: exit code 70)."""

    def __init__(self, store, rank: int, world: int, *, directory: str | Path | None = None, writer=None,
                 run_id: str = "", timeout_s: float = 300.0, poll_s: float = 2.0, grace_s: float = 15.0, abort=None):
        self.store, self.rank, self.world = store, rank, world
        self.writer, self.run_id = writer, run_id
        self.timeout_s, self.poll_s, self.grace_s = timeout_s, poll_s, grace_s
        self.files = HeartbeatWriter(directory, rank) if directory is not None else None
        self.abort = abort or (lambda: os._exit(70))
        self.lost: list[dict] = []
        self._reported = False
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._lock = threading.Lock()
        self.beat(0, "init")

    def _key(self, rank: int) -> str:
        return f"research_b200/heartbeat/{self.run_id}/{rank}"

    def _set(self, payload: dict) -> None:
        self.store.set(self._key(self.rank), json.dumps(payload))

    def beat(self, step: int, phase: str = "step") -> None:
        self._set({"rank": self.rank, "step": int(step), "phase": phase, "wall_time": time.time(), "pid": os.getpid()})
        if self.files is not None:
            self.files.beat(step, phase)

    def mark_failed(self, step: int, error: str) -> None:
        try:
            self._set({"rank": self.rank, "step": int(step), "phase": "failed", "wall_time": time.time(),
                       "pid": os.getpid(), "error": error[:500]})
        except Exception:  # noqa: BLE001 - the store may be gone already; the others then see a stale heartbeat
            pass

    def mark_done(self, step: int) -> None:
        self.beat(step, "done")

    def peers(self) -> dict[int, dict]:
        out = {}
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                if not self.store.check([self._key(r)]):
                    continue
                out[r] = json.loads(self.store.get(self._key(r)).decode())
            except Exception:  # noqa: BLE001 - unreadable entry: treated as "no heartbeat yet"
                continue
        return out

    def lost_ranks(self, now: float | None = None) -> list[dict]:
        now = time.time() if now is None else now
        lost = []
        for r, hb in sorted(self.peers().items()):
            if hb.get("phase") == "failed":
                lost.append({"rank": r, "reason": "failed", "step": hb.get("step"), "error": hb.get("error")})
            elif hb.get("phase") != "done" and now - float(hb.get("wall_time", now)) > self.timeout_s:
                lost.append({"rank": r, "reason": "stale_heartbeat", "step": hb.get("step"),
                             "age_s": now - float(hb["wall_time"])})
        return lost

    def _report(self, lost: list[dict]) -> None:
        with self._lock:
            if self._reported:
                return
            self._reported = True
            self.lost = lost
        if self.writer is not None:
            from research_b200.services.artifacts import utc_now

            self.writer.append_event({"schema_version": 1, "type": "rank_lost", "run_id": self.run_id,
                                      "created_at": utc_now(), "observed_by_rank": self.rank, "ranks": lost})

    def check(self) -> None:
        """Host-side check before a launch: raises when a peer is lost (the event is written once)."""

        lost = self.lost or self.lost_ranks()
        if lost:
            self._report(lost)
            raise ContractError(f"rank(s) {[item['rank'] for item in lost]} left the job: {lost}")

    def _poll(self) -> None:
        while not self._stop.wait(self.poll_s):
            try:
                lost = self.lost_ranks()
            except Exception:  # noqa: BLE001 - store unreachable: rank 0 (its host) is gone
                lost = [{"rank": 0, "reason": "store_unreachable"}]
            if not lost:
                continue
            self._report(lost)
            if self._stop.wait(self.grace_s):
                return               # the main thread noticed and is shutting down in an orderly way
            print(f"research_b200: rank {self.rank}: peers lost ({lost}); the main thread is still blocked after "
                  f"{self.grace_s:.0f} s, ending the process", file=sys.stderr, flush=True)
            self.abort()
            return

    def start(self) -> "RankMonitor":
        if self._thread is None:
            self._thread = threading.Thread(target=self._poll, name="rank-monitor", daemon=True)
            self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=self.poll_s + 1.0)
            self._thread = None
