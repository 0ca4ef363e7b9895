"""Rank-level failure detection in the training loop, on CPU ranks over gloo.

Failures are made on the host only: a rank raises between two steps (none of its collectives in flight), marks
itself failed in the process group's store, and the other ranks learn of it before their next launch.  No device is
involved, so nothing here can hang or fault a GPU."""

import json
import time

import pytest

from research_b200.errors import ContractError
from tests.helpers import run_gloo, tiny_dataset, tiny_raw_config, write_toml


class _FakeStore:
    """The three calls of a c10d store that the monitor uses."""

    def __init__(self):
        self.data = {}

    def set(self, key, value):
        self.data[key] = value.encode() if isinstance(value, str) else value

    def get(self, key):
        return self.data[key]

    def check(self, keys):
        return all(k in self.data for k in keys)


def test_monitor_sees_failed_and_stale_peers():
    from research_b200.runtime.watchdog import RankMonitor

    store = _FakeStore()
    events = []

    class Sink:
        def append_event(self, e):
            events.append(e)

    a = RankMonitor(store, 0, 3, writer=Sink(), run_id="r", timeout_s=10.0)
    b = RankMonitor(store, 1, 3, run_id="r", timeout_s=10.0)
    c = RankMonitor(store, 2, 3, run_id="r", timeout_s=10.0)
    for m in (a, b, c):
        m.beat(4)
    a.check()                                                    # everybody alive
    assert a.lost_ranks(now=time.time() + 11)[0]["reason"] == "stale_heartbeat"
    c.mark_done(5)                                               # a rank that finished is never "stale"
    assert [x["rank"] for x in a.lost_ranks(now=time.time() + 11)] == [1]
    b.mark_failed(4, "ValueError: boom")
    with pytest.raises(ContractError, match=r"rank\(s\) \[1\] left the job"):
        a.check()
    assert events[-1]["type"] == "rank_lost" and events[-1]["ranks"][0]["error"] == "ValueError: boom"
    with pytest.raises(ContractError):
        a.check()
    assert len(events) == 1                                      # reported once


def test_monitor_thread_reports_and_aborts_a_blocked_process():
    from research_b200.runtime.watchdog import RankMonitor

    store = _FakeStore()
    aborted = []
    a = RankMonitor(store, 0, 2, run_id="r", timeout_s=60.0, poll_s=0.05, grace_s=0.2, abort=lambda: aborted.append(1))
    b = RankMonitor(store, 1, 2, run_id="r")
    a.start()
    b.mark_failed(7, "gone")
    deadline = time.time() + 5.0
    while not aborted and time.time() < deadline:                # the "main thread" never calls check(): blocked
        time.sleep(0.05)
    a.stop()
    assert aborted and a.lost[0]["rank"] == 1 and a.lost[0]["step"] == 7


def _leaving_rank_job(rank, world, cfg):
    from research_b200.runtime.training import run_training

    def hook(trainer):
        fetch = trainer.next_accumulated_batch

        def wrapped():
            if trainer.step == 2:
                if rank == 1:
                    raise RuntimeError("rank 1 leaves between steps")
                time.sleep(1.5)          # the others reach their pre-launch check after rank 1 has left
            return fetch()

        trainer.next_accumulated_batch = wrapped

    try:
        run_training(cfg, trainer_hook=hook)
        return {"rank": rank, "outcome": "completed"}
    except Exception as exc:  # noqa: BLE001
        return {"rank": rank, "outcome": type(exc).__name__, "message": str(exc)}


def test_a_rank_that_leaves_between_steps_stops_the_others_before_their_next_launch(tmp_path, monkeypatch):
    monkeypatch.setenv("RESEARCH_B200_RANK_POLL_S", "0.2")
    manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, mesh={"data": 3}, parallelism={"mode": "ddp"}, steps=6, batch=6, run_id="leave",
                          output_dir=(tmp_path / "runs").as_posix())
    cfg = write_toml(raw, tmp_path / "leave.toml")
    results = run_gloo(3, _leaving_rank_job, str(cfg))
    by_rank = {r["rank"]: r for r in results}
    assert by_rank[1]["outcome"] == "RuntimeError"
    for r in (0, 2):
        assert by_rank[r]["outcome"] == "ContractError" and "left the job" in by_rank[r]["message"], by_rank[r]
    events = [json.loads(line) for line in (tmp_path / "runs" / "leave" / "events.jsonl").read_text().splitlines()]
    lost = next(e for e in events if e["type"] == "rank_lost")
    assert lost["ranks"][0]["rank"] == 1 and lost["ranks"][0]["reason"] == "failed"
    assert "rank 1 leaves" in lost["ranks"][0]["error"]
    assert events[-1]["type"] == "training_failed"
    train_rows = (tmp_path / "runs" / "leave" / "metrics" / "train.jsonl").read_text().splitlines()
    assert len(train_rows) == 2                                   # nobody launched a third step
    beats = sorted(p.name for p in (tmp_path / "runs" / "leave" / "diagnostics" / "heartbeats").iterdir())
    assert beats == ["heartbeat.rank0.json", "heartbeat.rank1.json", "heartbeat.rank2.json"]
