"""Failure detection on the host: heartbeats over a torch.distributed store, faults injected by the test."""
import os
import sys
import time

import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

from retinags_b200.parallel.watchdog import PeerFailure, Watchdog

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_silent_peer_is_detected():
    store = dist.HashStore()
    a = Watchdog(store, 0, 2, interval=0.05, timeout=0.4).start()
    b = Watchdog(store, 1, 2, interval=0.05, timeout=0.4).start()
    time.sleep(0.3)
    a.check(); b.check()          # both alive
    b.stop()                      # rank 1 goes silent (no kernel, no collective in flight)
    deadline = time.time() + 5
    while a.failed is None and time.time() < deadline:
        time.sleep(0.05)
    with pytest.raises(PeerFailure, match="rank 1"):
        a.check()
    a.stop()


def test_reported_failure_propagates_immediately():
    store = dist.HashStore()
    hits = []
    a = Watchdog(store, 0, 2, interval=0.05, timeout=60.0, on_failure=hits.append).start()
    b = Watchdog(store, 1, 2, interval=0.05, timeout=60.0).start()
    b.report_failure("ValueError: boom")
    deadline = time.time() + 5
    while a.failed is None and time.time() < deadline:
        time.sleep(0.05)
    with pytest.raises(PeerFailure, match="boom"):
        a.check()
    assert hits and "boom" in hits[0]
    a.stop(); b.stop()


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=30))
    wd = Watchdog(store, rank, world, interval=0.1, timeout=1.0).start()
    try:
        for step in range(100):
            wd.check()
            if rank == 1 and step == 3:
                raise RuntimeError("injected fault on rank 1")  # raised between steps
            time.sleep(0.1)
        result = "finished"
    except PeerFailure as exc:
        result = f"peer failure: {exc}"
    except RuntimeError as exc:
        wd.report_failure(repr(exc))
        result = "raised"
        time.sleep(1.0)  # keep the store reachable until the peers have read the report
    open(os.path.join(out_dir, f"r{rank}.txt"), "w").write(result)
    wd.stop()


@pytest.mark.timeout(120)
def test_rank_that_raises_stops_the_others(tmp_path):
    port = 29900 + os.getpid() % 90
    mp.spawn(_worker, args=(3, port, str(tmp_path)), nprocs=3, join=True)
    res = [open(os.path.join(tmp_path, f"r{r}.txt")).read() for r in range(3)]
    assert res[1] == "raised"
    assert res[0].startswith("peer failure") and "injected fault" in res[0]
    assert res[2].startswith("peer failure")


def test_rank_leaving_between_steps_is_noticed_by_training_ranks():
    """The scenario of the multi-GPU rank-loss test, on two gloo ranks: two real training steps, then the last rank leaves."""
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    port = 28100 + os.getpid() % 500
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   PYTHONPATH=root, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, os.path.join(root, "tests", "rank_loss_worker.py"), "--mode", "silent"],
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert [p.returncode for p in procs] == [0, 0], "\n".join(o[-2000:] for o in outs)
    assert "RANK_LOSS_DETECTED rank 0" in outs[0] and "no heartbeat" in outs[0]


def test_phase_timer_writes_a_chrome_trace(tmp_path):
    import json
    from retinags_b200.utils.profiler import PhaseTimer
    t = PhaseTimer("cpu", enabled=True)
    t.trace = True
    for _ in range(2):
        with t.phase("step"):
            with t.phase("forward"):
                time.sleep(0.002)
            with t.phase("backward"):
                time.sleep(0.001)
    path = str(tmp_path / "trace.json")
    t.export_chrome_trace(path, rank=3)
    ev = [e for e in json.load(open(path))["traceEvents"] if e["ph"] == "X"]
    assert [e["name"] for e in ev].count("forward") == 2 and all(e["pid"] == 3 for e in ev)
    step = [e for e in ev if e["name"] == "step"][0]
    fwd = [e for e in ev if e["name"] == "forward"][0]
    assert step["ts"] <= fwd["ts"] and fwd["ts"] + fwd["dur"] <= step["ts"] + step["dur"] + 1.0
    assert t.table(2)["forward"] >= 2.0
