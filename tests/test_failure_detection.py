"""Failure detection on the host: step watchdog and store-based peer heartbeat.  Failures are
made on the host (a rank that stops, leaves or exits); nothing here touches a GPU."""
import io
import os
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from omegalax_b200.utils.failure import PeerFailure, PeerHeartbeat, PeerLeft, StepWatchdog


def test_watchdog_fires_only_when_steps_stop():
    fired = []
    buf = io.StringIO()
    wd = StepWatchdog(0.3, on_timeout=lambda step, late: fired.append((step, late)), poll_s=0.05, stream=buf).start()
    for s in range(5):
        time.sleep(0.1)
        wd.beat(s)
    assert not fired
    wd.pause()
    time.sleep(0.5)          # a long checkpoint write: deadline suspended
    wd.resume()
    assert not fired
    time.sleep(0.6)          # the loop hangs
    wd.stop()
    assert fired and fired[0][0] == 4 and fired[0][1] > 0.3
    assert "exceeded its deadline" in buf.getvalue()


def test_heartbeat_detects_silent_and_leaving_peers():
    store = dist.HashStore()
    a = PeerHeartbeat(0, 3, store, interval_s=0.05, max_age_s=0.4).start()
    b = PeerHeartbeat(1, 3, store, interval_s=0.05, max_age_s=0.4).start()
    c = PeerHeartbeat(2, 3, store, interval_s=0.05, max_age_s=0.4).start()
    a.wait_all_alive(5.0)
    for _ in range(5):
        time.sleep(0.1)
        a.check()            # everybody alive
    b.stop()                 # rank 1 goes silent without a word
    t0 = time.monotonic()
    with pytest.raises(PeerFailure) as ei:
        while time.monotonic() - t0 < 3.0:
            a.check()
            time.sleep(0.05)
    assert ei.value.ranks == [1] and not isinstance(ei.value, PeerLeft)
    c.leave()                # rank 2 leaves in order
    with pytest.raises(PeerLeft) as ei:
        a.check()
    assert ei.value.ranks == [2]
    a.stop()
    c.stop()


def _worker(rank, world, port, mode, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    hb = PeerHeartbeat(rank, world, interval_s=0.05, max_age_s=0.6).start()
    hb.wait_all_alive(20.0)
    result = "finished"
    try:
        for step in range(50):
            if rank == world - 1 and step == 3:
                # this rank goes away between steps, with nothing of its own in flight
                if mode == "leave":
                    hb.leave()
                    os._exit(0)
                os._exit(0)                      # "crash": no announcement
            deadline = time.monotonic() + 1.5    # learn about peers on the host before the next collective
            while time.monotonic() < deadline:
                hb.check()
                if step < 3 or rank == world - 1:
                    break
                time.sleep(0.05)
            if step >= 3:
                raise AssertionError("peer loss was not detected")
            t = torch.ones(4) * (rank + 1)
            dist.all_reduce(t)
    except PeerFailure as e:
        result = f"{type(e).__name__}:{e.ranks}:step{step}"
    with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
        f.write(result)
    # keep beating (rank 0 also hosts the store) until every survivor has written its result
    t_end = time.monotonic() + 10.0
    while time.monotonic() < t_end and not all(os.path.exists(os.path.join(out_dir, f"r{r}.txt")) for r in range(world - 1)):
        time.sleep(0.05)
    hb.stop()
    os._exit(0)   # the group has lost a member: skip the collective teardown


@pytest.mark.parametrize("mode", ["leave", "crash"])
def test_ranks_learn_of_a_lost_peer_before_the_next_collective(tmp_path, mode):
    import socket

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_worker, args=(3, port, mode, str(tmp_path)), nprocs=3, join=True)
    want = "PeerLeft" if mode == "leave" else "PeerFailure"
    for r in (0, 1):
        got = (tmp_path / f"r{r}.txt").read_text()
        assert got == f"{want}:[2]:step3", got
    assert not (tmp_path / "r2.txt").exists()
