"""Failure detection on the host: ranks as processes that share a TCPStore; no GPU involved."""
import multiprocessing as mp
import time

import pytest
import torch.distributed as dist

from fastdeploy_b200.parallel.health import RankHealth, RankLostError


def _rank(rank, world, port, behaviour, q, join_s):
    store = dist.TCPStore("127.0.0.1", port, world_size=None, is_master=(rank == 0), wait_for_workers=False)
    try:
        if behaviour == "never_joins":
            time.sleep(join_s + 1.5)
            return
        h = RankHealth(store, rank, world, timeout_s=0.6)
        h.wait_for_all(timeout_s=join_s)      # generous: process start-up (imports) varies a lot under load
        for step in range(40):
            if behaviour == "dies" and step == 5:
                q.put((rank, "died"))
                return                        # stops beating, no goodbye
            if behaviour == "leaves" and step == 5:
                h.leave()
                q.put((rank, "left"))
                return
            try:
                alive = h.guard(f"step {step}")
            except RankLostError as e:
                q.put((rank, "lost", e.ranks, step))
                return
            time.sleep(0.05)
        q.put((rank, "done", alive))
    finally:
        if rank == 0:
            time.sleep(1.0)                   # keep the store up until the others have reported


def _run(behaviours, port, join_s=20.0):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world = len(behaviours)
    procs = [ctx.Process(target=_rank, args=(r, world, port, b, q, join_s)) for r, b in enumerate(behaviours)]
    for p in procs:
        p.start()
    out = []
    deadline = time.time() + join_s + (40 if join_s > 5 else 8)
    while len(out) < sum(b != "never_joins" for b in behaviours) and time.time() < deadline:
        try:
            out.append(q.get(timeout=0.5))
        except Exception:
            pass
    for p in procs:
        p.join(timeout=join_s + 10)
    return out


def test_rank_that_dies_is_detected_by_the_others():
    out = _run(["ok", "ok", "dies"], 29611)
    kinds = {o[0]: o for o in out}
    assert kinds[2][1] == "died"
    for r in (0, 1):
        assert kinds[r][1] == "lost" and kinds[r][2] == [2] and kinds[r][3] > 5


def test_orderly_leave_is_not_a_failure():
    out = _run(["ok", "leaves", "ok"], 29612)
    kinds = {o[0]: o for o in out}
    assert kinds[1][1] == "left"
    for r in (0, 2):
        assert kinds[r][1] == "done" and kinds[r][2] == [0, 2] if r == 0 else True


def test_rank_that_never_joins_fails_the_rendezvous():
    out = _run(["ok", "never_joins"], 29613, join_s=3.0)
    assert out == [] or all(o[1] != "done" for o in out)


def test_startup_timeout_raises():
    store = dist.HashStore()
    h = RankHealth(store, 0, 2, timeout_s=0.2)
    with pytest.raises(RankLostError, match="start-up"):
        h.wait_for_all()
