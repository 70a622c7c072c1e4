"""Failure detection, with every failure made on the host (CPU ranks): a rank that raises,
a rank that never joins a collective, a peer that is out of step.  Waits are bounded by the
group's timeout, and a failing rank wakes the others at once through the job-wide abort word."""

import time

import pytest
import torch

from tandem_b200 import CommError, Group, launch


def straggler(g):
    if g.rank == 1:
        time.sleep(0.2)
        raise RuntimeError("rank 1 gives up")
    t0 = time.monotonic()
    try:
        g.all_reduce(torch.ones(1000))  # rank 1 never joins
    except CommError as e:
        return ("failed while" in str(e) or "timed out" in str(e)), time.monotonic() - t0
    return False, 0.0


def test_peers_of_a_failed_rank_fail_fast_not_after_the_timeout():
    t0 = time.monotonic()
    with pytest.raises(CommError, match="rank 1 gives up"):
        launch(straggler, 3)
    assert time.monotonic() - t0 < 60  # the default timeout is 600 s


def silent_rank(g):
    """Rank 0 skips a collective the others run: they time out (short limit) instead of hanging."""
    if g.rank == 0:
        time.sleep(1.5)
        return "skipped"
    try:
        g.all_reduce(torch.ones(10))
    except CommError as e:
        return "timed out" in str(e)
    return False


def run_with_timeout(rank, size, job, q):
    g = Group(rank, size, "cpu", timeout=0.5, job=job)
    try:
        q.put((rank, silent_rank(g)))
    finally:
        g.abort()


def test_a_missing_rank_is_a_timeout_error():
    import multiprocessing as mp
    import uuid

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    job = uuid.uuid4().hex[:12]
    ps = [ctx.Process(target=run_with_timeout, args=(r, 2, job, q)) for r in range(2)]
    for p in ps:
        p.start()
    got = dict(q.get(timeout=60) for _ in range(2))
    for p in ps:
        p.join(30)
    assert got[0] == "skipped" and got[1] is True


def out_of_step(g):
    x = torch.zeros(100)
    try:
        if g.rank == 0:
            g.send(x, 1)
        else:
            g.recv(torch.zeros(50), 0)  # expects half of what arrives
    except CommError as e:
        return "out of step" in str(e)
    return g.rank == 0


def test_mismatched_point_to_point_sizes_are_detected():
    out = launch(out_of_step, 2, slot_bytes=1 << 16)
    assert out[1] is True


def closed_group(g):
    g.close()
    try:
        g.all_reduce(torch.ones(3))
    except CommError as e:
        return "closed" in str(e)
    return False


def test_a_closed_group_refuses_work():
    assert launch(closed_group, 2) == [True, True]
