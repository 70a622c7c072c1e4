"""Property tests of the native CPU collectives: every rank of a small group runs as a thread of this process
(the engine's waits release the GIL), with slots far smaller than the messages so that every transfer is cut into
many pieces and the slot ring wraps.  Integer-valued data make sums exact in any order, so results are compared
with torch.equal, as the reference's collective tests do (tests/test_comm.py:19-56)."""

import os
import threading
import time

import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import HealthCheck, given, settings, strategies as st

from tandem_b200.comm import DTYPE_CODE
from tandem_b200.engine import lib

DTYPES = [torch.float32, torch.float64, torch.bfloat16, torch.float16, torch.int64, torch.int32, torch.uint8]
_serial = [0]


def run_ranks(n, slots, slot_bytes, body):
    """Runs body(engine, rank) on n threads, each with its own Engine; returns the results in rank order."""
    _serial[0] += 1
    job = f"prop{os.getpid()}x{_serial[0]}x{time.monotonic_ns() % 1_000_000}"
    out, errors = [None] * n, []

    def rank_main(r):
        try:
            e = lib().Engine(job, r, n, slots, slot_bytes, 20.0)
            e.connect()
            e.barrier().wait()  # as Group does: nobody leaves (and unlinks its regions) while a peer is still connecting
            out[r] = body(e, r)
            e.close()
        except BaseException as ex:  # reported below, in the main thread
            errors.append((r, repr(ex)))

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    assert not any(t.is_alive() for t in threads), "a rank is stuck"
    assert not errors, errors
    return out


def values(rank, numel, dtype, seed):
    g = torch.Generator().manual_seed(seed * 131 + rank)
    hi = 3 if dtype == torch.uint8 else (30 if dtype in (torch.bfloat16, torch.float16) else 100)
    lo = 0 if dtype == torch.uint8 else -hi
    return torch.randint(lo, hi, (numel,), generator=g).to(dtype)


def partition(draw, total, n):
    cuts = sorted(draw(st.lists(st.integers(0, total), min_size=n - 1, max_size=n - 1)))
    edges = [0, *cuts, total]
    return [b - a for a, b in zip(edges, edges[1:])]


@settings(max_examples=25, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(n=st.integers(2, 4), numel=st.integers(0, 3000), dtype=st.sampled_from(DTYPES), slots=st.integers(2, 4),
       slot_bytes=st.sampled_from([64, 256, 1024]), seed=st.integers(0, 1000), data=st.data())
def test_cpu_collectives_match_torch_for_any_shape(n, numel, dtype, slots, slot_bytes, seed, data):
    sizes = partition(data.draw, numel, n)
    root = data.draw(st.integers(0, n - 1))
    code = DTYPE_CODE[dtype]
    inputs = [values(r, numel, dtype, seed) for r in range(n)]
    total = sum(x.to(torch.float64) for x in inputs).to(dtype) if numel else torch.empty(0, dtype=dtype)
    offs = [sum(sizes[:r]) for r in range(n + 1)]

    def body(e, r):
        res = {}
        x = inputs[r].clone()
        e.all_reduce(x.data_ptr(), numel, code, False).wait()
        res["all_reduce"] = x
        x = inputs[r].clone()
        e.reduce_scatter(x.data_ptr(), numel, code, sizes, False).wait()
        res["reduce_scatter"] = x[offs[r]:offs[r + 1]].clone()
        x = torch.zeros(numel, dtype=dtype)
        x[offs[r]:offs[r + 1]] = total[offs[r]:offs[r + 1]]
        e.all_gather(x.data_ptr(), numel, code, sizes).wait()
        res["all_gather"] = x
        x = inputs[r].clone()
        e.broadcast(x.data_ptr(), numel, code, root).wait()
        res["broadcast"] = x
        e.barrier().wait()
        return res

    for r, res in enumerate(run_ranks(n, slots, slot_bytes, body)):
        assert torch.equal(res["all_reduce"], total), ("all_reduce", r)
        assert torch.equal(res["reduce_scatter"], total[offs[r]:offs[r + 1]]), ("reduce_scatter", r, sizes)
        assert torch.equal(res["all_gather"], total), ("all_gather", r, sizes)
        assert torch.equal(res["broadcast"], inputs[root]), ("broadcast", r, root)


@settings(max_examples=10, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(n=st.integers(2, 4), nbytes=st.integers(0, 5000), slot_bytes=st.sampled_from([64, 512]), rounds=st.integers(1, 4))
def test_ring_of_sendrecv_moves_every_payload(n, nbytes, slot_bytes, rounds):
    def body(e, r):
        got = []
        for k in range(rounds):
            out = torch.full((nbytes,), (r * 7 + k) % 251, dtype=torch.uint8)
            inp = torch.zeros(nbytes, dtype=torch.uint8)
            e.sendrecv(out.data_ptr(), nbytes, (r + 1) % n, inp.data_ptr(), nbytes, (r - 1) % n).wait()
            got.append(inp)
        return got

    for r, got in enumerate(run_ranks(n, 2, slot_bytes, body)):
        for k, inp in enumerate(got):
            assert torch.equal(inp, torch.full((nbytes,), (((r - 1) % n) * 7 + k) % 251, dtype=torch.uint8)), (r, k)
