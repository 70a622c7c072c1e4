"""Collectives on 2, 3 and 4 CPU processes against locally computed values.
Integer-valued inputs make every sum exact, so comparisons are bit for bit;
64-byte slots force each message through many rounds and slot reuse.
Parity: tests/test_comm.py:19-112 of the reference."""

import pytest
import torch

from tandem_b200 import CommError, launch

SIZES = [0, 1, 5, 64, 1000, 4099]
DTYPES = (torch.float32, torch.float64, torch.bfloat16, torch.float16, torch.int64, torch.int32)


def data(rank, n, dtype, seed=0):
    g = torch.Generator().manual_seed(seed * 1000 + rank)
    hi = 30 if dtype in (torch.bfloat16, torch.float16) else 100
    return torch.randint(-hi, hi, (n,), generator=g).to(dtype)


def collectives(g):
    r, w = g.rank, g.size
    for dtype in DTYPES:
        for n in SIZES:
            want = sum(data(q, n, dtype).double() for q in range(w))
            x = data(r, n, dtype)
            assert g.all_reduce(x) is x
            assert torch.equal(x.double(), want), ("all_reduce", dtype, n)

            sizes = [n // w] * w  # uneven, rotated, one possibly empty
            sizes[-1] += n - sum(sizes)
            sizes = sizes[1:] + sizes[:1]
            lo = sum(sizes[:r])
            x = data(r, n, dtype)
            mine = g.reduce_scatter(x, sizes)
            assert mine.data_ptr() == x[lo:].data_ptr() or mine.numel() == 0
            assert torch.equal(mine.double(), want[lo:lo + sizes[r]]), ("reduce_scatter", dtype, n)

            x = data(r, n, dtype)
            mine = g.reduce_scatter(x)
            even = [len(c) for c in torch.tensor_split(torch.empty(n), w)]
            elo = sum(even[:r])
            assert torch.equal(mine.double(), want[elo:elo + even[r]]), ("reduce_scatter even", dtype, n)

            full = want.to(dtype)
            x = torch.full((n,), -7, dtype=dtype)
            x[lo:lo + sizes[r]] = full[lo:lo + sizes[r]]
            g.all_gather(x, sizes)
            assert torch.equal(x, full), ("all_gather", dtype, n)

            x = data(r, n, dtype, seed=1)
            g.broadcast(x, root=w - 1)
            assert torch.equal(x, data(w - 1, n, dtype, seed=1)), ("broadcast", dtype, n)

    x = data(r, 37, torch.float32)
    g.all_reduce(x, op="avg")
    want = sum(data(q, 37, torch.float32).double() for q in range(w)) / w
    assert torch.allclose(x.double(), want, rtol=0, atol=1e-5)
    return r


@pytest.mark.parametrize("world", [1, 2, 3, 4])
def test_collectives(world):
    assert launch(collectives, world, slot_bytes=64) == list(range(world))


def ring_order(g):
    """Non-associative data: the result must be the left fold over ranks
    c+1, c+2, ..., c for chunk c, which is what a ring reduce-scatter computes."""
    n, w = 1001, g.size
    xs = [torch.randn(n, generator=torch.Generator().manual_seed(q)) * 10 ** (q % 3) for q in range(w)]
    x = xs[g.rank].clone()
    g.all_reduce(x, op="avg")
    want = torch.empty(n)
    lo = 0
    for c, chunk in enumerate(torch.tensor_split(torch.arange(n), w)):
        k = len(chunk)
        acc = xs[(c + 1) % w][lo:lo + k] / w
        for j in range(2, w + 1):
            acc = acc + xs[(c + j) % w][lo:lo + k] / w
        want[lo:lo + k] = acc
        lo += k
    assert torch.equal(x, want)
    return True


@pytest.mark.parametrize("world", [2, 3, 4])
def test_fold_order_is_the_ring_order(world):
    assert all(launch(ring_order, world, slot_bytes=256))


def async_order(g):
    xs = [data(g.rank, 3000 + k, torch.float32, seed=k) for k in range(5)]
    works = [g.all_reduce(x, async_op=True) for x in xs]
    busy = torch.randn(200, 200) @ torch.randn(200, 200)
    for k, (x, wk) in enumerate(zip(xs, works)):
        assert wk.wait() is x
        assert wk.is_completed()
        want = sum(data(q, 3000 + k, torch.float32, seed=k) for q in range(g.size))
        assert torch.equal(x, want)
    return float(busy.sum())


def test_async_collectives_complete_in_submission_order():
    assert len(launch(async_order, 3, slot_bytes=256)) == 3


def ping_pong(g):
    other = 1 - g.rank
    x = torch.arange(10_000, dtype=torch.float32) * (g.rank + 1)
    y = torch.empty_like(x)
    for _ in range(3):
        if g.rank == 0:
            g.send(x, other)
            g.recv(y, other)
        else:
            g.recv(y, other)
            g.send(x, other)
        assert torch.equal(y, torch.arange(10_000, dtype=torch.float32) * (other + 1))
    z = torch.empty_like(x)
    g.sendrecv(x, other, z, other)
    assert torch.equal(z, y)
    return True


def test_send_recv_and_sendrecv():
    assert launch(ping_pong, 2, slot_bytes=512) == [True, True]


def failing(g):
    if g.rank == 1:
        raise ValueError("boom")
    return True


def test_a_failing_rank_fails_the_launch():
    with pytest.raises(Exception, match="boom"):
        launch(failing, 2)


def bad_calls(g):
    seen = []
    for call in (lambda: g.all_reduce(torch.zeros(4, 4).t()),
                 lambda: g.all_reduce(torch.zeros(4), op="max"),
                 lambda: g.reduce_scatter(torch.zeros(5), sizes=[1, 1]),
                 lambda: g.all_reduce(torch.zeros(4, dtype=torch.int64), op="avg"),
                 lambda: g.broadcast(torch.zeros(4), root=9)):
        try:
            call()
            seen.append(False)
        except CommError:
            seen.append(True)
    def job():
        raise KeyError("inside the job")
    try:
        g.submit("job", job)
        seen.append(False)
    except CommError as e:
        seen.append("inside the job" in str(e))
    assert g.submit("ok", lambda: 41 + 1) == 42
    return seen


def test_misuse_raises_comm_error():
    assert launch(bad_calls, 2) == [[True] * 6] * 2
