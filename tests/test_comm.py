"""Collectives between 1-4 CPU processes, checked against values every rank computes locally.

Operands are small integers stored in the dtype under test, so every sum is exact whatever the order of
additions and comparisons can be bit for bit; 64-byte slots cut each message into many rounds and make the
slot ring wrap.  Behaviours covered: the reference's tests/test_comm.py:19-112 (collective correctness over
dtypes and odd sizes incl. uneven and empty chunks, async ordering, point-to-point, error propagation) plus
the ring fold order on non-associative data and CommError on misuse."""

import itertools

import pytest
import torch

from tandem_b200 import CommError, launch

LENGTHS = (0, 1, 5, 64, 1000, 4099)
KINDS = (torch.float32, torch.float64, torch.bfloat16, torch.float16, torch.int64, torch.int32)


def operand(owner, length, kind, salt=0):
    """Rank `owner`'s input: integers small enough that sums over four ranks stay exact in 16-bit floats."""
    bound = 30 if kind in (torch.bfloat16, torch.float16) else 100
    gen = torch.Generator()
    gen.manual_seed(7919 * salt + owner + 1)
    return torch.randint(-bound, bound, (length,), generator=gen).to(kind)


def rotated_split(length, parts):
    """Uneven chunk sizes: floor(length / parts) each, the remainder on one chunk, rotated by one place
    (for short messages that leaves empty chunks)."""
    sizes = [length // parts] * parts
    sizes[-1] += length - sum(sizes)
    return sizes[1:] + sizes[:1]


def check_every_collective(group):
    me, world = group.rank, group.size
    for kind, length in itertools.product(KINDS, LENGTHS):
        inputs = [operand(q, length, kind) for q in range(world)]
        total = torch.stack([t.double() for t in inputs]).sum(0) if length else torch.zeros(0, dtype=torch.float64)
        label = (str(kind), length)

        buf = inputs[me].clone()
        assert group.all_reduce(buf) is buf, label
        assert torch.equal(buf.double(), total), ("all_reduce", *label)

        sizes = rotated_split(length, world)
        start = sum(sizes[:me])
        buf = inputs[me].clone()
        chunk = group.reduce_scatter(buf, sizes)
        assert chunk.numel() == sizes[me] and (chunk.numel() == 0 or chunk.data_ptr() == buf[start:].data_ptr()), label
        assert torch.equal(chunk.double(), total[start:start + sizes[me]]), ("reduce_scatter sizes", *label)

        even = [c.numel() for c in torch.tensor_split(torch.empty(length), world)]
        chunk = group.reduce_scatter(inputs[me].clone())
        first = sum(even[:me])
        assert torch.equal(chunk.double(), total[first:first + even[me]]), ("reduce_scatter even", *label)

        expected = total.to(kind)
        buf = torch.full((length,), -7, dtype=kind)
        buf[start:start + sizes[me]] = expected[start:start + sizes[me]]
        group.all_gather(buf, sizes)
        assert torch.equal(buf, expected), ("all_gather", *label)

        root = world - 1
        buf = operand(me, length, kind, salt=1)
        group.broadcast(buf, root=root)
        assert torch.equal(buf, operand(root, length, kind, salt=1)), ("broadcast", *label)

    mean_in = [operand(q, 37, torch.float32) for q in range(world)]
    buf = mean_in[me].clone()
    group.all_reduce(buf, op="avg")
    assert torch.allclose(buf.double(), torch.stack(mean_in).double().mean(0), rtol=0, atol=1e-5)
    return me


@pytest.mark.parametrize("world", [1, 2, 3, 4])
def test_collectives_are_exact_for_every_dtype_and_length(world):
    assert launch(check_every_collective, world, slot_bytes=64) == list(range(world))


def check_fold_order(group):
    """With data whose sums depend on the order of additions, chunk c must come out as the left fold over ranks
    c+1, c+2, ..., c (each operand divided first): what a ring reduce-scatter computes, and what keeps results
    bit-identical to the reference's engines."""
    length, world = 1001, group.size
    inputs = []
    for q in range(world):
        gen = torch.Generator()
        gen.manual_seed(q)
        inputs.append(torch.randn(length, generator=gen) * 10 ** (q % 3))
    buf = inputs[group.rank].clone()
    group.all_reduce(buf, op="avg")
    expected = torch.empty(length)
    at = 0
    for c, piece in enumerate(torch.tensor_split(torch.arange(length), world)):
        stop = at + piece.numel()
        order = [(c + j) % world for j in range(1, world + 1)]
        acc = inputs[order[0]][at:stop] / world
        for q in order[1:]:
            acc = acc + inputs[q][at:stop] / world
        expected[at:stop] = acc
        at = stop
    assert torch.equal(buf, expected)
    return True


@pytest.mark.parametrize("world", [2, 3, 4])
def test_fold_order_is_the_ring_order(world):
    assert all(launch(check_fold_order, world, slot_bytes=256))


def check_async_order(group):
    """Five all-reduces in flight while the caller computes something else: each handle's wait() returns its
    tensor, finished, with the right sum."""
    lengths = [3000 + k for k in range(5)]
    bufs = [operand(group.rank, n, torch.float32, salt=k) for k, n in enumerate(lengths)]
    handles = [group.all_reduce(b, async_op=True) for b in bufs]
    meanwhile = (torch.randn(200, 200) @ torch.randn(200, 200)).sum()
    for k, (buf, handle) in enumerate(zip(bufs, handles)):
        assert handle.wait() is buf and handle.is_completed()
        expected = torch.stack([operand(q, lengths[k], torch.float32, salt=k) for q in range(group.size)]).sum(0)
        assert torch.equal(buf, expected), k
    return float(meanwhile)


def test_async_collectives_complete_in_submission_order():
    assert len(launch(check_async_order, 3, slot_bytes=256)) == 3


def check_point_to_point(group):
    peer = 1 - group.rank
    ramp = torch.arange(10_000, dtype=torch.float32)
    mine, theirs = ramp * (group.rank + 1), ramp * (peer + 1)
    got = torch.empty_like(mine)
    for _ in range(3):  # rank 0 serves, rank 1 returns
        steps = (group.send, group.recv) if group.rank == 0 else (group.recv, group.send)
        for step in steps:
            step(mine if step == group.send else got, peer)
        assert torch.equal(got, theirs)
    both = torch.empty_like(mine)
    group.sendrecv(mine, peer, both, peer)
    assert torch.equal(both, theirs)
    return True


def test_send_recv_and_sendrecv():
    assert launch(check_point_to_point, 2, slot_bytes=512) == [True, True]


def rank_one_raises(group):
    if group.rank == 1:
        raise ValueError("boom")
    return True


def test_a_failing_rank_fails_the_launch():
    with pytest.raises(Exception, match="boom"):
        launch(rank_one_raises, 2)


def check_misuse(group):
    def raises_comm_error(call):
        try:
            call()
        except CommError:
            return True
        return False

    verdicts = [raises_comm_error(call) for call in (
        lambda: group.all_reduce(torch.zeros(4, 4).t()),                       # not contiguous
        lambda: group.all_reduce(torch.zeros(4), op="max"),                    # unknown op
        lambda: group.reduce_scatter(torch.zeros(5), sizes=[1, 1]),            # sizes do not partition the tensor
        lambda: group.all_reduce(torch.zeros(4, dtype=torch.int64), op="avg"),  # mean of integers
        lambda: group.broadcast(torch.zeros(4), root=9),                       # no such rank
    )]

    def broken_job():
        raise KeyError("inside the job")

    try:
        group.submit("job", broken_job)
        verdicts.append(False)
    except CommError as e:
        verdicts.append("inside the job" in str(e))
    assert group.submit("ok", lambda: 41 + 1) == 42
    return verdicts


def test_misuse_raises_comm_error():
    assert launch(check_misuse, 2) == [[True] * 6] * 2


def _pass_descriptors(g):
    """Every rank writes its rank into a temporary file and hands the open descriptor to every peer; then rank 1
    alone hands out a second file (the one-to-all form the multicast handle uses)."""
    import os
    import tempfile

    from tandem_b200.parallel.symm import swap_fds

    def scratch(text):
        fd, path = tempfile.mkstemp()
        os.unlink(path)
        os.write(fd, text.encode())
        return fd

    mine = scratch(f"rank {g.rank}")
    got = swap_fds(g.job, "t0", g.rank, g.size, g.barrier, 20.0, mine)
    assert sorted(got) == list(range(g.size))
    for q, fd in got.items():
        assert os.pread(fd, 64, 0).decode() == f"rank {q}"
        assert (fd == mine) == (q == g.rank)
    for fd in got.values():
        os.close(fd)
    special = scratch("from the root") if g.rank == 1 else None
    got = swap_fds(g.job, "t1", g.rank, g.size, g.barrier, 20.0, special, root=1)
    assert list(got) == [1]
    assert os.pread(got[1], 64, 0).decode() == "from the root"
    os.close(got[1])


def test_descriptors_travel_between_ranks():
    launch(_pass_descriptors, 3, device="cpu")
