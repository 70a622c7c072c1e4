"""Native host runtime: shared-memory regions and the SPSC channel.

Behavioural parity with the reference's tests/test_engine.py:56-207 (M0 shared
memory, M1 channel), written against tandem_b200._host."""

import multiprocessing as mp
import os
import time
import zlib

import pytest

from tandem_b200.engine import lib


def region(tag):
    return f"/tb2-test-{os.getpid()}-{tag}-{time.monotonic_ns()}"


def in_child(target, *args, timeout=60):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_call, args=(q, target, args))
    p.start()
    p.join(timeout)
    if p.is_alive():
        p.kill()
        raise AssertionError(f"{target.__name__} still running after {timeout}s")
    ok, value = q.get(timeout=5)
    assert ok, f"{target.__name__} raised in the child: {value}"
    return value


def _call(q, target, args):
    try:
        q.put((True, target(*args)))
    except BaseException as e:
        q.put((False, repr(e)))


# ------------------------------------------------------------------ shared memory
def _child_io(name):
    s = lib().SharedMemory.open(name)
    first = s.read(0, 5)
    s.write(100, b"child was here")
    return first, s.size, s.owner


def test_shm_new_region_is_zeroed_and_writable():
    s = lib().SharedMemory.create(region("rw"), 4096)
    assert s.size == 4096 and s.owner and not s.closed
    assert s.read(0, 32) == bytes(32)
    s.write(7, b"payload")
    assert s.read(7, 7) == b"payload"
    with pytest.raises(IndexError):
        s.read(4090, 16)
    s.close()
    assert s.closed


def test_shm_is_shared_between_processes():
    name = region("share")
    s = lib().SharedMemory.create(name, 8192)
    s.write(0, b"hello")
    first, size, owner = in_child(_child_io, name)
    assert (first, size, owner) == (b"hello", 8192, False)
    assert s.read(100, 14) == b"child was here"
    s.close()


def test_shm_creator_removes_the_name_but_mappings_survive():
    name = region("unlink")
    s = lib().SharedMemory.create(name, 4096)
    other = lib().SharedMemory.open(name)
    s.close()
    with pytest.raises(RuntimeError, match="shm_open"):
        lib().SharedMemory.open(name)
    other.write(0, b"z")
    assert other.read(0, 1) == b"z"
    other.close()


def test_shm_errors_name_the_failing_call():
    with pytest.raises(RuntimeError, match="shm_open"):
        lib().SharedMemory.open(region("absent"))
    name = region("dup")
    s = lib().SharedMemory.create(name, 4096)
    with pytest.raises(RuntimeError, match="shm_open"):
        lib().SharedMemory.create(name, 4096)
    s.close()


def test_shm_failed_create_leaves_no_name():
    name = region("huge")
    with pytest.raises(RuntimeError):
        lib().SharedMemory.create(name, 1 << 62)
    with pytest.raises(RuntimeError, match="shm_open"):
        lib().SharedMemory.open(name)


def test_shm_move_semantics():
    a, b = region("mv-a"), region("mv-b")
    r = lib()._move_check(a, b)
    assert r == {"source_emptied": True, "target_took_over": True, "assigned": True, "self_assign_safe": True}
    for name in (a, b):
        with pytest.raises(RuntimeError, match="shm_open"):
            lib().SharedMemory.open(name)


# ------------------------------------------------------------------ channel
def _msg(i):
    n = (i * 37) % 61 + 1
    return bytes((i + k) % 256 for k in range(n))


def _producer(name, count):
    c = lib().Channel.open(name)
    for i in range(count):
        c.send(_msg(i), timeout=30)
    return count


def _consumer(name, count):
    c = lib().Channel.open(name)
    crc = 0
    for i in range(count):
        got = c.recv(64, timeout=30)
        if got != _msg(i):
            return f"message {i} arrived as {got[:8]!r} ({len(got)} bytes)"
        crc = zlib.crc32(got, crc)
    return crc


def test_channel_roundtrip():
    c = lib().Channel.create(region("one"), 4, 64)
    assert (c.slots, c.slot_bytes) == (4, 64)
    for m in (b"a", b"hello", bytes(range(64)), b""):
        c.send(m)
        assert c.recv(64) == m


def test_channel_validation():
    e = lib()
    with pytest.raises(ValueError):
        e.Channel.create(region("zero"), 0, 64)
    c = e.Channel.create(region("val"), 2, 8)
    with pytest.raises(ValueError):
        c.send(b"123456789")
    c.send(b"12345678")
    with pytest.raises(ValueError):
        c.recv(4)
    assert c.recv(8) == b"12345678"  # the message that did not fit is still there
    name = region("plain")
    s = e.SharedMemory.create(name, 4096)
    with pytest.raises(RuntimeError):
        e.Channel.open(name)
    s.close()


def test_channel_blocks_until_timeout():
    c = lib().Channel.create(region("block"), 2, 8)
    t = time.monotonic()
    with pytest.raises(TimeoutError):
        c.recv(8, timeout=0.2)
    assert 0.15 < time.monotonic() - t < 2.0
    c.send(b"1")
    c.send(b"2")
    with pytest.raises(TimeoutError):
        c.send(b"3", timeout=0.2)
    assert c.recv(8) == b"1"
    c.send(b"3")
    assert [c.recv(8), c.recv(8)] == [b"2", b"3"]


@pytest.mark.parametrize("slots", [1, 4])
def test_channel_stress_between_processes(slots):
    name = region(f"many{slots}")
    keep = lib().Channel.create(name, slots, 64)
    count = 20_000
    ctx = mp.get_context("spawn")
    with ctx.Pool(2) as pool:
        r = pool.apply_async(_consumer, (name, count))
        s = pool.apply_async(_producer, (name, count))
        assert s.get(timeout=120) == count
        got = r.get(timeout=120)
    want = 0
    for i in range(count):
        want = zlib.crc32(_msg(i), want)
    assert got == want, got
    del keep
