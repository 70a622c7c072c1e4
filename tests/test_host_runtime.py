"""The native host runtime's two lowest layers, driven through tandem_b200._host: named shared-memory regions
and the one-way message ring built on them.

Behaviours checked are those of the reference's milestones M0 and M1 (tests/test_engine.py:56-207): a region is
zeroed, shared by name, unlinked by its creator while live mappings survive, errors name the failing call, a
failed create leaves nothing behind, moves transfer ownership; a channel round-trips messages (also empty ones),
validates sizes, blocks until its timeout, and survives 20,000 variable-length messages between two processes
through rings of one and of four entries."""

import hashlib
import multiprocessing as mp
import os
import time

import pytest

from tandem_b200.engine import lib

SPAWN = mp.get_context("spawn")


@pytest.fixture
def fresh_name():
    """Makes names no other test or run can collide with."""
    made = []

    def make(tag):
        made.append(f"/tb2-test-{os.getpid()}-{tag}-{time.monotonic_ns()}")
        return made[-1]

    return make


def call_in_child(function, *args, limit=60):
    """function(*args) in a spawned process; its return value, or an AssertionError with what it raised."""
    mailbox = SPAWN.Queue()
    child = SPAWN.Process(target=_child_main, args=(mailbox, function, args))
    child.start()
    child.join(limit)
    if child.is_alive():
        child.kill()
        raise AssertionError(f"{function.__name__} was still running after {limit}s")
    worked, value = mailbox.get(timeout=5)
    assert worked, f"{function.__name__} raised in the child: {value}"
    return value


def _child_main(mailbox, function, args):
    try:
        mailbox.put((True, function(*args)))
    except BaseException as error:
        mailbox.put((False, repr(error)))


def assert_name_is_gone(name):
    with pytest.raises(RuntimeError, match="shm_open"):
        lib().SharedMemory.open(name)


# ---------------------------------------------------------------------------------------------- shared memory
class TestSharedMemory:
    def test_new_region_is_zeroed_and_bounds_checked(self, fresh_name):
        region = lib().SharedMemory.create(fresh_name("rw"), 4096)
        assert (region.size, region.owner, region.closed) == (4096, True, False)
        assert region.read(0, 32) == bytes(32)
        region.write(7, b"payload")
        assert region.read(7, 7) == b"payload"
        with pytest.raises(IndexError):
            region.read(4090, 16)
        with pytest.raises(IndexError):
            region.write(4095, b"xx")
        region.close()
        assert region.closed
        with pytest.raises(ValueError):
            region.read(0, 1)

    def test_two_processes_see_the_same_bytes(self, fresh_name):
        name = fresh_name("share")
        mine = lib().SharedMemory.create(name, 8192)
        mine.write(0, b"hello")
        assert call_in_child(_read_then_sign, name) == (b"hello", 8192, False)
        assert mine.read(100, 14) == b"child was here"
        mine.close()

    def test_creator_unlinks_the_name_and_live_mappings_survive(self, fresh_name):
        name = fresh_name("unlink")
        creator = lib().SharedMemory.create(name, 4096)
        guest = lib().SharedMemory.open(name)
        creator.close()
        assert_name_is_gone(name)
        guest.write(0, b"z")
        assert guest.read(0, 1) == b"z"
        guest.close()

    def test_errors_name_the_call_that_failed(self, fresh_name):
        assert_name_is_gone(fresh_name("absent"))
        name = fresh_name("twice")
        first = lib().SharedMemory.create(name, 4096)
        with pytest.raises(RuntimeError, match="shm_open"):
            lib().SharedMemory.create(name, 4096)
        first.close()

    def test_a_create_that_fails_leaves_no_name_behind(self, fresh_name):
        name = fresh_name("huge")
        with pytest.raises(RuntimeError):
            lib().SharedMemory.create(name, 1 << 62)
        assert_name_is_gone(name)

    def test_moves_hand_over_ownership(self, fresh_name):
        names = fresh_name("mv-a"), fresh_name("mv-b")
        observed = lib()._move_check(*names)
        assert observed and all(observed.values()), observed
        assert set(observed) == {"source_emptied", "target_took_over", "assigned", "self_assign_safe"}
        for name in names:  # both regions were owned by objects that are gone now
            assert_name_is_gone(name)


def _read_then_sign(name):
    region = lib().SharedMemory.open(name)
    seen = region.read(0, 5)
    region.write(100, b"child was here")
    return seen, region.size, region.owner


# ---------------------------------------------------------------------------------------------- channel
def message(k):
    """Message k of the stress stream: 1 to 64 bytes that depend on k."""
    length = 1 + (k * 29) % 64
    return hashlib.blake2b(k.to_bytes(4, "little"), digest_size=64).digest()[:length]


def _feed(name, count):
    ring = lib().Channel.open(name)
    for k in range(count):
        ring.send(message(k), timeout=30)
    return count


def _drain(name, count):
    ring = lib().Channel.open(name)
    digest = hashlib.blake2b()
    for k in range(count):
        got = ring.recv(64, timeout=30)
        if got != message(k):
            return f"message {k} arrived as {got[:8]!r} ({len(got)} bytes)"
        digest.update(got)
    return digest.hexdigest()


class TestChannel:
    def test_messages_round_trip_in_order(self, fresh_name):
        ring = lib().Channel.create(fresh_name("one"), 4, 64)
        assert (ring.slots, ring.slot_bytes) == (4, 64)
        for payload in (b"a", b"hello", bytes(range(64)), b""):
            ring.send(payload)
            assert ring.recv(64) == payload
        burst = [bytes([k]) * (k + 1) for k in range(4)]  # fills the ring, then empties it
        for payload in burst:
            ring.send(payload)
        assert [ring.recv(64) for _ in burst] == burst

    def test_sizes_are_validated(self, fresh_name):
        host = lib()
        with pytest.raises(ValueError):
            host.Channel.create(fresh_name("zero"), 0, 64)
        ring = host.Channel.create(fresh_name("val"), 2, 8)
        with pytest.raises(ValueError):
            ring.send(b"123456789")  # one byte more than an entry holds
        ring.send(b"12345678")
        with pytest.raises(ValueError):
            ring.recv(4)  # too small a buffer ...
        assert ring.recv(8) == b"12345678"  # ... leaves the message in the ring
        plain = fresh_name("plain")
        region = host.SharedMemory.create(plain, 4096)
        with pytest.raises(RuntimeError):
            host.Channel.open(plain)  # no channel header in there
        region.close()

    def test_full_and_empty_rings_block_until_the_timeout(self, fresh_name):
        ring = lib().Channel.create(fresh_name("block"), 2, 8)

        def timed_out_after(action):
            began = time.monotonic()
            with pytest.raises(TimeoutError):
                action()
            return time.monotonic() - began

        assert 0.15 < timed_out_after(lambda: ring.recv(8, timeout=0.2)) < 2.0
        ring.send(b"1")
        ring.send(b"2")
        assert 0.15 < timed_out_after(lambda: ring.send(b"3", timeout=0.2)) < 2.0
        assert ring.recv(8) == b"1"
        ring.send(b"3")
        assert [ring.recv(8), ring.recv(8)] == [b"2", b"3"]

    @pytest.mark.parametrize("entries", [1, 4])
    def test_twenty_thousand_messages_between_two_processes(self, fresh_name, entries):
        name = fresh_name(f"stream{entries}")
        keep_alive = lib().Channel.create(name, entries, 64)
        count = 20_000
        with SPAWN.Pool(2) as workers:
            reader = workers.apply_async(_drain, (name, count))
            writer = workers.apply_async(_feed, (name, count))
            assert writer.get(timeout=120) == count
            received = reader.get(timeout=120)
        expected = hashlib.blake2b()
        for k in range(count):
            expected.update(message(k))
        assert received == expected.hexdigest(), received
        del keep_alive
