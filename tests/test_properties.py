"""Property tests (hypothesis) of the host-side bookkeeping that every rank must compute identically:
chunk offsets, flat-buffer shard overlaps, the symmetric heap's allocator, pipeline schedules."""

import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings, strategies as st

from tandem_b200.parallel.pipeline import plan, split_units
from tandem_b200.parallel.symm import ALIGN, Heap, split_offsets
from tandem_b200.parallel.zero import FlatLayout


@given(numel=st.integers(0, 10_000), n=st.integers(1, 8))
def test_split_offsets_match_tensor_split(numel, n):
    offs = split_offsets(numel, n)
    want = [0]
    for c in torch.tensor_split(torch.empty(numel), n):
        want.append(want[-1] + c.numel())
    assert offs == want


@given(sizes=st.lists(st.integers(0, 500), min_size=1, max_size=8))
def test_split_offsets_with_explicit_sizes(sizes):
    offs = split_offsets(sum(sizes), len(sizes), sizes)
    assert offs[0] == 0 and offs[-1] == sum(sizes)
    assert [b - a for a, b in zip(offs, offs[1:])] == sizes


@given(shapes=st.lists(st.integers(1, 300), min_size=1, max_size=12), world=st.integers(1, 8), data=st.data())
def test_bucket_sizes_partition_every_flat_range(shapes, world, data):
    params = [torch.nn.Parameter(torch.empty(s)) for s in shapes]
    layouts = [FlatLayout(params, world, r) for r in range(world)]
    total = sum(shapes)
    assert [(l.lo, l.hi) for l in layouts] == list(zip(split_offsets(total, world), split_offsets(total, world)[1:]))
    a = data.draw(st.integers(0, total))
    b = data.draw(st.integers(a, total))
    sizes = layouts[0].bucket_sizes(a, b)
    assert sum(sizes) == b - a and all(s >= 0 for s in sizes)
    for r, l in enumerate(layouts):  # each rank's share is the overlap with its own shard
        assert sizes[r] == max(0, min(b, l.hi) - max(a, l.lo))
        assert l.bucket_sizes(a, b) == sizes  # every rank computes the same split


@settings(max_examples=60)
@given(ops=st.lists(st.one_of(st.tuples(st.just("take"), st.integers(1, 5000)), st.tuples(st.just("give"), st.integers(0, 30))),
                    min_size=1, max_size=60))
def test_heap_allocations_never_overlap_and_repeat_on_every_rank(ops):
    def replay(bases):
        h = Heap()
        h.add_segment(64 << 10, bases)
        live, trace = [], []
        for kind, v in ops:
            if kind == "take":
                got = h.take(v)
                trace.append(got)
                if got is not None:
                    live.append((got, (max(v, 1) + ALIGN - 1) // ALIGN * ALIGN))
            elif live:
                (seg, off), _ = live.pop(v % len(live))
                h.give(seg, off)
            spans = sorted((off, off + size) for (_, off), size in live)
            assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:])), "live blocks overlap"
            assert all(off % ALIGN == 0 and end <= (64 << 10) for off, end in spans)
        for (seg, off), _ in live:
            h.give(seg, off)
        assert h.free == [(0, 0, 64 << 10)]  # everything coalesces back into one block
        return trace

    # two ranks with different base addresses make the same decisions
    assert replay([0x1000_0000, 0x2000_0000]) == replay([0x7000_0000, 0x3000_0000])


@given(stages=st.integers(1, 6), m=st.integers(1, 12), schedule=st.sampled_from(["gpipe", "1f1b"]))
def test_pipeline_plans_are_consistent_across_stages(stages, m, schedule):
    plans = [plan(schedule, stages, r, m) for r in range(stages)]
    for r, acts in enumerate(plans):
        f = [a[1] for a in acts if a[0] == "F"]
        b = [a[1] for a in acts if a[0] == "B"]
        assert f == list(range(m)) and b == list(range(m))
        pos = {a: i for i, a in enumerate(acts) if a[0] in "FB"}
        assert all(pos[("F", i)] < pos[("B", i)] for i in range(m))
        if schedule == "1f1b":  # at most `stages - rank` activations are alive at once
            alive = peak = 0
            for a in acts:
                alive += (a[0] == "F") - (a[0] == "B")
                peak = max(peak, alive)
            assert peak <= min(stages - r, m)
    # every activation / gradient a stage sends is received by its neighbour, in the same order
    def count(acts, *names):
        return sum(a[0] in names for a in acts)

    for r in range(stages - 1):
        assert count(plans[r], "send_act", "send_act_recv_grad") == count(plans[r + 1], "recv_act", "send_grad_recv_act") == m
        assert count(plans[r + 1], "send_grad", "send_grad_recv_act") == count(plans[r], "recv_grad", "send_act_recv_grad") == m


@given(units=st.integers(1, 40), stages=st.integers(1, 8))
def test_split_units_is_an_even_contiguous_cover(units, stages):
    parts = split_units(units, stages)
    assert len(parts) == stages
    assert parts[0][0] == 0 and parts[-1][1] == units
    assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
    sizes = [hi - lo for lo, hi in parts]
    assert max(sizes) - min(sizes) <= 1 and sorted(sizes, reverse=True) == sizes  # the longer stages come first
