"""Where a step's time goes on each rank.

Three inputs, all on the host's perf_counter clock: compute spans recorded by the
training thread through `Timeline`, communication spans recorded by the
collectives (`Group.trace`: name, start, end, bytes) and the intervals the
training thread spent blocked in `Work.wait` (`Group.waits`).  `summarize` turns
them into the row the benchmark driver prints; `chrome_trace` writes them as a
chrome://tracing / Perfetto file with one process per rank.  Function names, the
row's keys and the trace layout are those of the reference's tandem/profile.py:14-93;
the interval arithmetic here is a sweep over sorted endpoints.
"""

import json
import time

import torch


class _OpenSpan:
    """Context manager returned by Timeline.span: stamps both ends, after the device has caught up."""

    __slots__ = ("timeline", "name", "begin")

    def __init__(self, timeline, name):
        self.timeline, self.name, self.begin = timeline, name, None

    def __enter__(self):
        tl = self.timeline
        if tl.enabled:
            tl.settle()
            self.begin = time.perf_counter()
        return self

    def __exit__(self, *exc):
        tl = self.timeline
        if self.begin is not None:
            tl.settle()
            tl.spans.append((self.name, self.begin, time.perf_counter()))
        return False


class Timeline:
    """Named spans of the training thread: `with timeline.span("forward"): ...` appends
    (name, start, end) to `spans`.  With a CUDA device each end first waits for the device,
    so a span covers the work launched inside it; a disabled timeline records nothing."""

    def __init__(self, enabled=True, device=None):
        self.enabled = bool(enabled)
        self.device = None if device is None else torch.device(device)
        self.spans = []

    def settle(self):
        dev = self.device
        if dev is not None and dev.type == "cuda":
            torch.cuda.synchronize(dev)

    def span(self, name):
        return _OpenSpan(self, name)


def _time_where_both_active(first, second):
    """Total time during which at least one interval of `first` AND at least one of `second` is open.
    One pass over the sorted endpoints, keeping how many intervals of each set are open."""
    marks = []
    for which, group in enumerate((first, second)):
        for start, end in group:
            if end > start:
                marks.append((start, 1, which))
                marks.append((end, -1, which))
    marks.sort(key=lambda m: (m[0], m[1]))  # at equal times close before opening: touching intervals do not overlap
    depth = [0, 0]
    total, since = 0.0, None
    for at, step, which in marks:
        was_both = depth[0] > 0 and depth[1] > 0
        depth[which] += step
        now_both = depth[0] > 0 and depth[1] > 0
        if now_both and not was_both:
            since = at
        elif was_both and not now_both:
            total += at - since
    return total


def summarize(compute_spans, comm_spans, waits, step_time):
    """One row per rank and step:
      compute_s        time inside Timeline spans
      comm_s           time collectives ran (each span counted, even when several overlap)
      exposed_comm_s   time the training thread was blocked in Work.wait WHILE a collective was running;
                       waiting with nothing in flight is compute the collective depends on, not communication
      overlap          1 - exposed / comm: the share of communication hidden behind compute (None without any)
      comm_bytes       bytes the collectives moved
    """
    comm_s = 0.0
    comm_bytes = 0
    running = []
    for _name, start, end, nbytes in comm_spans:
        comm_s += end - start
        comm_bytes += nbytes
        running.append((start, end))
    blocked = [(start, end) for _name, start, end in waits]
    exposed = _time_where_both_active(blocked, running)
    compute_s = 0.0
    for _name, start, end in compute_spans:
        compute_s += end - start
    overlap = None if comm_s <= 0 else max(0.0, 1.0 - exposed / comm_s)
    return {"step_s": step_time, "compute_s": compute_s, "comm_s": comm_s, "exposed_comm_s": exposed,
            "overlap": overlap, "comm_bytes": comm_bytes}


_ROWS = ((0, "compute"), (1, "communication"))  # thread ids within a rank's process


def _trace_events(per_rank):
    origin = None
    for compute, comm in per_rank:
        for span in (*compute, *comm):
            origin = span[1] if origin is None else min(origin, span[1])
    origin = 0.0 if origin is None else origin

    def complete(rank, row, name, start, end, **extra):
        event = {"ph": "X", "pid": rank, "tid": row, "name": name, "ts": (start - origin) * 1e6, "dur": (end - start) * 1e6}
        event.update(extra)
        return event

    for rank, (compute, comm) in enumerate(per_rank):
        yield {"ph": "M", "pid": rank, "name": "process_name", "args": {"name": f"rank {rank}"}}
        for row, label in _ROWS:
            yield {"ph": "M", "pid": rank, "tid": row, "name": "thread_name", "args": {"name": label}}
        for name, start, end in compute:
            yield complete(rank, 0, name, start, end)
        for name, start, end, nbytes in comm:
            yield complete(rank, 1, name, start, end, args={"bytes": nbytes})


def chrome_trace(per_rank, path):
    """Writes {"traceEvents": [...]}: per_rank[r] = (compute_spans, comm_spans) of rank r, all on one clock.
    Rank r is process r with thread 0 "compute" and thread 1 "communication"; spans are complete ("X") events
    in microseconds from the earliest span, communication events carry args.bytes."""
    with open(path, "w") as f:
        json.dump({"traceEvents": list(_trace_events(per_rank))}, f)
