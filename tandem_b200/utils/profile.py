"""Where a step's time goes on each rank: compute spans from the training
thread, communication spans from the collectives, the share of communication
the training thread actually waited for, and a Chrome trace of both.
Same functions and row schema as the reference's tandem/profile.py:14-93."""

import contextlib
import json
import time

import torch


class Timeline:
    """Named host-clock spans; on a GPU each end waits for the device first."""

    def __init__(self, enabled=True, device=None):
        self.enabled = enabled
        self.device = torch.device(device) if device is not None else None
        self.spans = []  # (name, start, end)

    def _settle(self):
        if self.device is not None and self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    @contextlib.contextmanager
    def span(self, name):
        if not self.enabled:
            yield
            return
        self._settle()
        begin = time.perf_counter()
        try:
            yield
        finally:
            self._settle()
            self.spans.append((name, begin, time.perf_counter()))


def _merged(intervals):
    out = []
    for s, e in sorted(intervals):
        if out and s <= out[-1][1]:
            out[-1][1] = max(out[-1][1], e)
        else:
            out.append([s, e])
    return out


def _overlap(a, b):
    """Total length of the intersection of two sets of intervals."""
    a, b = _merged(a), _merged(b)
    i = j = 0
    total = 0.0
    while i < len(a) and j < len(b):
        total += max(0.0, min(a[i][1], b[j][1]) - max(a[i][0], b[j][0]))
        if a[i][1] < b[j][1]:
            i += 1
        else:
            j += 1
    return total


def summarize(compute_spans, comm_spans, waits, step_time):
    """comm_s: time collectives ran; exposed_comm_s: the part of it during which
    the training thread was blocked in Work.wait (waiting while nothing is in
    flight is compute the collective depends on, and is not counted);
    overlap: share of communication hidden behind compute."""
    comm = sum(e - s for _, s, e, _ in comm_spans)
    exposed = _overlap([(s, e) for _, s, e in waits], [(s, e) for _, s, e, _ in comm_spans])
    return {
        "step_s": step_time,
        "compute_s": sum(e - s for _, s, e in compute_spans),
        "comm_s": comm,
        "exposed_comm_s": exposed,
        "overlap": max(0.0, 1 - exposed / comm) if comm > 0 else None,
        "comm_bytes": sum(b for *_, b in comm_spans),
    }


def chrome_trace(per_rank, path):
    """Writes chrome://tracing JSON.  per_rank: [(compute_spans, comm_spans)] on
    one clock; one process per rank, thread 0 compute, thread 1 communication."""
    starts = [s for comp, comm in per_rank for _, s, *_ in (*comp, *comm)]
    origin = min(starts) if starts else 0.0
    events = []
    for rank, (comp, comm) in enumerate(per_rank):
        events.append({"ph": "M", "pid": rank, "name": "process_name", "args": {"name": f"rank {rank}"}})
        events.append({"ph": "M", "pid": rank, "tid": 0, "name": "thread_name", "args": {"name": "compute"}})
        events.append({"ph": "M", "pid": rank, "tid": 1, "name": "thread_name", "args": {"name": "communication"}})
        for name, s, e in comp:
            events.append({"ph": "X", "pid": rank, "tid": 0, "name": name, "ts": (s - origin) * 1e6, "dur": (e - s) * 1e6})
        for name, s, e, nbytes in comm:
            events.append({"ph": "X", "pid": rank, "tid": 1, "name": name, "ts": (s - origin) * 1e6,
                           "dur": (e - s) * 1e6, "args": {"bytes": nbytes}})
    with open(path, "w") as f:
        json.dump({"traceEvents": events}, f)
