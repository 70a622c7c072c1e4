"""The profiler's pure functions and the Chrome trace it writes (tandem/profile.py:61-93;
the reference unit-tests summarize in tests/test_comm.py:106-112)."""

import json
import time

from tandem_b200.profile import Timeline, chrome_trace, summarize


def test_summarize_counts_only_waits_that_overlap_communication():
    compute = [("forward", 0.0, 1.0), ("backward", 1.0, 3.0)]
    comm = [("all_reduce", 1.5, 2.5, 100), ("all_reduce", 2.5, 3.5, 50)]
    waits = [("all_reduce", 0.2, 0.4), ("all_reduce", 3.0, 3.5)]  # the first wait precedes any collective
    row = summarize(compute, comm, waits, 3.5)
    assert row["step_s"] == 3.5
    assert row["compute_s"] == 3.0
    assert row["comm_s"] == 2.0
    assert abs(row["exposed_comm_s"] - 0.5) < 1e-12
    assert abs(row["overlap"] - 0.75) < 1e-12
    assert row["comm_bytes"] == 150


def test_summarize_merges_overlapping_spans_and_handles_no_communication():
    comm = [("a", 0.0, 2.0, 1), ("b", 1.0, 3.0, 1)]  # two collectives in flight at once
    row = summarize([], comm, [("a", 0.5, 2.5)], 3.0)
    assert abs(row["exposed_comm_s"] - 2.0) < 1e-12  # the wait intersects the union [0, 3), once
    assert summarize([("f", 0, 1)], [], [], 1.0)["overlap"] is None


def test_timeline_records_named_spans_in_order_and_can_be_switched_off():
    tl = Timeline()
    with tl.span("F0"):
        time.sleep(0.002)
    with tl.span("B0"):
        pass
    assert [s[0] for s in tl.spans] == ["F0", "B0"]
    assert tl.spans[0][2] - tl.spans[0][1] >= 0.002 and tl.spans[0][2] <= tl.spans[1][1]
    off = Timeline(enabled=False)
    with off.span("x"):
        pass
    assert off.spans == []


def test_chrome_trace_schema(tmp_path):
    per_rank = [([("forward", 10.0, 10.5)], [("all_reduce", 10.2, 10.4, 4096)]),
                ([("forward", 10.1, 10.6)], [])]
    path = tmp_path / "trace.json"
    chrome_trace(per_rank, str(path))
    events = json.loads(path.read_text())["traceEvents"]
    meta = [e for e in events if e["ph"] == "M"]
    assert {(e["pid"], e["args"]["name"]) for e in meta if e["name"] == "process_name"} == {(0, "rank 0"), (1, "rank 1")}
    assert {(e["pid"], e["tid"], e["args"]["name"]) for e in meta if e["name"] == "thread_name"} == {
        (0, 0, "compute"), (0, 1, "communication"), (1, 0, "compute"), (1, 1, "communication")}
    spans = [e for e in events if e["ph"] == "X"]
    assert len(spans) == 3 and all(e["dur"] > 0 and e["ts"] >= 0 for e in spans)
    comm = [e for e in spans if e["tid"] == 1]
    assert comm[0]["name"] == "all_reduce" and comm[0]["args"] == {"bytes": 4096} and comm[0]["pid"] == 0
    first = min(e["ts"] for e in spans)
    assert first == 0  # times are microseconds from the earliest span
    assert abs(comm[0]["ts"] - 0.2e6) < 1 and abs(comm[0]["dur"] - 0.2e6) < 1
