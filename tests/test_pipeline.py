"""GPipe and 1F1B against one process accumulating over the same micro-batches:
each stage computes per micro-batch what that process computes for its units,
with backwards in the same order, so losses and weights after AdamW must match
bit for bit for any number of stages.  Parity: tests/test_pipeline.py:61-76."""

import pytest
import torch

from tandem_b200 import launch
from tandem_b200.data import synthetic
from tandem_b200.model import GPT, loss_fn
from tandem_b200.pipeline import Pipeline, plan, split_units
from tandem_b200.profile import Timeline

from test_ddp import CFG

STEPS, BATCH, MICRO = 3, 12, 6


def stage_rank(g, schedule):
    torch.manual_seed(0)
    text = synthetic(20_000)
    model = GPT(CFG)
    tl = Timeline()
    pipe = Pipeline(model, g, MICRO, schedule, timeline=tl)
    opt = torch.optim.AdamW(pipe.parameters(), lr=3e-3, weight_decay=0.1, foreach=False)
    losses = []
    for step in range(STEPS):
        x, y = text.batch(step, BATCH, CFG.seq)
        loss = pipe.train_step(x, y)
        losses.append(None if loss is None else loss.item())
        opt.step()
        opt.zero_grad()
    names = [n for n, _, _ in tl.spans[: 2 * MICRO]]
    return losses, torch.cat([p.detach().reshape(-1) for p in pipe.parameters()]), names


def single():
    torch.set_num_threads(1)
    torch.manual_seed(0)
    text = synthetic(20_000)
    model = GPT(CFG)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3, weight_decay=0.1, foreach=False)
    losses = []
    for step in range(STEPS):
        x, y = text.batch(step, BATCH, CFG.seq)
        total = 0
        for xb, yb in zip(x.chunk(MICRO), y.chunk(MICRO)):
            loss = loss_fn(model(xb), yb) / MICRO
            loss.backward()
            total = total + loss.detach()
        losses.append(total.item())
        opt.step()
        opt.zero_grad()
    return losses, [torch.cat([p.detach().reshape(-1) for p in u.parameters()]) for u in model.units()]


@pytest.fixture(scope="module")
def accumulated():
    return single()


@pytest.mark.parametrize("schedule", ["gpipe", "1f1b"])
@pytest.mark.parametrize("stages", [2, 3, 4])
def test_bit_identical_to_accumulation(schedule, stages, accumulated):
    ours = launch(stage_rank, stages, schedule, slot_bytes=1024)
    ref_losses, ref_units = accumulated
    for r, (lo, hi) in enumerate(split_units(len(ref_units), stages)):
        assert torch.equal(ours[r][1], torch.cat(ref_units[lo:hi])), f"stage {r} weights differ"
    assert ours[-1][0] == ref_losses
    first = ours[0][2]  # the schedules really differ on stage 0
    if schedule == "gpipe":
        assert first == [f"F{i}" for i in range(MICRO)] + [f"B{i}" for i in range(MICRO)]
    else:
        warm = stages - 1
        assert first[: warm + 2] == [f"F{i}" for i in range(warm + 1)] + ["B0"]


def test_split_units_is_even_and_contiguous():
    assert split_units(4, 2) == [(0, 2), (2, 4)]
    assert split_units(26, 4) == [(0, 7), (7, 14), (14, 20), (20, 26)]
    assert split_units(3, 3) == [(0, 1), (1, 2), (2, 3)]


@pytest.mark.parametrize("schedule", ["gpipe", "1f1b"])
@pytest.mark.parametrize("stages,m", [(2, 4), (4, 6), (4, 2), (3, 1)])
def test_plans_pair_up(schedule, stages, m):
    """Every send has the matching receive on the neighbour, in the same order."""
    plans = [plan(schedule, stages, r, m) for r in range(stages)]
    for r in range(stages):
        fs = [a[1] for a in plans[r] if a[0] == "F"]
        bs = [a[1] for a in plans[r] if a[0] == "B"]
        assert fs == list(range(m)) and bs == list(range(m))

    def sends(r, what):  # activations sent down / gradients sent up, in order
        n = 0
        for a in plans[r]:
            if what == "act" and a[0] in ("send_act", "send_act_recv_grad"):
                n += 1
            if what == "grad" and a[0] in ("send_grad", "send_grad_recv_act"):
                n += 1
        return n

    def recvs(r, what):
        n = 0
        for a in plans[r]:
            if what == "act" and a[0] in ("recv_act", "send_grad_recv_act"):
                n += 1
            if what == "grad" and a[0] in ("recv_grad", "send_act_recv_grad"):
                n += 1
        return n

    for r in range(stages - 1):
        assert sends(r, "act") == recvs(r + 1, "act") == m
        assert sends(r + 1, "grad") == recvs(r, "grad") == m
