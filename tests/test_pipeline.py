"""GPipe and 1F1B over 2, 3 and 4 stages against one process that accumulates gradients over the same
micro-batches.  A stage computes for each micro-batch exactly what that process computes for the stage's units,
and runs its backwards in the same order, so losses and the weights after AdamW must agree bit for bit; the
recorded F/B spans show that the two schedules really order the work differently.
Behaviours: tests/test_pipeline.py:61-76 of the reference, plus checks of the schedules' action lists."""

import pytest
import torch

from tandem_b200 import launch
from tandem_b200.model import loss_fn
from tandem_b200.pipeline import Pipeline, plan, split_units
from tandem_b200.profile import Timeline

from training import Batches, flat_weights, optimize, plain_adamw, seeded_model

OPT_STEPS, ROWS, MICRO = 3, 12, 6


def stage_rank(group, schedule):
    spans = Timeline()
    pipe = Pipeline(seeded_model(), group, MICRO, schedule, timeline=spans)
    opt = plain_adamw(pipe.parameters())
    batches = Batches(rows=ROWS)  # every stage is handed the whole batch
    losses = []
    for k in range(OPT_STEPS):
        loss = pipe.train_step(*batches(k))
        opt.step()
        opt.zero_grad()
        losses.append(loss.item() if loss is not None else None)
    first_step = [name for name, _begin, _end in spans.spans[:2 * MICRO]]
    return losses, flat_weights(pipe.parameters()), first_step


@pytest.fixture(scope="module")
def accumulated():
    torch.set_num_threads(1)
    model = seeded_model()
    opt = plain_adamw(model.parameters())
    batches = Batches(rows=ROWS)
    step_losses = []

    def micro_batches(x, y, _last):
        total = 0
        for xs, ys in zip(x.chunk(MICRO), y.chunk(MICRO)):
            piece = loss_fn(model(xs), ys) / MICRO
            piece.backward()
            total = total + piece.detach()
        step_losses.append(total.item())
        return total

    optimize(micro_batches, lambda: (opt.step(), opt.zero_grad()), batches, steps=OPT_STEPS)
    return step_losses, [flat_weights(unit.parameters()) for unit in model.units()]


@pytest.mark.parametrize("schedule", ["gpipe", "1f1b"])
@pytest.mark.parametrize("stages", [2, 3, 4])
def test_bit_identical_to_accumulation(schedule, stages, accumulated):
    want_losses, unit_weights = accumulated
    ours = launch(stage_rank, stages, schedule, slot_bytes=1024)
    for rank, (lo, hi) in enumerate(split_units(len(unit_weights), stages)):
        assert torch.equal(ours[rank][1], torch.cat(unit_weights[lo:hi])), f"stage {rank}: weights differ"
    assert ours[-1][0] == want_losses  # the last stage sees the losses
    order = ours[0][2]
    forwards = [f"F{i}" for i in range(MICRO)]
    if schedule == "gpipe":
        assert order == forwards + [f"B{i}" for i in range(MICRO)]
    else:  # stage 0 warms up with `stages` forwards, then its first backward comes straight away
        assert order[:stages + 1] == forwards[:stages] + ["B0"]


def test_split_units_is_even_and_contiguous():
    assert split_units(4, 2) == [(0, 2), (2, 4)]
    assert split_units(26, 4) == [(0, 7), (7, 14), (14, 20), (20, 26)]
    assert split_units(3, 3) == [(0, 1), (1, 2), (2, 3)]


SENDS = {"act": ("send_act", "send_act_recv_grad"), "grad": ("send_grad", "send_grad_recv_act")}
RECEIVES = {"act": ("recv_act", "send_grad_recv_act"), "grad": ("recv_grad", "send_act_recv_grad")}


@pytest.mark.parametrize("schedule", ["gpipe", "1f1b"])
@pytest.mark.parametrize("stages,m", [(2, 4), (4, 6), (4, 2), (3, 1)])
def test_plans_pair_up(schedule, stages, m):
    """Each stage runs every micro-batch forward and backward once, in order, and every transfer a stage sends has
    its receive on the neighbouring stage."""
    plans = [plan(schedule, stages, rank, m) for rank in range(stages)]

    def count(rank, names):
        return sum(action[0] in names for action in plans[rank])

    for rank, actions in enumerate(plans):
        for kind in "FB":
            assert [a[1] for a in actions if a[0] == kind] == list(range(m)), (rank, kind)
    for upper in range(stages - 1):
        lower = upper + 1
        assert count(upper, SENDS["act"]) == count(lower, RECEIVES["act"]) == m
        assert count(lower, SENDS["grad"]) == count(upper, RECEIVES["grad"]) == m
