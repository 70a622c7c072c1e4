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
from tandem_b200.parallel.pipeline import split_by_cost, unit_costs
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


class GlooWire:
    """The transfer interface of parallel/p2p.py (lanes, receives posted ahead, grouped exchanges) over gloo, so that
    the scheduling a GPU stage does -- what is posted when, on which lane, in which order -- runs on CPU ranks."""

    def __init__(self, group, rendezvous):
        import torch.distributed as dist

        self.dist = dist
        dist.init_process_group("gloo", init_method=f"file://{rendezvous}", rank=group.rank, world_size=group.size)
        self.lanes = {"act": None, "grad": dist.new_group(list(range(group.size)), backend="gloo")}
        self.log = []

    def lane(self, name):
        return self.lanes[name]

    def post_recv(self, shape, dtype, src, lane):
        buf = torch.empty(shape, dtype=dtype)
        self.log.append(("recv", lane, src))
        return self.dist.irecv(buf, src, group=self.lanes[lane]), buf

    def claim(self, work, buf):
        work.wait()
        return buf

    def post_send(self, tensor, dst, lane):
        self.log.append(("send", lane, dst))
        return self.dist.isend(tensor, dst, group=self.lanes[lane]), tensor

    def exchange(self, sends, recvs, shape, dtype):
        received = [torch.empty(shape, dtype=dtype) for _ in recvs]
        works = [self.dist.isend(t, dst) for t, dst in sends] + [self.dist.irecv(b, src) for b, src in zip(received, recvs)]
        self.log.append(("exchange", len(sends), len(recvs)))

        class Both:
            def wait(self):
                for w in works:
                    w.wait()

        return Both(), [t for t, _ in sends] + received, received

    def close(self):
        self.dist.destroy_process_group()


def lanes_rank(group, schedule, rendezvous):
    pipe = Pipeline(seeded_model(), group, MICRO, schedule)
    pipe.wire = GlooWire(group, rendezvous)
    opt = plain_adamw(pipe.parameters())
    batches = Batches(rows=ROWS)
    losses = []
    for k in range(OPT_STEPS):
        loss = pipe.train_step(*batches(k))
        opt.step()
        opt.zero_grad()
        losses.append(loss.item() if loss is not None else None)
    log = pipe.wire.log
    pipe.wire.close()
    return losses, flat_weights(pipe.parameters()), log


@pytest.mark.parametrize("schedule", ["gpipe", "1f1b"])
@pytest.mark.parametrize("stages", [2, 4])
def test_gpu_stage_scheduling_on_cpu_ranks(schedule, stages, accumulated, tmp_path):
    want_losses, unit_weights = accumulated
    ours = launch(lanes_rank, stages, schedule, str(tmp_path / "rendezvous"), slot_bytes=1024)
    for rank, (lo, hi) in enumerate(split_units(len(unit_weights), stages)):
        assert torch.equal(ours[rank][1], torch.cat(unit_weights[lo:hi])), f"stage {rank}: weights differ"
    assert ours[-1][0] == want_losses
    for rank in range(stages):
        log = ours[rank][2][:len(ours[rank][2]) // OPT_STEPS]  # one step
        if schedule == "1f1b":
            assert all(entry[0] == "exchange" for entry in log)
            continue
        # GPipe: a receive is never posted before the send that forwards the previous tensor of its kind, so on a
        # lane's stream no receive stands in front of a send its own sender may be waiting for
        for lane in ("act", "grad"):
            on_lane = [e[0] for e in log if e[1] == lane]
            forwards = "send" in on_lane and "recv" in on_lane
            if forwards:
                assert on_lane == ["recv", "send"] * MICRO, (rank, lane, on_lane)
            else:
                assert len(on_lane) == MICRO and len(set(on_lane)) == 1


def test_split_by_cost_minimises_the_heaviest_stage():
    import itertools

    assert split_by_cost([1, 1, 1], 3) == [(0, 1), (1, 2), (2, 3)]
    assert split_by_cost([5, 1, 1, 1, 1, 5], 2) == [(0, 3), (3, 6)]
    costs = [0.0] + [13.6] * 24 + [51.5]  # embedding, 24 blocks, a 50k-row output projection
    assert split_by_cost(costs, 2) == [(0, 15), (15, 26)]
    gen = torch.Generator().manual_seed(0)
    for _ in range(30):  # against brute force over every placement of the cuts
        n, stages = int(torch.randint(3, 9, (1,), generator=gen)), int(torch.randint(1, 4, (1,), generator=gen))
        costs = torch.randint(0, 20, (n,), generator=gen).tolist()
        got = split_by_cost(costs, stages)
        assert got[0][0] == 0 and got[-1][1] == n and all(a[1] == b[0] for a, b in zip(got, got[1:])) and all(lo < hi for lo, hi in got)
        heaviest = max(sum(costs[lo:hi]) for lo, hi in got)
        best = min(max(sum(costs[a:b]) for a, b in zip((0,) + cuts, cuts + (n,)))
                   for cuts in itertools.combinations(range(1, n), stages - 1))
        assert heaviest == best


def test_unit_costs_count_linear_weights_and_attention():
    model = seeded_model()
    costs = unit_costs(model.units(), model.config.seq)
    assert costs[0] == 0  # an embedding lookup
    width = model.config.dim
    assert costs[1] == 12 * width * width + model.config.seq * width
    head = model.config.vocab * width
    assert costs[-1] == (head / 1.6 if model.config.vocab >= 8 * width else head)


def cost_balanced_rank(group):
    pipe = Pipeline(seeded_model(), group, MICRO, "1f1b", balance="cost")
    loss = pipe.train_step(*Batches(rows=ROWS)(0))
    return pipe.ranges, None if loss is None else loss.item()


def test_cost_balanced_stages_compute_the_same_loss(accumulated):
    ours = launch(cost_balanced_rank, 2, slot_bytes=1024)
    assert ours[0][0] == ours[1][0] and ours[0][0][0][0] == 0
    assert ours[-1][1] == accumulated[0][0]


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
