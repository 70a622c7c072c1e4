"""DDP against torch's DistributedDataParallel (gloo) and against one process.

With 2 ranks the average is (a/2)+(b/2) whatever the algorithm, which floating
point evaluates identically in either order, so losses and weights must equal
torch DDP's bit for bit.  Against a single process the batch is summed in a
different order, so the match is to rounding.
Parity: tests/test_ddp.py:105-125 of the reference."""

import contextlib
import os
import tempfile

import pytest
import torch
import torch.multiprocessing as mp

from tandem_b200 import launch
from tandem_b200.data import synthetic
from tandem_b200.ddp import DDP
from tandem_b200.model import GPT, Config

CFG = Config(seq=32, layers=2, heads=2, dim=32)
STEPS, BATCH = 6, 8


def train(build, rank, world, accumulate=1, zero_with_wrapper=False):
    torch.manual_seed(0)
    text = synthetic(20_000)
    model, step_fn, wrapper = build()
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3, weight_decay=0.1, foreach=False)
    losses = []
    for step in range(STEPS):
        for micro in range(accumulate):
            x, y = text.batch(step * accumulate + micro, BATCH, CFG.seq, rank=rank, world=world)
            loss = step_fn(x, y, micro == accumulate - 1) / accumulate
            losses.append(loss.item())
        opt.step()
        if zero_with_wrapper:
            wrapper.zero_grad()
        else:
            opt.zero_grad()
    return losses, torch.cat([p.detach().reshape(-1) for p in model.parameters()])


def ours_rank(g, bucket_bytes, accumulate, zero_with_wrapper=False):
    def build():
        model = GPT(CFG)
        ddp = DDP(model, g, bucket_bytes=bucket_bytes)

        def step(x, y, last):
            with contextlib.nullcontext() if last else ddp.no_sync():
                loss = ddp(x, y)
                (loss / accumulate).backward()
            return loss

        return model, step, ddp

    return train(build, g.rank, g.size, accumulate, zero_with_wrapper)


def torch_rank(rank, world, init, out, accumulate):
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel

    torch.set_num_threads(1)
    dist.init_process_group("gloo", init_method=f"file://{init}", rank=rank, world_size=world)

    def build():
        model = GPT(CFG)
        ddp = DistributedDataParallel(model)

        def step(x, y, last):
            with contextlib.nullcontext() if last else ddp.no_sync():
                loss = ddp(x, y)
                (loss / accumulate).backward()
            return loss

        return model, step, ddp

    torch.save(train(build, rank, world, accumulate), f"{out}.{rank}")
    dist.destroy_process_group()


def run_torch(world, accumulate=1):
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(torch_rank, args=(world, os.path.join(d, "init"), os.path.join(d, "out"), accumulate), nprocs=world)
        return [torch.load(os.path.join(d, f"out.{r}")) for r in range(world)]


def single(accumulate=1):
    torch.set_num_threads(1)

    def build():
        model = GPT(CFG)

        def step(x, y, last):
            loss = model(x, y)
            (loss / accumulate).backward()
            return loss

        return model, step, None

    return train(build, 0, 1, accumulate)


@pytest.fixture(scope="module")
def torch_ddp_2():
    return run_torch(2)


def test_bit_identical_to_torch_ddp(torch_ddp_2):
    ours = launch(ours_rank, 2, 64 << 10, 1)  # small buckets: several all-reduces in flight
    for r in range(2):
        assert ours[r][0] == torch_ddp_2[r][0], f"rank {r} losses differ"
        assert torch.equal(ours[r][1], torch_ddp_2[r][1]), f"rank {r} weights differ"
    assert torch.equal(ours[0][1], ours[1][1])


def test_wrapper_zero_grad_accumulates_into_buckets(torch_ddp_2):
    ours = launch(ours_rank, 2, 64 << 10, 1, True)
    assert ours[0][0] == torch_ddp_2[0][0]
    assert torch.equal(ours[0][1], torch_ddp_2[0][1])


def test_gradient_accumulation_bit_identical():
    ours = launch(ours_rank, 2, 1 << 20, 2)
    ref = run_torch(2, accumulate=2)
    assert ours[0][0] == ref[0][0]
    assert torch.equal(ours[0][1], ref[0][1])


def test_matches_single_process():
    ours = launch(ours_rank, 2, 1 << 20, 1)
    _, w = single()
    assert torch.allclose(ours[0][1], w, rtol=0, atol=1e-5), (ours[0][1] - w).abs().max()


def four_ranks(g):
    losses, w = ours_rank(g, 32 << 10, 1)
    return losses, w


def test_four_ranks_stay_in_step_and_match_single_process():
    ours = launch(four_ranks, 4)
    for r in range(1, 4):
        assert torch.equal(ours[0][1], ours[r][1])
    _, w = single()
    assert torch.allclose(ours[0][1], w, rtol=0, atol=5e-4), (ours[0][1] - w).abs().max()


def unused(g):
    model = GPT(CFG)
    ddp = DDP(model, g)
    x = torch.randint(0, 256, (2, CFG.seq))
    try:
        ddp.module.embed(x).sum().backward()  # only the embedding gets gradients
    except RuntimeError as e:
        return "received no gradient" in str(e)
    return False


def test_unused_parameters_are_reported():
    assert launch(unused, 2) == [True, True]


def bucket_adamw_rank(g):
    from tandem_b200.ddp import BucketAdamW

    torch.manual_seed(0)
    m1, m2 = GPT(CFG), GPT(CFG)
    m2.load_state_dict(m1.state_dict())
    d1 = DDP(m1, g, rebuild=False)
    o1 = BucketAdamW(d1, lr=3e-3, weight_decay=0.1)
    d2 = DDP(m2, g)
    o2 = torch.optim.AdamW(m2.parameters(), lr=3e-3, weight_decay=0.1, foreach=False)
    text = synthetic(20_000)
    for step in range(4):
        x, y = text.batch(step, BATCH, CFG.seq, rank=g.rank, world=g.size)
        l1 = d1(x, y)
        l1.backward()
        o1.step()
        o1.zero_grad()
        l2 = d2(x, y)
        l2.backward()
        o2.step()
        o2.zero_grad()
        assert l1.item() == l2.item()
    return torch.equal(torch.cat([p.detach().reshape(-1) for p in m1.parameters()]),
                       torch.cat([p.detach().reshape(-1) for p in m2.parameters()]))


def test_bucket_adamw_equals_per_parameter_adamw():
    assert launch(bucket_adamw_rank, 2) == [True, True]
