"""ZeRO-1/2/3 against torch DDP + torch AdamW (gloo, 2 ranks): the stages move
gradients, optimizer state and parameters around but never change arithmetic,
so losses and weights must be bit-identical, with each rank holding only its
share of the optimizer state.  Parity: tests/test_zero.py:19-66 of the reference."""

import pytest
import torch

from tandem_b200 import launch
from tandem_b200.data import synthetic
from tandem_b200.model import GPT
from tandem_b200.optim import ShardedAdamW
from tandem_b200.zero import FSDP, ZeRO

from test_ddp import BATCH, CFG, STEPS, run_torch


def zero_rank(g, stage, bucket_bytes):
    torch.manual_seed(0)
    text = synthetic(20_000)
    model = GPT(CFG)
    opt = ShardedAdamW(lr=3e-3, weight_decay=0.1)
    z = ZeRO(model, g, stage, opt, bucket_bytes) if stage < 3 else FSDP(model, g, opt)
    losses = []
    for step in range(STEPS):
        x, y = text.batch(step, BATCH, CFG.seq, rank=g.rank, world=g.size)
        loss = z(x, y)
        loss.backward()
        losses.append(loss.item())
        z.step()
        z.zero_grad()
    if stage < 3:
        w = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
        if stage == 2:
            assert all(p.grad is None for p in model.parameters())
    else:
        # the running unit, the prefetched one and the head kept for backward
        assert z.max_live <= 3, z.max_live
        assert z.live == 0
        w = z.full_parameters()
    return losses, w, opt.state_bytes()


@pytest.fixture(scope="module")
def reference_run():
    return run_torch(2)


@pytest.mark.parametrize("stage", [1, 2, 3])
def test_stage_bit_identical_to_torch_ddp(stage, reference_run):
    ours = launch(zero_rank, 2, stage, 4 << 10)
    nparams = reference_run[0][1].numel()
    for r in range(2):
        assert ours[r][0] == reference_run[r][0], f"stage {stage}, rank {r}: losses differ"
        assert torch.equal(ours[r][1], reference_run[r][1]), f"stage {stage}, rank {r}: weights differ"
        assert ours[r][2] <= 2 * 4 * (nparams // 2 + 1)  # two moments for half the parameters


@pytest.mark.parametrize("stage", [2, 3])
def test_four_ranks_agree_with_each_other(stage):
    ours = launch(zero_rank, 4, stage, 4 << 10)
    assert ours[0][0] != ours[1][0]  # different data per rank
    assert all(torch.equal(ours[0][1], ours[r][1]) for r in range(1, 4))
