"""ZeRO-1, ZeRO-2 and FSDP (ZeRO-3) against torch DDP + torch AdamW on two gloo ranks.

The stages only change where gradients, optimizer state and parameters live; the arithmetic stays torch's
(mean of two = (a / 2) + (b / 2), exact copies in the all-gathers, AdamW element by element), so losses and
weights must match torch DDP bit for bit while each rank keeps only its share of the optimizer state.
Behaviours: tests/test_zero.py:19-66 of the reference (stage 2 keeps no full gradients, stage 3 holds at most
three units whole), plus four-rank runs."""

import pytest
import torch

from tandem_b200 import launch
from tandem_b200.optim import ShardedAdamW
from tandem_b200.zero import FSDP, ZeRO

from training import LEARNING_RATE, WEIGHT_DECAY, Batches, flat_weights, optimize, seeded_model, torch_ddp_run

SMALL_BUCKETS = 4 << 10  # many reduce-scatters per backward, most of them with empty chunks for some rank


def sharded_rank(group, stage):
    model = seeded_model()
    opt = ShardedAdamW(lr=LEARNING_RATE, weight_decay=WEIGHT_DECAY)
    wrapper = FSDP(model, group, opt) if stage == 3 else ZeRO(model, group, stage, opt, SMALL_BUCKETS)

    def forward_backward(x, y, _last):
        loss = wrapper(x, y)
        loss.backward()
        return loss

    def update():
        wrapper.step()
        wrapper.zero_grad()

    losses = optimize(forward_backward, update, Batches(group.rank, group.size))
    facts = {"state_bytes": opt.state_bytes()}
    if stage == 3:
        facts.update(max_live=wrapper.max_live, live=wrapper.live)
        weights = wrapper.full_parameters()
    else:
        facts["full_grads_kept"] = sum(p.grad is not None for p in model.parameters())
        weights = flat_weights(model.parameters())
    return losses, weights, facts


@pytest.fixture(scope="module")
def torch_two_ranks():
    return torch_ddp_run(2)


@pytest.mark.parametrize("stage", [1, 2, 3])
def test_stage_bit_identical_to_torch_ddp(stage, torch_two_ranks):
    ours = launch(sharded_rank, 2, stage)
    parameters = torch_two_ranks[0][1].numel()
    for rank, (losses, weights, facts) in enumerate(ours):
        assert losses == torch_two_ranks[rank][0], f"stage {stage}, rank {rank}: losses differ"
        assert torch.equal(weights, torch_two_ranks[rank][1]), f"stage {stage}, rank {rank}: weights differ"
        assert facts["state_bytes"] <= 2 * 4 * (parameters // 2 + 1)  # two fp32 moments for half the parameters
        if stage == 2:
            assert facts["full_grads_kept"] == 0  # only the gradient shard survives backward
        if stage == 3:
            # whole at once: the running unit, the prefetched one, and the head kept from forward to backward
            assert facts["max_live"] <= 3 and facts["live"] == 0, facts


@pytest.mark.parametrize("stage", [2, 3])
def test_four_ranks_agree_with_each_other(stage):
    ours = launch(sharded_rank, 4, stage)
    assert ours[0][0] != ours[1][0]  # every rank trains on its own rows
    assert all(torch.equal(ours[0][1], ours[rank][1]) for rank in (1, 2, 3))
