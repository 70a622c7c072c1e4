"""DDP against torch's DistributedDataParallel (gloo) and against one process.

With two ranks the mean of the gradients is (a / 2) + (b / 2) whatever algorithm moves the data, and floating
point gives that the same value in either order, so losses and weights must equal torch DDP's bit for bit: with
small buckets (several all-reduces in flight), with gradient accumulation under no_sync, and when the wrapper's
own zero_grad keeps gradients inside the buckets.  One process sums the batch in a different order, so that
comparison is to rounding.  Behaviours: tests/test_ddp.py:105-125 of the reference, plus four ranks."""

import pytest
import torch

from tandem_b200 import launch
from tandem_b200.ddp import DDP

from training import (LEARNING_RATE, TINY, WEIGHT_DECAY, Batches, data_parallel_pass, flat_weights, optimize, plain_adamw,
                      seeded_model, single_process_run, torch_ddp_run)


def ddp_rank(group, bucket_bytes, passes=1, clear_through_wrapper=False):
    model = seeded_model()
    wrapper = DDP(model, group, bucket_bytes=bucket_bytes)
    opt = plain_adamw(model.parameters())

    def update():
        opt.step()
        (wrapper if clear_through_wrapper else opt).zero_grad()

    losses = optimize(data_parallel_pass(wrapper, passes), update, Batches(group.rank, group.size), passes=passes)
    return losses, flat_weights(model.parameters())


@pytest.fixture(scope="module")
def torch_two_ranks():
    return torch_ddp_run(2)


def assert_same_run(ours, theirs, ranks):
    for rank in ranks:
        assert ours[rank][0] == theirs[rank][0], f"rank {rank}: losses differ"
        assert torch.equal(ours[rank][1], theirs[rank][1]), f"rank {rank}: weights differ"


def test_bit_identical_to_torch_ddp(torch_two_ranks):
    ours = launch(ddp_rank, 2, 64 << 10)  # 64 KiB buckets: many all-reduces overlap backward
    assert_same_run(ours, torch_two_ranks, (0, 1))
    assert torch.equal(ours[0][1], ours[1][1])


def test_wrapper_zero_grad_accumulates_into_buckets(torch_two_ranks):
    ours = launch(ddp_rank, 2, 64 << 10, 1, True)
    assert_same_run(ours, torch_two_ranks, (0,))


def test_gradient_accumulation_bit_identical():
    ours = launch(ddp_rank, 2, 1 << 20, 2)
    assert_same_run(ours, torch_ddp_run(2, passes=2), (0,))


def test_matches_single_process():
    ours = launch(ddp_rank, 2, 1 << 20)
    _, alone, _ = single_process_run()
    assert torch.allclose(ours[0][1], alone, rtol=0, atol=1e-5), (ours[0][1] - alone).abs().max()


def test_four_ranks_stay_in_step_and_match_single_process():
    ours = launch(ddp_rank, 4, 32 << 10)
    assert all(torch.equal(ours[0][1], ours[rank][1]) for rank in (1, 2, 3))
    _, alone, _ = single_process_run()
    assert torch.allclose(ours[0][1], alone, rtol=0, atol=5e-4), (ours[0][1] - alone).abs().max()


def backward_through_the_embedding_only(group):
    wrapper = DDP(seeded_model(), group)
    tokens = torch.randint(0, TINY.vocab, (2, TINY.seq))
    try:
        wrapper.module.embed(tokens).sum().backward()  # blocks and head get no gradient
    except RuntimeError as e:
        return "received no gradient" in str(e)
    return False


def test_unused_parameters_are_reported():
    assert launch(backward_through_the_embedding_only, 2) == [True, True]


def bucket_optimizer_rank(group):
    """BucketAdamW (one update per bucket, on the flat gradient buffer) against torch's per-parameter AdamW on a
    twin model fed the same batches."""
    from tandem_b200.ddp import BucketAdamW

    bucketed, plain = seeded_model(), seeded_model()
    wrap_a = DDP(bucketed, group, rebuild=False)
    opt_a = BucketAdamW(wrap_a, lr=LEARNING_RATE, weight_decay=WEIGHT_DECAY)
    wrap_b = DDP(plain, group)
    opt_b = plain_adamw(plain.parameters())
    batches = Batches(group.rank, group.size)
    for k in range(4):
        x, y = batches(k)
        losses = []
        for wrapper, opt in ((wrap_a, opt_a), (wrap_b, opt_b)):
            loss = wrapper(x, y)
            loss.backward()
            opt.step()
            opt.zero_grad()
            losses.append(loss.item())
        assert losses[0] == losses[1], k
    return torch.equal(flat_weights(bucketed.parameters()), flat_weights(plain.parameters()))


def test_bucket_adamw_equals_per_parameter_adamw():
    assert launch(bucket_optimizer_rank, 2) == [True, True]
