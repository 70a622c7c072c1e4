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


def eager_update_rank(group):
    """BucketAdamW updating each span right behind its all-reduce, during backward, against the same optimizer
    stepping after backward; also under gradient accumulation with no_sync()."""
    from tandem_b200.ddp import BucketAdamW

    during, after = seeded_model(), seeded_model()
    wrap_a = DDP(during, group, bucket_bytes=64 << 10, rebuild=False)
    opt_a = BucketAdamW(wrap_a, lr=LEARNING_RATE, weight_decay=WEIGHT_DECAY, during_backward=True)
    wrap_b = DDP(after, group, bucket_bytes=64 << 10, rebuild=False)
    opt_b = BucketAdamW(wrap_b, lr=LEARNING_RATE, weight_decay=WEIGHT_DECAY)
    batches = Batches(group.rank, group.size)
    for k in range(4):
        losses = []
        for wrapper, opt in ((wrap_a, opt_a), (wrap_b, opt_b)):
            with wrapper.no_sync():  # the first of two backward passes only accumulates: no update may happen here
                before = flat_weights(wrapper.module.parameters()).clone()
                wrapper(*batches(2 * k)).backward()
                assert torch.equal(flat_weights(wrapper.module.parameters()), before)
            loss = wrapper(*batches(2 * k + 1))
            loss.backward()
            opt.step()
            opt.zero_grad()
            losses.append(loss.item())
        assert losses[0] == losses[1], k
    return torch.equal(flat_weights(during.parameters()), flat_weights(after.parameters()))


def test_bucket_adamw_during_backward_equals_after_backward():
    assert launch(eager_update_rank, 2) == [True, True]


def sharded_optimizer_rank(group):
    """ShardedBucketAdamW (reduce-scatter, update of the owned chunk, all-gather, all during backward) against
    torch's per-parameter AdamW behind a plain DDP wrapper on a twin model fed the same batches."""
    from tandem_b200.ddp import ShardedBucketAdamW

    sharded, plain = seeded_model(), seeded_model()
    wrap_a = DDP(sharded, group, bucket_bytes=16 << 10, rebuild=False)
    opt_a = ShardedBucketAdamW(wrap_a, lr=LEARNING_RATE, weight_decay=WEIGHT_DECAY)
    wrap_b = DDP(plain, group, bucket_bytes=16 << 10, rebuild=False)  # the same spans: the same fold order per element
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
    total = sum(p.numel() for p in sharded.parameters())
    return (torch.equal(flat_weights(sharded.parameters()), flat_weights(plain.parameters())),
            opt_a.state_bytes() <= 2 * 4 * (total // group.size + len(wrap_a.buckets)))


@pytest.mark.parametrize("ranks", [2, 4])
def test_sharded_bucket_adamw_equals_per_parameter_adamw(ranks):
    """Reduce-scatter + all-gather folds each chunk in the same order as the all-reduce, so even with four ranks the
    weights equal those of the twin model behind the all-reducing wrapper."""
    out = launch(sharded_optimizer_rank, ranks)
    assert all(same for same, _ in out)
    assert all(small for _, small in out)


class CountingGroup:
    """Stands in for a Group on one rank: counts what the wrapper takes from the (symmetric) heap."""

    size, rank = 1, 0

    def __init__(self):
        self.taken, self.released = [], []

    def empty(self, numel, dtype, device=None, zero=True):
        self.taken.append(numel)
        return torch.zeros(numel, dtype=dtype)

    def release(self, t):
        self.released.append(t.numel())

    def broadcast(self, t, root=0):
        return t

    def all_reduce(self, t, op="sum", async_op=False):
        class Done:
            def wait(self):
                return t

        return Done()


def test_learning_the_arrival_order_allocates_nothing():
    """The spans are re-cut inside the arena: one heap allocation per dtype for the life of the wrapper."""
    group = CountingGroup()
    model = seeded_model()
    wrapper = DDP(model, group, bucket_bytes=8 << 10)
    assert len(group.taken) == 1 and group.taken[0] == sum(p.numel() for p in model.parameters())
    before = [tuple(id(p) for p in s.params) for s in wrapper.buckets]
    x, y = Batches()(0)
    wrapper(x, y).backward()
    want = {p: p.grad.clone() for p in model.parameters()}
    assert not wrapper.rebuilding
    after = [tuple(id(p) for p in s.params) for s in wrapper.buckets]
    assert len(group.taken) == 1 and not group.released
    assert sorted(i for s in after for i in s) == sorted(i for s in before for i in s)
    for s in wrapper.buckets:  # every gradient moved with its slot, and the spans tile the arena
        for p in s.params:
            assert p.grad.data_ptr() == s.slot[p].data_ptr() and torch.equal(p.grad, want[p])
    assert [s.lo for s in wrapper.buckets] == [0] + [s.hi for s in wrapper.buckets][:-1]
