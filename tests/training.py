"""Shared pieces of the training-equality tests: one tiny GPT, one corpus, one AdamW recipe, and runners that
produce (losses, flat weights) for a wrapper under test, for torch's DistributedDataParallel over gloo, and for
a single process.  Every runner seeds torch the same way before it builds the model, so all of them start from
identical weights and, rank for rank, see identical batches."""

import contextlib
import os
import tempfile

import torch
import torch.multiprocessing as mp

from tandem_b200.data import synthetic
from tandem_b200.model import GPT, Config

TINY = Config(seq=32, layers=2, heads=2, dim=32)
LEARNING_RATE, WEIGHT_DECAY = 3e-3, 0.1
CORPUS_BYTES = 20_000
OPT_STEPS, ROWS = 6, 8  # optimizer steps per run, rows of the global batch


def seeded_model(config=TINY):
    torch.manual_seed(0)
    return GPT(config)


def plain_adamw(parameters):
    """torch's single-tensor AdamW: the update every strategy must reproduce."""
    return torch.optim.AdamW(parameters, lr=LEARNING_RATE, weight_decay=WEIGHT_DECAY, foreach=False)


def flat_weights(parameters):
    return torch.cat([p.detach().reshape(-1) for p in parameters])


class Batches:
    """Batch k of the shared corpus, cut for one rank of `world`."""

    def __init__(self, rank=0, world=1, rows=ROWS, config=TINY):
        self.text = synthetic(CORPUS_BYTES)
        self.rank, self.world, self.rows, self.seq = rank, world, rows, config.seq

    def __call__(self, k):
        return self.text.batch(k, self.rows, self.seq, rank=self.rank, world=self.world)


def optimize(loss_and_backward, after_backwards, batches, steps=OPT_STEPS, passes=1):
    """`steps` optimizer steps of `passes` forward/backward passes each.  loss_and_backward(x, y, last_pass)
    returns the (unscaled) loss after having run backward on loss / passes; after_backwards() applies the
    update and clears the gradients.  Returns every pass's loss / passes as a float."""
    seen = []
    for step in range(steps):
        for k in range(passes):
            x, y = batches(step * passes + k)
            loss = loss_and_backward(x, y, k == passes - 1)
            seen.append((loss / passes).item())
        after_backwards()
    return seen


def data_parallel_pass(wrapper, passes):
    """Forward/backward through a DDP-style wrapper; all but the last pass of a step run under no_sync()."""

    def run(x, y, last_pass):
        guard = contextlib.nullcontext() if last_pass else wrapper.no_sync()
        with guard:
            loss = wrapper(x, y)
            (loss / passes).backward()
        return loss

    return run


def _torch_ddp_worker(rank, world, rendezvous, prefix, passes):
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel

    torch.set_num_threads(1)
    dist.init_process_group("gloo", init_method=f"file://{rendezvous}", rank=rank, world_size=world)
    model = seeded_model()
    wrapper = DistributedDataParallel(model)
    opt = plain_adamw(model.parameters())
    losses = optimize(data_parallel_pass(wrapper, passes), lambda: (opt.step(), opt.zero_grad()), Batches(rank, world),
                      passes=passes)
    torch.save((losses, flat_weights(model.parameters())), f"{prefix}.{rank}")
    dist.destroy_process_group()


def torch_ddp_run(world, passes=1):
    """[(losses, weights)] per rank of torch DDP over gloo with the shared recipe."""
    with tempfile.TemporaryDirectory() as scratch:
        prefix = os.path.join(scratch, "result")
        mp.spawn(_torch_ddp_worker, args=(world, os.path.join(scratch, "rendezvous"), prefix, passes), nprocs=world)
        return [torch.load(f"{prefix}.{rank}") for rank in range(world)]


def single_process_run(passes=1, rows=ROWS):
    """One process over the whole batch: (losses, weights, model)."""
    torch.set_num_threads(1)
    model = seeded_model()
    opt = plain_adamw(model.parameters())

    def run(x, y, _last):
        loss = model(x, y)
        (loss / passes).backward()
        return loss

    losses = optimize(run, lambda: (opt.step(), opt.zero_grad()), Batches(rows=rows), passes=passes)
    return losses, flat_weights(model.parameters()), model
