"""Token batches for training runs and benchmarks.

Every rank derives the WHOLE global batch of a step from a seed that depends only on (seed, step) and keeps the
rows that belong to it, so N ranks together see exactly the rows one process would.  `Text` (byte-level text,
vocabulary 256) and `synthetic` produce the same batches as the reference's tandem/data.py:9-41 for the same
arguments; `uniform_tokens` is the benchmark input of the baseline configurations: ids uniform in [0, vocab).
"""

import torch


def _step_generator(seed, step):
    gen = torch.Generator()
    gen.manual_seed(seed * 1_000_003 + step)
    return gen


def _rows_of_rank(count, rank, world):
    """The slice of a global batch of `count` rows that rank `rank` of `world` trains on."""
    if count % world:
        raise ValueError(f"global batch {count} does not divide over {world} ranks")
    share = count // world
    return slice(rank * share, (rank + 1) * share)


class Text:
    """A byte string as a token stream; batches are windows of seq + 1 bytes at random offsets."""

    def __init__(self, path=None, data=None):
        if data is None:
            with open(path, "rb") as source:
                data = source.read()
        self.data = torch.frombuffer(bytearray(data), dtype=torch.uint8).long()

    def batch(self, step, batch, seq, seed=0, rank=0, world=1, device="cpu"):
        """(inputs, targets) for this rank's rows of global batch `step`; targets are the inputs shifted by one."""
        mine = _rows_of_rank(batch, rank, world)
        last_start = self.data.numel() - seq - 1
        offsets = torch.randint(0, last_start, (batch,), generator=_step_generator(seed, step))[mine]
        windows = self.data[offsets.unsqueeze(1) + torch.arange(seq + 1).unsqueeze(0)]
        inputs, targets = windows[:, :seq], windows[:, 1:]
        return inputs.to(device, non_blocking=True), targets.to(device, non_blocking=True)


def synthetic(n=200_000, seed=0):
    """Pseudo-text a model can learn from without a corpus on disk: a walk of `n` steps over 256 states, each
    with four seeded successors."""
    gen = torch.Generator()
    gen.manual_seed(seed)
    successors = torch.randint(0, 256, (256, 4), generator=gen).tolist()
    turns = torch.randint(0, 4, (n,), generator=gen).tolist()
    walk = bytearray()
    state = 0
    for turn in turns:
        state = successors[state][turn]
        walk.append(state)
    return Text(data=bytes(walk))


def uniform_tokens(step, batch, seq, vocab, seed=0, rank=0, world=1, pin=False):
    """This rank's rows of global batch `step`, ids uniform in [0, vocab), on the host (pinned on request)."""
    mine = _rows_of_rank(batch, rank, world)
    rows = torch.randint(0, vocab, (batch, seq + 1), generator=_step_generator(seed, step))[mine]
    pair = rows[:, :seq].contiguous(), rows[:, 1:].contiguous()
    return tuple(t.pin_memory() for t in pair) if pin else pair
