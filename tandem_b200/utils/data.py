"""Token batches.  `Text` and `synthetic` follow the reference's tandem/data.py:9-41
(every rank draws the global batch from a per-step seed and keeps its rows, so N
ranks see exactly what one process would).  `uniform_tokens` is the benchmark
input named by the baseline configs: token ids uniform in [0, vocab) from a seed."""

import torch


class Text:
    def __init__(self, path=None, data=None):
        if data is None:
            with open(path, "rb") as f:
                data = f.read()
        self.data = torch.frombuffer(bytearray(data), dtype=torch.uint8).long()

    def batch(self, step, batch, seq, seed=0, rank=0, world=1, device="cpu"):
        """Rows [rank*batch/world, (rank+1)*batch/world) of global batch `step`,
        as (inputs, targets) shifted by one position."""
        if batch % world:
            raise ValueError(f"global batch {batch} does not divide over {world} ranks")
        gen = torch.Generator().manual_seed(seed * 1_000_003 + step)
        starts = torch.randint(0, self.data.numel() - seq - 1, (batch,), generator=gen)
        per = batch // world
        idx = starts[rank * per:(rank + 1) * per, None] + torch.arange(seq + 1)[None, :]
        rows = self.data[idx]
        return rows[:, :-1].to(device, non_blocking=True), rows[:, 1:].to(device, non_blocking=True)


def synthetic(n=200_000, seed=0):
    """Learnable pseudo-text without a corpus on disk: a seeded 256-state Markov chain."""
    gen = torch.Generator().manual_seed(seed)
    table = torch.randint(0, 256, (256, 4), generator=gen).tolist()
    pick = torch.randint(0, 4, (n,), generator=gen).tolist()
    out = bytearray(n)
    state = 0
    for i, c in enumerate(pick):
        state = table[state][c]
        out[i] = state
    return Text(data=bytes(out))


def uniform_tokens(step, batch, seq, vocab, seed=0, rank=0, world=1, pin=False):
    """This rank's rows of global batch `step`: ids uniform in [0, vocab), targets
    are the inputs shifted by one.  Returned on the host (optionally pinned)."""
    if batch % world:
        raise ValueError(f"global batch {batch} does not divide over {world} ranks")
    gen = torch.Generator().manual_seed(seed * 1_000_003 + step)
    rows = torch.randint(0, vocab, (batch, seq + 1), generator=gen)
    per = batch // world
    rows = rows[rank * per:(rank + 1) * per]
    x, y = rows[:, :-1].contiguous(), rows[:, 1:].contiguous()
    if pin:
        x, y = x.pin_memory(), y.pin_memory()
    return x, y
