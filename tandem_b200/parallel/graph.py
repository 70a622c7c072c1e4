"""A whole training step (forward, backward with its overlapped gradient
all-reduces, optimizer) captured once as a CUDA graph and replayed.

At the benchmark sizes a step is several hundred kernel launches of a few
microseconds each; issued one by one from Python they cost more host time than
GPU time.  Replaying a captured graph removes that: the GPU sees one launch.
This works because nothing in the step needs the host: collectives are kernels
whose barrier counters live in device memory, `Work.wait()` is a stream
dependency, and the optimizer's step-dependent constants are computed on the
device (`BucketAdamW`).  The reference has no counterpart (its engines are driven
piece by piece from a host thread: tandem/comm.py:211-233).
"""

import torch


class GraphedStep:
    """step = GraphedStep(ddp, optimizer, x, y); loss = step(x, y)

    `ddp` is a DDP wrapper around a module whose forward(x, y) returns the loss,
    `optimizer` a BucketAdamW; x / y fix the batch shape.  A few eager steps run
    first (they train for real), then one step is captured.  `step(x, y)` copies
    the batch into the captured input buffers and replays; it returns the loss
    tensor of that step (a device scalar, overwritten by the next call).
    """

    def __init__(self, ddp, optimizer, x, y, warmup=3, autocast=None):
        self.ddp, self.opt = ddp, optimizer
        dev = x.device
        self.x, self.y = x.clone(), y.clone()
        self.autocast = autocast
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self._one_step()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        from .symm import cuda_lib

        self.graph = torch.cuda.CUDAGraph()
        before = cuda_lib().tb_launch_count(0)
        with torch.cuda.graph(self.graph):
            self.loss = self._one_step()
        self.launches_per_step = int(cuda_lib().tb_launch_count(0) - before)  # this library's kernels inside the graph
        if ddp.g.size > 1:
            ddp.g.barrier()

    def _one_step(self):
        if self.autocast is not None:
            with torch.autocast("cuda", dtype=self.autocast):
                loss = self.ddp(self.x, self.y)
        else:
            loss = self.ddp(self.x, self.y)
        loss.backward()
        self.opt.step()
        for p in self.ddp.params:  # set_to_none: the next backward writes fresh gradients, packed per bucket
            p.grad = None
        return loss.detach()

    def __call__(self, x, y):
        self.x.copy_(x, non_blocking=True)
        self.y.copy_(y, non_blocking=True)
        self.opt.step_count += 1.0
        self.graph.replay()
        return self.loss
