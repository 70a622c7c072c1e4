"""A whole training step (forward, backward with its overlapped collectives,
optimizer) captured once as a CUDA graph and replayed.

At the benchmark sizes a step is several hundred kernel launches of a few
microseconds each; issued one by one from Python they cost more host time than
GPU time.  Replaying a captured graph removes that: the GPU sees one launch.
This works because nothing in a step needs the host: collectives are kernels
whose barrier counters live in device memory, `Work.wait()` is a stream
dependency, every buffer a collective touches has a fixed address (gradient
arenas, slot rings), and the optimizers compute their step-dependent constants
on the device (`BucketAdamW`, `ShardedBucketAdamW`, `ShardedAdamW` with device
scalars).  The reference has no counterpart (its engines are driven piece by
piece from a host thread: tandem/comm.py:211-233).
"""

import torch


class GraphedStep:
    """step = GraphedStep(wrapper, optimizer, x, y); loss = step(x, y)

    `wrapper` is a DDP, ZeRO or FSDP wrapper around a module whose forward(x, y) returns the loss.
    `optimizer` is the object whose step() / zero_grad() close the step: a BucketAdamW or
    ShardedBucketAdamW for DDP, the wrapper itself for ZeRO / FSDP (built with capturable=True).
    x / y fix the batch shape.  A few eager steps run first (they train for real), then one step is
    captured.  `step(x, y)` copies the batch into the captured input buffers and replays; it returns the
    loss tensor of that step (a device scalar, overwritten by the next call).
    """

    def __init__(self, wrapper, optimizer, x, y, warmup=3, autocast=None):
        self.wrapper, self.opt = wrapper, optimizer
        self.group = wrapper.g
        dev = x.device
        self.x, self.y = x.clone(), y.clone()
        self.autocast = autocast
        # gradients of DDP-style wrappers are dropped after each step so that backward writes fresh ones (packed per
        # span by one kernel); the sharded wrappers clear their own gradient shards in zero_grad()
        self._drop_grads = list(getattr(wrapper, "params", [])) if hasattr(wrapper, "arenas") else None
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
        if self.group.size > 1:
            self.group.barrier()

    def _one_step(self):
        if self.autocast is not None:
            with torch.autocast("cuda", dtype=self.autocast):
                loss = self.wrapper(self.x, self.y)
        else:
            loss = self.wrapper(self.x, self.y)
        loss.backward()
        self.opt.step()
        if self._drop_grads is not None:
            for p in self._drop_grads:
                p.grad = None
        else:
            self.opt.zero_grad()
        return loss.detach()

    def __call__(self, x, y):
        self.x.copy_(x, non_blocking=True)
        self.y.copy_(y, non_blocking=True)
        if hasattr(self.opt, "step_count"):
            self.opt.step_count += 1.0  # the host-side mirror of the device counter
        self.graph.replay()
        return self.loss
