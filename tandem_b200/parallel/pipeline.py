"""Pipeline parallelism: contiguous runs of model.units() become stages, one per
rank; a batch is cut into micro-batches whose activations flow forward and
whose gradients flow back.

Schedules (same contract as the reference's tandem/pipeline.py:35-166):
  gpipe  all forwards, then all backwards (Huang et al., 2019).
  1f1b   (stages - rank - 1) warm-up forwards, then one forward / one backward
         alternately, then drain (PipeDream-Flush, Megatron-LM).  Steady-state
         transfers are paired (send one tensor while receiving the other), so
         neighbouring stages never wait on each other.
Backwards run in micro-batch order on every stage, so gradients accumulate as in
one process accumulating over the same micro-batches.

The schedule is written once as a list of actions per stage (`plan`); running it
is a small interpreter.  On GPU ranks the transfers are NCCL send/recv pairs and
activations travel in the model's compute dtype.
"""

import torch

from ..models.gpt import loss_fn
from ..utils.profile import Timeline


def split_units(n_units, stages):
    """Contiguous (lo, hi) ranges of units, one per stage, as even as possible."""
    base, extra = divmod(n_units, stages)
    out, lo = [], 0
    for s in range(stages):
        hi = lo + base + (1 if s < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


def plan(schedule, stages, rank, m):
    """The stage's step as a list of actions:
      ("F", i) / ("B", i)          compute micro-batch i forward / backward
      ("recv_act",) ("send_act",) ("recv_grad",) ("send_grad",)
      ("send_act_recv_grad",) ("send_grad_recv_act",)   paired transfers
    Transfers that do not exist at the first / last stage are left out by the runner."""
    acts = []
    if schedule == "gpipe":
        for i in range(m):
            acts += [("recv_act",), ("F", i), ("send_act",)]
        for i in range(m):
            acts += [("recv_grad",), ("B", i), ("send_grad",)]
        return acts
    if schedule != "1f1b":
        raise ValueError(f"unknown schedule {schedule}")
    warm = min(stages - rank - 1, m)
    steady = m - warm
    for i in range(warm):
        acts += [("recv_act",), ("F", i), ("send_act",)]
    if steady > 0:
        acts.append(("recv_act",))
    for k in range(steady):
        acts += [("F", warm + k), ("send_act_recv_grad",), ("B", k)]
        acts.append(("send_grad",) if k == steady - 1 else ("send_grad_recv_act",))
    for k in range(steady, m):
        acts += [("recv_grad",), ("B", k), ("send_grad",)]
    return acts


class Pipeline:
    def __init__(self, model, group, micro_batches, schedule="1f1b", timeline=None):
        if schedule not in ("gpipe", "1f1b"):
            raise ValueError(f"unknown schedule {schedule}")
        self.g, self.m, self.schedule = group, micro_batches, schedule
        units = model.units()
        lo, hi = split_units(len(units), group.size)[group.rank]
        self.units = torch.nn.ModuleList(units[lo:hi])
        self.first, self.last = group.rank == 0, group.rank == group.size - 1
        self.dim = model.config.dim
        self.kernels = getattr(model.config, "kernels", "torch")
        self.timeline = timeline or Timeline(enabled=False)
        self.act_dtype = None  # None: the dtype of this stage's parameters

    def parameters(self):
        return self.units.parameters()

    def _run_units(self, x):
        for u in self.units:
            x = u(x)
        return x

    def train_step(self, x, y):
        """Forward and backward over the global batch (x, y), which every rank
        passes (stage 0 reads x, the last stage reads y).  Gradients accumulate
        in this stage's parameters.  Returns the mean loss on the last stage,
        None elsewhere."""
        xs, ys = x.chunk(self.m), y.chunk(self.m)
        if len(xs) != self.m or any(c.shape[0] != xs[0].shape[0] for c in xs):
            raise ValueError("the batch must divide evenly into micro-batches")
        first_param = next(self.parameters())
        dev = first_param.device
        dtype = self.act_dtype or (torch.get_autocast_dtype(dev.type) if torch.is_autocast_enabled(dev.type)
                                   else first_param.dtype)
        shape = (xs[0].shape[0], xs[0].shape[1], self.dim)
        g, up, down = self.g, self.g.rank - 1, self.g.rank + 1
        saved, losses = {}, []
        act = grad = out = None

        def fresh():
            return torch.empty(shape, device=dev, dtype=dtype)

        actions = plan(self.schedule, g.size, g.rank, self.m)
        if dev.type == "cuda" and getattr(g, "transport", "device") == "device" and g.size > 1:
            return self._run_on_lanes(actions, xs, ys, dev, dtype, shape)
        for a in actions:
            kind = a[0]
            if kind == "F":
                i = a[1]
                with self.timeline.span(f"F{i}"):
                    inp = xs[i].to(dev) if self.first else act.requires_grad_()
                    out = self._run_units(inp)
                    if self.last:
                        out = loss_fn(out, ys[i].to(dev), self.kernels) / self.m
                        losses.append(out.detach())
                    saved[i] = (inp, out)
            elif kind == "B":
                i = a[1]
                with self.timeline.span(f"B{i}"):
                    inp, res = saved.pop(i)
                    if self.last:
                        res.backward()
                    else:
                        res.backward(grad)
                    grad = None if self.first else inp.grad
            elif kind == "recv_act":
                if not self.first:
                    act = fresh()
                    g.recv(act, up)
            elif kind == "send_act":
                if not self.last:
                    g.send(out.detach().contiguous(), down)
            elif kind == "recv_grad":
                if not self.last:
                    grad = fresh()
                    g.recv(grad, down)
            elif kind == "send_grad":
                if not self.first:
                    g.send(grad.contiguous(), up)
            elif kind == "send_act_recv_grad":
                if not self.last:
                    grad = fresh()
                    g.sendrecv(out.detach().contiguous(), down, grad, down)
            elif kind == "send_grad_recv_act":
                if not self.first:
                    act = fresh()
                    g.sendrecv(grad.contiguous(), up, act, up)
        return sum(losses) if self.last else None

    def _run_on_lanes(self, actions, xs, ys, dev, dtype, shape):
        """GPU stages.  Transfers use two NCCL lanes (activations down, gradients up), so paired actions fall
        apart into an asynchronous send and a receive that was posted ahead of time: as soon as one receive
        has been claimed the next one of its kind is posted, before this stage computes anything on what it just
        received (the first of each kind is posted when the schedule first asks for it).  Sends never hold up the
        compute stream; they are collected and awaited when the step ends."""
        g, up, down = self.g, self.g.rank - 1, self.g.rank + 1
        wire = g._p2p()
        takes_act = {"recv_act", "send_grad_recv_act"}
        takes_grad = {"recv_grad", "send_act_recv_grad"}
        acts_due = 0 if self.first else sum(a[0] in takes_act for a in actions)
        grads_due = 0 if self.last else sum(a[0] in takes_grad for a in actions)
        posted = {"act": None, "grad": None}

        def post(kind):
            nonlocal acts_due, grads_due
            if kind == "act" and acts_due:
                acts_due -= 1
                posted["act"] = wire.post_recv(shape, dtype, up, "act")
            elif kind == "grad" and grads_due:
                grads_due -= 1
                posted["grad"] = wire.post_recv(shape, dtype, down, "grad")

        def claim(kind):
            if posted[kind] is None:
                post(kind)  # the first of its kind in this step is posted when it is first needed
            handle, posted[kind] = posted[kind], None
            tensor = wire.claim(*handle)
            post(kind)  # the next one starts arriving while this one is being used
            return tensor

        saved, losses, in_flight = {}, [], []
        act = grad = out = None
        for a in actions:
            kind = a[0]
            if kind == "F":
                i = a[1]
                with self.timeline.span(f"F{i}"):
                    inp = xs[i].to(dev) if self.first else act.requires_grad_()
                    out = self._run_units(inp)
                    if self.last:
                        out = loss_fn(out, ys[i].to(dev), self.kernels) / self.m
                        losses.append(out.detach())
                    saved[i] = (inp, out)
            elif kind == "B":
                i = a[1]
                with self.timeline.span(f"B{i}"):
                    inp, res = saved.pop(i)
                    if self.last:
                        res.backward()
                    else:
                        res.backward(grad)
                    grad = None if self.first else inp.grad
            else:
                if kind in ("send_act", "send_act_recv_grad") and not self.last:
                    in_flight.append(wire.post_send(out.detach().contiguous(), down, "act"))
                if kind in ("send_grad", "send_grad_recv_act") and not self.first:
                    in_flight.append(wire.post_send(grad.contiguous(), up, "grad"))
                if kind in takes_act and not self.first:
                    act = claim("act")
                if kind in takes_grad and not self.last:
                    grad = claim("grad")
        for work, _tensor in in_flight:
            work.wait()
        return sum(losses) if self.last else None
