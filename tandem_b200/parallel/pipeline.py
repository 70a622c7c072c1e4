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


def unit_costs(units, seq):
    """Relative compute per unit: the weights of its Linear layers (GEMM work per token is proportional to them) plus,
    for a unit with causal attention, seq x dim for the score and value products.  Embedding lookups cost nothing.
    With a large vocabulary the output projection weighs as much as two or three transformer blocks, which is why an
    even split by unit count leaves the last stage with the most work."""
    costs = []
    for unit in units:
        c = 0.0
        for module in unit.modules():
            if isinstance(module, torch.nn.Linear):
                work = float(module.weight.numel())
                if module.out_features >= 8 * module.in_features:
                    # a vocabulary-sized projection is one large GEMM that runs about 1.6x closer to the tensor peak
                    # than a block's 20-50 us GEMMs (measured: 1.29 vs 0.7-0.95 PFLOP/s)
                    work /= 1.6
                c += work
        attn = getattr(unit, "attn", None)
        if attn is not None:
            width = next(attn.parameters()).shape[-1]
            c += float(seq) * width
        costs.append(c)
    return costs


def split_by_cost(costs, stages):
    """Contiguous (lo, hi) ranges, one per stage and none empty, that minimise the largest stage cost."""
    n = len(costs)
    if stages > n:
        raise ValueError("more stages than units")
    prefix = [0.0]
    for c in costs:
        prefix.append(prefix[-1] + c)
    inf = float("inf")
    best = [[inf] * (n + 1) for _ in range(stages + 1)]  # best[s][i]: the first i units on s stages
    cut = [[0] * (n + 1) for _ in range(stages + 1)]
    best[0][0] = 0.0
    for s in range(1, stages + 1):
        for i in range(s, n - (stages - s) + 1):
            for j in range(s - 1, i):
                worst = max(best[s - 1][j], prefix[i] - prefix[j])
                if worst < best[s][i]:
                    best[s][i], cut[s][i] = worst, j
    out, hi = [], n
    for s in range(stages, 0, -1):
        lo = cut[s][hi]
        out.append((lo, hi))
        hi = lo
    return out[::-1]


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
    def __init__(self, model, group, micro_batches, schedule="1f1b", timeline=None, balance="units"):
        """balance="units": stages get equal numbers of units (the reference's split, tandem/pipeline.py:20-32);
        balance="cost": the contiguous split that minimises the largest stage's estimated compute (unit_costs)."""
        if schedule not in ("gpipe", "1f1b"):
            raise ValueError(f"unknown schedule {schedule}")
        if balance not in ("units", "cost"):
            raise ValueError(f"unknown balance {balance}")
        self.g, self.m, self.schedule = group, micro_batches, schedule
        units = model.units()
        if balance == "cost":
            self.ranges = split_by_cost(unit_costs(units, model.config.seq), group.size)
        else:
            self.ranges = split_units(len(units), group.size)
        lo, hi = self.ranges[group.rank]
        self.units = torch.nn.ModuleList(units[lo:hi])
        self.first, self.last = group.rank == 0, group.rank == group.size - 1
        self.dim = model.config.dim
        self.kernels = getattr(model.config, "kernels", "torch")
        self.timeline = timeline or Timeline(enabled=False)
        self.act_dtype = None  # None: the dtype of this stage's parameters
        self.wire = None  # None: NCCL lanes between GPU stages, the group's own send / recv elsewhere

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
        wire = self.wire
        if wire is None and dev.type == "cuda" and getattr(g, "transport", "device") == "device" and g.size > 1:
            wire = g._p2p()
        if wire is not None:
            return self._run_on_lanes(wire, actions, xs, ys, dev, dtype, shape)
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

    def _run_on_lanes(self, wire, actions, xs, ys, dev, dtype, shape):
        """GPU stages over NCCL.  Nothing here blocks the host: a transfer is ordered after the compute stream when it
        is issued, and claiming a received tensor makes the compute stream wait for it.  Sends are collected and
        awaited when the step ends.

        GPipe: activations travel down on one communicator and gradients up on another, and a stage never has both
        phases in flight, so receives are posted ahead of time -- the next one of a kind as soon as the previous one
        has been claimed (on a middle stage: as soon as the send that forwards it has been issued, so that on the
        lane's stream a receive never stands in front of the send its own sender is waiting for).

        1F1B: in the steady state a stage sends one way and receives the other at the same moment.  The pair is ONE
        grouped NCCL call on one communicator (both directions inside one kernel), issued in the schedule's order,
        which every stage shares; it needs no second NCCL kernel to make progress next to it.  Receives posted ahead
        on a second communicator were measured to stall at 8 MB messages on two B200s (each side spinning in a
        receive while the send that would release the other waited to be scheduled), so this schedule does not
        use them."""
        up, down = self.g.rank - 1, self.g.rank + 1
        wire.lane("act")  # first use: both communicators exist and every neighbour pair is connected before real traffic
        ahead = self.schedule == "gpipe"
        takes_act = {"recv_act", "send_grad_recv_act"}
        takes_grad = {"recv_grad", "send_act_recv_grad"}
        due = {"act": 0 if self.first else sum(a[0] in takes_act for a in actions),
               "grad": 0 if self.last else sum(a[0] in takes_grad for a in actions)}
        source = {"act": up, "grad": down}
        forwards = {"act": not self.last, "grad": not self.first}  # does this stage pass that kind on?
        posted = {"act": None, "grad": None}
        owed = {"act": False, "grad": False}  # a receive to post once the matching send has been issued

        def post(kind):
            owed[kind] = False
            if due[kind]:
                due[kind] -= 1
                posted[kind] = wire.post_recv(shape, dtype, source[kind], kind)

        def claim(kind):
            if posted[kind] is None:
                post(kind)  # the first of its kind in a step is posted when the schedule first asks for it
            handle, posted[kind] = posted[kind], None
            tensor = wire.claim(*handle)
            if forwards[kind]:
                owed[kind] = True
            else:
                post(kind)  # the next one arrives while this one is being used
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
                continue
            if kind == "B":
                i = a[1]
                with self.timeline.span(f"B{i}"):
                    inp, res = saved.pop(i)
                    if self.last:
                        res.backward()
                    else:
                        res.backward(grad)
                    grad = None if self.first else inp.grad
                continue
            send_act = kind in ("send_act", "send_act_recv_grad") and not self.last
            send_grad = kind in ("send_grad", "send_grad_recv_act") and not self.first
            recv_act = kind in takes_act and not self.first
            recv_grad = kind in takes_grad and not self.last
            if not ahead:
                sends = ([(out.detach().contiguous(), down)] if send_act else []) + ([(grad.contiguous(), up)] if send_grad else [])
                recvs = ([up] if recv_act else []) + ([down] if recv_grad else [])
                if sends or recvs:
                    work, kept, received = wire.exchange(sends, recvs, shape, dtype)
                    if recv_act:
                        act = wire.claim(work, received[0])  # orders this stage after the whole exchange
                    elif recv_grad:
                        grad = wire.claim(work, received[0])
                    else:
                        in_flight.append((work, kept))
                continue
            if send_act:
                in_flight.append(wire.post_send(out.detach().contiguous(), down, "act"))
                if owed["act"]:
                    post("act")
            if send_grad:
                in_flight.append(wire.post_send(grad.contiguous(), up, "grad"))
                if owed["grad"]:
                    post("grad")
            if recv_act:
                act = claim("act")
            if recv_grad:
                grad = claim("grad")
        for work, _kept in in_flight:
            work.wait()
        return sum(losses) if self.last else None
