"""Data parallelism over gradient arenas.

What a user sees is the contract of the reference's tandem/ddp.py:35-129 (and of
torch's DDP): every rank starts from rank 0's weights, gradients are averaged
bucket by bucket while backward is still running (op="avg": divide, then sum),
every rank issues the same sequence of collectives, the bucket order follows the
order in which gradients really arrive, `no_sync()` accumulates locally, and a
parameter that received no gradient is an error.

How it is laid out here.  All gradients of one dtype live in ONE allocation, the
arena, taken once from the group's symmetric heap (peer-mapped on GPU ranks).  A
bucket ("span") is nothing but a slice [lo, hi) of its arena plus the parameters
whose gradient slots fall inside it, so its collective runs in place on memory
every peer can already address: no staging copy, no second buffer, and the
divide is fused into the kernel's loads.  Learning the arrival order re-plans
the offsets INSIDE the arena (one temporary snapshot carries the gradients over);
nothing is allocated or released on the heap after construction.

Spans are reduced through a pluggable reducer.  The default averages a span with
one all-reduce.  `ShardedBucketAdamW` replaces it with reduce-scatter + AdamW on
the freshly reduced chunk (inside the reduce-scatter kernel on GPUs) + all-gather
of the updated parameters: the same NVLink bytes as the all-reduce, 1/n of the
optimizer's memory traffic and state, identical values.
"""

import collections
import contextlib

import torch
from torch.autograd import Variable


class Span:
    """A slice of an arena that one collective reduces: the unit of overlap."""

    __slots__ = ("arena", "lo", "hi", "params", "slot", "missing", "stray", "flight")

    def __init__(self, arena, lo, hi, params):
        self.arena, self.lo, self.hi, self.params = arena, lo, hi, params
        self.slot = {p: arena.slot_of(p) for p in params}  # parameter -> its gradient's home, shaped like the parameter
        self.missing = len(params)  # gradients of this backward still to come
        self.stray = []             # parameters whose fresh gradient autograd left outside its slot
        self.flight = None          # the collective in flight, if any

    @property
    def flat(self):
        return self.arena.flat[self.lo:self.hi]

    def rearm(self):
        self.missing, self.stray, self.flight = len(self.params), [], None


class GradArena:
    """Every gradient of one (dtype, device) in one flat allocation; `where[p]` is p's offset."""

    def __init__(self, group, params):
        first = params[0]
        self.params = list(params)
        self.flat = group.empty(sum(p.numel() for p in params), first.dtype, first.device)
        self.where = {}

    def place(self, order):
        """Assigns offsets in the given order (a permutation of this arena's parameters)."""
        at = 0
        for p in order:
            self.where[p] = at
            at += p.numel()

    def slot_of(self, p):
        a = self.where[p]
        return self.flat[a:a + p.numel()].view_as(p)

    def snapshot(self):
        """(copy of the gradients, copy of the offsets): what carry_over() needs after a re-plan."""
        return self.flat.clone(), dict(self.where)

    def carry_over(self, snapshot):
        """After place() with a new order: moves every gradient from its old offset to its new one."""
        old_flat, old_where = snapshot
        for p in self.params:
            n = p.numel()
            self.flat[self.where[p]:self.where[p] + n].copy_(old_flat[old_where[p]:old_where[p] + n])


class AllReduceSpans:
    """Default reducer: one averaging all-reduce per span, in place on the arena."""

    def __init__(self, group):
        self.g = group

    def __call__(self, span):
        return self.g.all_reduce(span.flat, op="avg", async_op=True)


class DDP(torch.nn.Module):
    def __init__(self, module, group, bucket_bytes=25 << 20, overlap=True, rebuild=True):
        super().__init__()
        self.module = module
        self.g = group
        self.bucket_bytes = bucket_bytes
        self.overlap = overlap
        self.params = [p for p in module.parameters() if p.requires_grad]
        self._share_initial_weights()
        self.arenas = {}
        for p in self.params:
            self.arenas.setdefault((p.dtype, p.device), []).append(p)
        self.arenas = {key: GradArena(group, ps) for key, ps in self.arenas.items()}
        # Until a backward shows the real order, expect gradients in reverse registration order.
        self._plan(list(reversed(self.params)))
        self.reducer = AllReduceSpans(group)
        self._reducing = True            # False inside no_sync()
        self._learning = bool(rebuild)   # still recording the arrival order of the first reduced backward
        self._seen = []
        self._drain_armed = False
        for p in self.params:
            p.register_post_accumulate_grad_hook(self._arrived)

    # ------------------------------------------------------------------ set-up
    @torch.no_grad()
    def _share_initial_weights(self):
        """Rank 0's weights to everyone: one flat transfer per dtype instead of one per parameter."""
        groups = {}
        for p in self.params:
            groups.setdefault((p.dtype, p.device), []).append(p)
        for ps in groups.values():
            packed = torch.cat([p.detach().reshape(-1) for p in ps])
            self.g.broadcast(packed, root=0)
            at = 0
            for p in ps:
                p.copy_(packed[at:at + p.numel()].view_as(p))
                at += p.numel()

    def _plan(self, order):
        """Cuts `order` into spans of about bucket_bytes (a span never mixes dtypes) and places every
        arena's parameters in that order, so each span is one contiguous slice."""
        for key, arena in self.arenas.items():
            arena.place([p for p in order if (p.dtype, p.device) == key])
        self.buckets, self._span_of = [], {}
        run, size = [], 0

        def close():
            arena = self.arenas[(run[0].dtype, run[0].device)]
            lo = arena.where[run[0]]
            span = Span(arena, lo, lo + sum(p.numel() for p in run), list(run))
            self.buckets.append(span)
            for p in run:
                self._span_of[p] = span

        for p in order:
            nbytes = p.numel() * p.element_size()
            if run and (size + nbytes > self.bucket_bytes or (p.dtype, p.device) != (run[0].dtype, run[0].device)):
                close()
                run, size = [], 0
            run.append(p)
            size += nbytes
        if run:
            close()
        self._queue = collections.deque(self.buckets)

    @property
    def rebuilding(self):
        """True until the span layout is final (optimizers that mirror the layout wait for that)."""
        return self._learning

    # ------------------------------------------------------------------ the wrapper's surface
    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    @contextlib.contextmanager
    def no_sync(self):
        """Backward passes inside only accumulate; the next one outside reduces the sum."""
        was, self._reducing = self._reducing, False
        try:
            yield
        finally:
            self._reducing = was

    def zero_grad(self):
        """Zeroes the arenas and points every .grad at its slot, so the next backward accumulates
        straight into the arena (no pack step).  `optimizer.zero_grad()` (set_to_none) works too:
        fresh gradients are then moved into their slots span by span."""
        for arena in self.arenas.values():
            arena.flat.zero_()
        for span in self.buckets:
            for p in span.params:
                p.grad = span.slot[p]

    # ------------------------------------------------------------------ backward
    def _settle(self, span):
        """Moves the span's stray gradients into their slots: one multi-tensor copy on a GPU
        (the reference copies parameter by parameter: tandem/ddp.py:92-94)."""
        if not span.stray:
            return
        from ..ops import pack_into

        pack_into(span.flat, [(span.slot[p], p.grad) for p in span.stray])
        for p in span.stray:
            p.grad = span.slot[p]
        span.stray = []

    def _arrived(self, p):
        span = self._span_of[p]
        if p.grad.data_ptr() != span.slot[p].data_ptr():
            span.stray.append(p)
            if not p.grad.is_cuda or not self._reducing:
                self._settle(span)  # CPU, or accumulating: the slot must hold the sum before the next backward
        if not self._reducing:
            return
        if not self._drain_armed:
            self._drain_armed = True
            Variable._execution_engine.queue_callback(self._drain)
        if self._learning:
            self._seen.append(p)
        span.missing -= 1
        # Spans go out strictly in plan order, whichever fills first: all ranks issue the same sequence.
        while self._queue and self._queue[0].missing == 0:
            head = self._queue.popleft()
            self._settle(head)
            head.flight = self.reducer(head)
            if not self.overlap:
                head.flight.wait()

    def _drain(self):
        """End of backward: every span's collective has been issued (or something is missing)."""
        self._drain_armed = False
        starved = [s for s in self.buckets if s.missing]
        if starved:
            shapes = [tuple(p.shape) for s in starved for p in s.params if p.grad is None]
            for s in self.buckets:
                s.rearm()
            self._queue = collections.deque(self.buckets)
            self._seen = []
            raise RuntimeError(f"tandem_b200 DDP: some parameters received no gradient ({shapes[:3]}...); "
                               "every parameter must be used in the forward pass")
        for s in self.buckets:
            s.flight.wait()
            s.rearm()
        self._queue = collections.deque(self.buckets)
        seen, self._seen = self._seen, []
        if self._learning and len(seen) == len(self.params):
            self._learning = False
            self._adopt_order(seen)

    @torch.no_grad()
    def _adopt_order(self, order):
        """The spans, re-cut in the order gradients really arrived; gradients move with their slots."""
        kept = {key: arena.snapshot() for key, arena in self.arenas.items()}
        self._plan(order)
        for key, arena in self.arenas.items():
            arena.carry_over(kept[key])
        for span in self.buckets:
            for p in span.params:
                p.grad = span.slot[p]


def _mirror_parameters(ddp, symmetric):
    """Re-lays the parameters as views of one flat buffer per arena, at their gradients' offsets, so a span's
    parameters, gradients and optimizer state are parallel slices.  Returns {arena: flat parameter buffer}."""
    if ddp.rebuilding:
        raise RuntimeError("the span layout is not final yet: create the optimizer after the first backward or pass "
                           "rebuild=False to DDP")
    out = {}
    with torch.no_grad():
        for arena in ddp.arenas.values():
            first = arena.params[0]
            n = arena.flat.numel()
            flat = ddp.g.empty(n, first.dtype, first.device) if symmetric else torch.empty(n, dtype=first.dtype, device=first.device)
            for p in arena.params:
                view = flat[arena.where[p]:arena.where[p] + p.numel()].view_as(p)
                view.copy_(p)
                p.data = view
            out[arena] = flat
    return out


class _AfterEvent:
    """What a reducer returns when its last piece of work ran on a stream of its own: waiting is a stream dependency."""

    def __init__(self, event, device):
        self._event, self._device = event, device

    def wait(self):
        torch.cuda.current_stream(self._device).wait_event(self._event)

    def is_completed(self):
        return self._event.query()


class BucketAdamW:
    """AdamW over a DDP wrapper's spans, replicated on every rank: one fused kernel per span.

    A span's {parameters, gradients, moments} are four parallel flat slices, so a step is `len(buckets)`
    launches instead of nine ATen kernels per parameter (torch.optim.AdamW(foreach=False), which the
    reference pairs with its DDP: bench/run.py:102).  With 16-bit parameters the optimizer keeps fp32
    master weights and moments and writes the 16-bit parameters back in the same kernel.  On CPU ranks
    it runs torch's operation sequence, so results equal torch's per-parameter AdamW bit for bit.

    Create it once the span layout is final: pass rebuild=False to DDP, or create it after the first backward.

    during_backward: a span is updated as soon as its all-reduce has finished (on GPU ranks on a stream of its own
    beside the rest of backward) instead of all spans after backward (the update streams through HBM while the
    remaining backward GEMMs keep the tensor pipes busy; nothing in backward reads a parameter again once its
    gradient is complete).  `step()` then only closes the step.  As with the sharded form, every backward that
    reduces also updates: accumulate over several backward passes under `no_sync()`.
    """

    def __init__(self, ddp, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, during_backward=False):
        from .optim import ShardedAdamW

        self.ddp = ddp
        self.rule = ShardedAdamW(lr, betas, eps, weight_decay)
        self.step_count = 0.0
        flats = _mirror_parameters(ddp, symmetric=False)
        self.slots = []
        for span in ddp.buckets:
            flat = flats[span.arena][span.lo:span.hi]
            master = flat if flat.dtype == torch.float32 else flat.float()
            self.slots.append({"bucket": span, "flat": flat, "master": master, "m": torch.zeros_like(master), "v": torch.zeros_like(master)})
        dev = ddp.params[0].device
        self.during_backward = bool(during_backward)
        self._on_gpu = dev.type == "cuda"
        if self._on_gpu:  # step counter and per-step constants live on the device: the step is graph-capturable
            self._step_dev = torch.zeros(1, dtype=torch.float64, device=dev)
            self._scalars_dev = torch.zeros(8, dtype=torch.float32, device=dev)
        if self.during_backward:
            self._slot_of = {id(s["bucket"]): s for s in self.slots}
            self._reduce = ddp.reducer
            if self._on_gpu:
                self._update_stream = torch.cuda.Stream(dev)
                self._prepare_next()  # the constants of step 1
            ddp.reducer = self._reduce_then_update

    def _prepare_next(self):
        from ..ops.elementwise import adam_prepare

        adam_prepare(self._step_dev, (self.rule.lr, self.rule.betas, self.rule.eps, self.rule.weight_decay), self._scalars_dev)

    def _reduce_then_update(self, span):
        from ..ops.elementwise import adamw_step_dev

        s = self._slot_of[id(span)]
        reduced = self._reduce(span)
        if not self._on_gpu:  # CPU ranks: the same order of events, with torch's operation sequence
            reduced.wait()
            shadow = None if s["master"] is s["flat"] else s["flat"]
            with torch.no_grad():
                self.rule.state["b"] = [self.step_count, s["m"], s["v"]]
                self.rule.update("b", s["master"], span.flat.float(), shadow)
            return reduced
        dev = s["flat"].device
        side = self._update_stream
        side.wait_stream(torch.cuda.current_stream(dev))  # the gradients, and every use of these parameters in backward
        with torch.cuda.stream(side), torch.no_grad():
            reduced.wait()  # a stream dependency on the all-reduce
            shadow = None if s["master"] is s["flat"] else s["flat"]
            adamw_step_dev(s["master"], span.flat, s["m"], s["v"], self._scalars_dev, shadow)
            done = torch.cuda.Event()
            done.record(side)
        return _AfterEvent(done, dev)

    @torch.no_grad()
    def step(self):
        self.step_count += 1.0
        if self.during_backward:
            if self._on_gpu:
                self._prepare_next()  # the updates ran during backward; these are the next step's constants
            return
        on_gpu = self.slots[0]["flat"].is_cuda
        if on_gpu:
            from ..ops.elementwise import adam_prepare, adamw_step_dev

            adam_prepare(self._step_dev, (self.rule.lr, self.rule.betas, self.rule.eps, self.rule.weight_decay), self._scalars_dev)
        for s in self.slots:
            grad = s["bucket"].flat
            shadow = None if s["master"] is s["flat"] else s["flat"]
            if on_gpu:
                adamw_step_dev(s["master"], grad, s["m"], s["v"], self._scalars_dev, shadow)
            else:
                self.rule.state["b"] = [self.step_count - 1.0, s["m"], s["v"]]
                self.rule.update("b", s["master"], grad.float(), shadow)

    def zero_grad(self):
        self.ddp.zero_grad()

    def state_bytes(self):
        return sum(s[k].numel() * s[k].element_size() for s in self.slots for k in ("m", "v"))


class ShardedBucketAdamW:
    """AdamW for a DDP wrapper with the update sharded over the ranks, span by span, during backward.

    Rank r owns chunk r (torch.tensor_split) of every span: it keeps fp32 master weights and moments for
    that chunk only.  The wrapper's reducer becomes: reduce-scatter the span's gradients (average), apply
    AdamW to the owned chunk -- inside the reduce-scatter kernel on GPU ranks, on the values it has just
    reduced -- and all-gather the span's updated parameters.  The bytes on the wire equal the all-reduce's;
    the optimizer reads and writes 1/n of what a replicated step does, and every rank ends with the same
    parameters as `BucketAdamW` produces.  By the time backward returns the new parameters are in
    place; `step()` only advances the step counter (and prepares the next step's bias corrections on the
    device), so the whole step stays capturable as a CUDA graph.

    Not compatible with accumulating gradients over several backward passes that each reduce (use
    `no_sync()` for all but the last, as with any DDP).
    """

    def __init__(self, ddp, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2):
        from .optim import ShardedAdamW
        from .zero import split_sizes

        self.ddp, self.g = ddp, ddp.g
        self.rule = ShardedAdamW(lr, betas, eps, weight_decay)
        self.step_count = 0.0
        flats = _mirror_parameters(ddp, symmetric=True)
        n, r = self.g.size, self.g.rank
        self.slots = []
        for span in ddp.buckets:
            flat = flats[span.arena][span.lo:span.hi]
            sizes = split_sizes(span.hi - span.lo, n)
            lo = sum(sizes[:r])
            mine = flat[lo:lo + sizes[r]]
            master = mine if mine.dtype == torch.float32 else mine.float()  # fp32 parameters are their own master
            self.slots.append({"bucket": span, "flat": flat, "sizes": sizes, "lo": lo, "master": master,
                               "m": torch.zeros_like(master), "v": torch.zeros_like(master)})
        self._slot_of = {id(s["bucket"]): s for s in self.slots}
        dev = ddp.params[0].device
        kinds = {p.dtype for p in ddp.params}
        self._fused = bool(dev.type == "cuda" and getattr(self.g, "fused", False) and kinds <= {torch.float32, torch.bfloat16})
        if self._fused:
            from ..ops.elementwise import adam_prepare

            self._step_dev = torch.zeros(1, dtype=torch.float64, device=dev)
            self._scalars_dev = torch.zeros(8, dtype=torch.float32, device=dev)
            self._prepare = lambda: adam_prepare(self._step_dev, (lr, betas, eps, weight_decay), self._scalars_dev)
            self._prepare()  # the constants of step 1
        ddp.reducer = self._reduce_update_gather

    def _reduce_update_gather(self, span):
        s = self._slot_of[id(span)]
        count = s["sizes"][self.g.rank]
        own = s["flat"][s["lo"]:s["lo"] + count]
        if self._fused:
            from .symm import AdamArgs

            shadow = own if own.dtype == torch.bfloat16 else None  # fp32: the kernel updates the parameter chunk in place
            args = AdamArgs.on_device(s["master"], s["m"], s["v"], self._scalars_dev, shadow)
            self.g.reduce_scatter(span.flat, s["sizes"], op="avg", async_op=True, adam=args)
        else:
            mine = self.g.reduce_scatter(span.flat, s["sizes"], op="avg")
            if count:
                self.rule.state["s"] = [self.step_count, s["m"], s["v"]]
                self.rule.update("s", s["master"], mine.to(s["master"].dtype))
                if s["master"].data_ptr() != own.data_ptr():
                    own.copy_(s["master"])
        return self.g.all_gather(s["flat"], s["sizes"], async_op=True)

    @torch.no_grad()
    def step(self):
        """The update ran during backward; this closes the step."""
        self.step_count += 1.0
        if self._fused:
            self._prepare()  # bias corrections of the next step, computed on the device

    def zero_grad(self):
        for p in self.ddp.params:
            p.grad = None

    def state_bytes(self):
        return sum(s[k].numel() * s[k].element_size() for s in self.slots for k in ("m", "v"))
