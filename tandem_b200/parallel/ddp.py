"""Data parallelism with bucketed, overlapped gradient averaging.

Same contract as the reference's tandem/ddp.py:35-129 (and torch's DDP): every
rank starts from rank 0's weights; gradients are views into flat buckets of
about `bucket_bytes`; a bucket's all-reduce (op="avg": divide, then sum) is
submitted as soon as its last gradient is produced, buckets are submitted
strictly in index order so all ranks issue the same sequence, and after the
first backward the buckets are rebuilt in the order gradients really arrived.
`no_sync()` accumulates locally.

What is different underneath on GPUs: bucket storage comes from the group's
symmetric heap, so the all-reduce kernel reads the peers' buckets in place over
NVLink with the divide fused into its loads (no staging copy, no separate div_
kernel), on a high-priority stream while backward continues; the initial
broadcast is one transfer per dtype instead of one per parameter; and gradients
that autograd produced outside a bucket are packed by one multi-tensor kernel
per bucket instead of one copy per parameter.
"""

import contextlib

import torch
from torch.autograd import Variable


class Bucket:
    def __init__(self, params, group):
        self.params = params
        first = params[0]
        total = sum(p.numel() for p in params)
        self.flat = group.empty(total, first.dtype, first.device)
        self.views, at = {}, 0
        for p in params:
            self.views[p] = self.flat[at:at + p.numel()].view_as(p)
            at += p.numel()
        self.ready = 0
        self.work = None
        self.loose = []  # parameters whose fresh gradient still sits outside the bucket


class DDP(torch.nn.Module):
    def __init__(self, module, group, bucket_bytes=25 << 20, overlap=True, rebuild=True):
        super().__init__()
        self.module = module
        self.g = group
        self.bucket_bytes = bucket_bytes
        self.overlap = overlap
        self._rebuild = rebuild
        self.params = [p for p in module.parameters() if p.requires_grad]
        self._broadcast_initial()
        # Until a backward shows the real order, assume reverse registration order.
        self._make_buckets(list(reversed(self.params)))
        self._sync = True
        self._order = []
        self._queued = False
        for p in self.params:
            p.register_post_accumulate_grad_hook(self._on_grad)

    @torch.no_grad()
    def _broadcast_initial(self):
        """Rank 0's weights to everyone, one flat transfer per dtype."""
        by_dtype = {}
        for p in self.params:
            by_dtype.setdefault((p.dtype, p.device), []).append(p)
        for ps in by_dtype.values():
            flat = torch.cat([p.detach().reshape(-1) for p in ps])
            self.g.broadcast(flat, root=0)
            at = 0
            for p in ps:
                p.copy_(flat[at:at + p.numel()].view_as(p))
                at += p.numel()

    def _make_buckets(self, order):
        self.buckets, self.bucket_of = [], {}
        current, size = [], 0
        for p in order:
            nbytes = p.numel() * p.element_size()
            if current and (size + nbytes > self.bucket_bytes or p.dtype != current[0].dtype):
                self._close_bucket(current)
                current, size = [], 0
            current.append(p)
            size += nbytes
        if current:
            self._close_bucket(current)
        self._next = 0

    def _close_bucket(self, params):
        b = Bucket(params, self.g)
        for p in params:
            self.bucket_of[p] = b
        self.buckets.append(b)

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    @contextlib.contextmanager
    def no_sync(self):
        """Backward passes inside only accumulate; the next one outside reduces the sum."""
        before, self._sync = self._sync, False
        try:
            yield
        finally:
            self._sync = before

    def zero_grad(self):
        """Zeroes the buckets and keeps every .grad a bucket view, so the next
        backward accumulates straight into the buckets (no pack step).
        `optimizer.zero_grad()` (set_to_none) works too: the hook then moves each
        fresh gradient into its bucket."""
        for b in self.buckets:
            b.flat.zero_()
            for p in b.params:
                p.grad = b.views[p]

    def _pack(self, b):
        """Moves gradients that autograd left outside the bucket into it."""
        if not b.loose:
            return
        from ..ops import pack_into

        pack_into(b.flat, [(b.views[p], p.grad) for p in b.loose])
        for p in b.loose:
            p.grad = b.views[p]
        b.loose = []

    def _on_grad(self, p):
        b = self.bucket_of[p]
        if p.grad is not b.views[p]:
            b.loose.append(p)
            if not p.grad.is_cuda or not self._sync:
                self._pack(b)  # CPU, or accumulating: the view must hold the sum before the next backward
        if not self._sync:
            return
        if not self._queued:
            self._queued = True
            Variable._execution_engine.queue_callback(self._finish_backward)
        if self._rebuild:
            self._order.append(p)
        b.ready += 1
        while self._next < len(self.buckets) and self.buckets[self._next].ready == len(self.buckets[self._next].params):
            nb = self.buckets[self._next]
            self._pack(nb)
            nb.work = self.g.all_reduce(nb.flat, op="avg", async_op=True)
            if not self.overlap:
                nb.work.wait()
            self._next += 1

    def _finish_backward(self):
        self._queued = False
        missing = [b for b in self.buckets if b.ready != len(b.params)]
        if missing:
            for b in self.buckets:
                b.ready, b.work, b.loose = 0, None, []
            self._next, self._order = 0, []
            shapes = [tuple(p.shape) for b in missing for p in b.params if p.grad is None]
            raise RuntimeError(f"tandem_b200 DDP: some parameters received no gradient ({shapes[:3]}...); "
                               "every parameter must be used in the forward pass")
        for b in self.buckets:
            b.work.wait()
            b.ready, b.work = 0, None
        self._next = 0
        if self._rebuild and len(self._order) == len(self.params):
            order, self._order, self._rebuild = self._order, [], False
            grads = {p: p.grad.detach().clone() for p in self.params}
            self._make_buckets(order)
            for p in self.params:
                view = self.bucket_of[p].views[p]
                view.copy_(grads[p])
                p.grad = view
        else:
            self._order = []


class BucketAdamW:
    """AdamW over a DDP wrapper's buckets: one fused kernel per bucket.

    Parameters are re-laid as views of one flat buffer per bucket, in the
    bucket's gradient order, so a bucket's {parameters, gradients, moments} are
    four parallel flat arrays and a step is `len(buckets)` launches instead of
    nine ATen kernels per parameter (torch.optim.AdamW(foreach=False), which the
    reference pairs with its DDP: bench/run.py:102).  With 16-bit parameters the
    optimizer keeps fp32 master weights and moments and writes the 16-bit
    parameters back as a shadow copy in the same kernel.

    Create it once the buckets are final: pass rebuild=False to DDP, or create it
    after the first backward.
    """

    def __init__(self, ddp, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2):
        from .optim import ShardedAdamW

        self.ddp = ddp
        self.rule = ShardedAdamW(lr, betas, eps, weight_decay)
        self.step_count = 0.0
        self.slots = []
        with torch.no_grad():
            for b in ddp.buckets:
                first = b.params[0]
                flat = torch.empty(b.flat.numel(), dtype=first.dtype, device=first.device)
                at = 0
                for p in b.params:
                    view = flat[at:at + p.numel()].view_as(p)
                    view.copy_(p)
                    p.data = view
                    at += p.numel()
                master = flat if first.dtype == torch.float32 else flat.float()
                self.slots.append({"bucket": b, "flat": flat, "master": master, "m": torch.zeros_like(master),
                                   "v": torch.zeros_like(master)})
        dev = ddp.params[0].device
        if dev.type == "cuda":  # step counter and per-step constants live on the device: the step is graph-capturable
            self._step_dev = torch.zeros(1, dtype=torch.float64, device=dev)
            self._scalars_dev = torch.zeros(8, dtype=torch.float32, device=dev)

    @torch.no_grad()
    def step(self):
        from ..ops import fused_adamw

        if self.ddp._rebuild:
            raise RuntimeError("the buckets are not final yet: create BucketAdamW after the first backward or use rebuild=False")
        self.step_count += 1.0
        sc = self.rule.scalars(self.step_count)
        on_gpu = self.slots[0]["bucket"].flat.is_cuda
        if on_gpu:
            from ..ops.elementwise import adam_prepare, adamw_step_dev

            adam_prepare(self._step_dev, (self.rule.lr, self.rule.betas, self.rule.eps, self.rule.weight_decay), self._scalars_dev)
        for s in self.slots:
            b = s["bucket"]
            shadow = None if s["master"] is s["flat"] else s["flat"]
            if on_gpu:
                adamw_step_dev(s["master"], b.flat, s["m"], s["v"], self._scalars_dev, shadow)
            else:
                self.rule.state["b"] = [self.step_count - 1.0, s["m"], s["v"]]
                self.rule.update("b", s["master"], b.flat.float(), shadow)

    def zero_grad(self):
        self.ddp.zero_grad()

    def state_bytes(self):
        return sum(s[k].numel() * s[k].element_size() for s in self.slots for k in ("m", "v"))
