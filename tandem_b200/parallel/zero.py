"""ZeRO stages 1-3: data parallelism that shards optimizer state, then gradients,
then parameters (Rajbhandari et al., 2020).

Contract and flat layouts follow the reference's tandem/zero.py:29-336:
  ZeRO(stage=1|2)  all parameters are views of one flat buffer in
                   module.parameters() order; rank r owns chunk r of
                   torch.tensor_split(numel, world).  Stage 1 all-reduces bucket
                   slices of a full flat gradient; stage 2 reduce-scatters each
                   bucket with per-rank sizes = the overlap of the bucket's range
                   with each shard (often zero) and keeps only a shard of the
                   gradient.  step() = sharded AdamW + all-gather of the buffer.
  FSDP             the same per unit of model.units(): a unit's full parameters
                   exist only around its forward and its backward; the next
                   unit's gather is started early; a unit's gradients are
                   reduce-scattered as soon as they are complete.
Train with: loss = z(x, y); loss.backward(); z.step(); z.zero_grad().

What runs on GPU ranks (group.fused), beyond that contract:

  Memory.  The flat parameter buffer (stages 1/2), each bucket's gradient staging and
  each unit's parameter shard (stage 3) come from the group's symmetric heap, so every
  peer can address them; every rank allocates the same sizes in the same order (a unit's
  shard is allocated at the largest rank's size), which keeps heap offsets identical.

  Gradients.  Autograd's gradients are not copied into the staging buffer one by one:
  the (view, gradient) pairs of a bucket or unit are collected and packed by ONE
  multi-tensor kernel when its last gradient has arrived.  The reduce-scatter is then a
  single kernel that reads the peers' staging buffers in place, divides each operand
  as it is loaded, and finishes with an epilogue instead of a separate pass:
  `accumulate_into=` adds the reduced chunk to the gradient shard (stage 2/3), and with
  `ZeRO(fused_step=True)` the AdamW update itself runs there, on the chunk that was just
  reduced (fp32 master weights and moments, bf16 shadow written back), so step() only
  has to all-gather the parameters.

  Parameters (stage 3).  A unit's shards only change inside step(), and step() is fenced
  by device barriers on both sides; gathers of a unit therefore need no handshake at
  all: each rank pulls the peers' shards with one kernel that opens with a system-scope
  fence (gather_shards), on the communication stream, one unit ahead of the compute.
  With `FSDP(fuse_gather_gemm=True)` a block's qkv weight and bias are not gathered
  ahead at all in the forward pass: the unit is pulled in two parts around them
  (what precedes the weight is awaited before the first LayerNorm, the rest while the
  GEMM runs), the qkv GEMM kernel fetches its own weight from the owners' shards while
  it multiplies (ops.gemm.GatheredLinear, registered in ops.gemm.GATHERED under the
  weight's address), and the stream waits for the second part right after that GEMM.

  Mixed precision.  With bf16 parameters the optimizer keeps an fp32 master copy of
  each shard next to the moments (ShardedAdamW.master); gradients stay bf16 on the wire.

On CPU ranks the same classes run the reference's sequence of collectives and torch
operations, which is what makes them bit-identical to torch DDP + AdamW.
"""

import warnings

import torch
from torch.autograd import Variable

from .optim import ShardedAdamW


def split_sizes(numel, world):
    """Chunk lengths of torch.tensor_split(numel, world)."""
    base, extra = divmod(numel, world)
    return [base + (1 if r < extra else 0) for r in range(world)]


class FlatLayout:
    """Offsets of parameters inside one flat buffer, and the rank shards of it."""

    def __init__(self, params, world, rank):
        self.params = params
        self.offset, at = {}, 0
        for p in params:
            self.offset[p] = at
            at += p.numel()
        self.numel = at
        self.sizes = split_sizes(at, world)
        self.lo = sum(self.sizes[:rank])
        self.hi = self.lo + self.sizes[rank]

    def span(self, p):
        return self.offset[p], self.offset[p] + p.numel()

    def bucket_sizes(self, a, b):
        """How many elements of the flat range [a, b) fall in each rank's shard."""
        out, lo = [], 0
        for s in self.sizes:
            out.append(max(0, min(b, lo + s) - max(a, lo)))
            lo += s
        return out


class _Range:
    """A contiguous run of parameters reduced together."""

    def __init__(self, params, a, b):
        self.params, self.a, self.b = params, a, b
        self.ready = 0
        self.work = None
        self.staging = None
        self.fused_acc = False
        self.loose = []  # (staging view, gradient) pairs waiting for the bucket's one pack kernel


def _flatten_into(buf, layout):
    for p in layout.params:
        a, b = layout.span(p)
        buf[a:b].copy_(p.detach().reshape(-1))


def _point_into(buf, layout):
    for p in layout.params:
        a, b = layout.span(p)
        p.data = buf[a:b].view_as(p)


class ZeRO(torch.nn.Module):
    """Stages 1 and 2."""

    def __init__(self, module, group, stage=1, optimizer=None, bucket_bytes=25 << 20, fused_step=False):
        """fused_step (stage 2, GPU kernels only): apply the sharded AdamW update inside each bucket's
        reduce-scatter kernel, on the freshly reduced gradient chunk, instead of in step().  One pass over
        the gradients instead of three (reduce, accumulate, optimizer); step() then only all-gathers the
        parameters.  Not compatible with accumulating gradients over several backward passes."""
        super().__init__()
        if stage not in (1, 2):
            raise ValueError("ZeRO handles stages 1 and 2; stage 3 is FSDP")
        self.module, self.g, self.stage = module, group, stage
        self.fused_step = bool(fused_step) and stage == 2 and group.fused
        self.opt = optimizer or ShardedAdamW()
        params = [p for p in module.parameters() if p.requires_grad]
        dev, dtype = params[0].device, params[0].dtype
        if any(p.dtype != dtype or p.device != dev for p in params):
            raise ValueError("ZeRO needs all parameters on one device with one dtype")
        self.flat = FlatLayout(params, group.size, group.rank)
        self.buf = group.empty(self.flat.numel, dtype, dev)
        with torch.no_grad():
            _flatten_into(self.buf, self.flat)
            group.broadcast(self.buf, root=0)
            _point_into(self.buf, self.flat)
        if stage == 1:
            self.grad = group.empty(self.flat.numel, dtype, dev)
        else:
            self.grad_shard = torch.zeros(self.flat.hi - self.flat.lo, device=dev, dtype=dtype)
        # Ranges run from the end of the buffer, the order backward produces gradients in.
        self.buckets, self.bucket_of = [], {}
        run, size = [], 0
        for p in reversed(params):
            nbytes = p.numel() * p.element_size()
            if run and size + nbytes > bucket_bytes:
                self._close(run)
                run, size = [], 0
            run.append(p)
            size += nbytes
        if run:
            self._close(run)
        self._next = 0
        self._queued = False
        for p in params:
            p.register_post_accumulate_grad_hook(self._on_grad)

    def _close(self, params):
        a = min(self.flat.offset[p] for p in params)
        b = max(self.flat.offset[p] + p.numel() for p in params)
        r = _Range(params, a, b)
        for p in params:
            self.bucket_of[p] = r
        self.buckets.append(r)

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def _on_grad(self, p):
        r = self.bucket_of[p]
        a, b = self.flat.span(p)
        if self.stage == 1:
            view = self.grad[a:b].view_as(p)
            if p.grad is not view:
                view.copy_(p.grad)
                p.grad = view
        else:
            if r.staging is None:
                r.staging = self.g.empty(r.b - r.a, p.dtype, p.device, zero=False)
            if p.grad.is_cuda:  # packed by one multi-tensor copy when the bucket is complete
                r.loose.append((r.staging[a - r.a:b - r.a].view_as(p), p.grad))
            else:
                r.staging[a - r.a:b - r.a].copy_(p.grad.reshape(-1))
            p.grad = None  # the full-size gradient is not kept
        if not self._queued:
            self._queued = True
            Variable._execution_engine.queue_callback(self._finish_backward)
        r.ready += 1
        while self._next < len(self.buckets) and self.buckets[self._next].ready == len(self.buckets[self._next].params):
            nxt = self.buckets[self._next]
            if nxt.loose:
                from ..ops import pack_into

                pack_into(nxt.staging, nxt.loose)
                nxt.loose = []
            if self.stage == 1:
                nxt.work = self.g.all_reduce(self.grad[nxt.a:nxt.b], op="avg", async_op=True)
            else:
                sizes = self.flat.bucket_sizes(nxt.a, nxt.b)
                if self.fused_step and nxt.staging.is_cuda and sizes[self.g.rank]:
                    at = max(nxt.a, self.flat.lo) - self.flat.lo
                    nxt.work = self.g.reduce_scatter(nxt.staging, sizes, op="avg", async_op=True,
                                                     adam=self._adam_args(at, sizes[self.g.rank]))
                    nxt.fused_acc = True
                elif self.g.fused and nxt.staging.is_cuda and sizes[self.g.rank]:
                    at = max(nxt.a, self.flat.lo) - self.flat.lo
                    nxt.work = self.g.reduce_scatter(nxt.staging, sizes, op="avg", async_op=True,
                                                     accumulate_into=self.grad_shard[at:at + sizes[self.g.rank]])
                    nxt.fused_acc = True
                else:
                    nxt.work = self.g.reduce_scatter(nxt.staging, sizes, op="avg", async_op=True)
                    nxt.fused_acc = False
            self._next += 1

    def _finish_backward(self):
        self._queued = False
        incomplete = any(r.ready != len(r.params) for r in self.buckets)
        for r in self.buckets:
            if r.work is not None:
                mine = r.work.wait()
                if self.stage == 2 and mine.numel() and not r.fused_acc:
                    at = max(r.a, self.flat.lo) - self.flat.lo
                    self.grad_shard[at:at + mine.numel()].add_(mine)
            if self.stage == 2 and r.staging is not None:
                self.g.release(r.staging)
                r.staging = None
            r.ready, r.work = 0, None
        self._next = 0
        if incomplete:
            raise RuntimeError("tandem_b200 ZeRO: every parameter must receive a gradient")

    def _adam_args(self, at, count):
        """AdamArgs for elements [at, at+count) of this rank's shard, for the step the current backward feeds."""
        from .symm import AdamArgs

        lo = self.flat.lo
        shard = self.buf[lo:self.flat.hi]
        st = self.opt._state("flat", shard)
        master = self.opt.master.get("flat")
        step = st[0] + 1.0
        param = (master if master is not None else shard)[at:at + count]
        shadow = shard[at:at + count] if master is not None else None
        return AdamArgs.make(param, st[1][at:at + count], st[2][at:at + count], self.opt.scalars(step),
                             self.opt.weight_decay != 0, shadow)

    @torch.no_grad()
    def step(self):
        lo, hi = self.flat.lo, self.flat.hi
        if self.fused_step:
            self.opt._state("flat", self.buf[lo:hi])[0] += 1.0  # the update itself ran inside the reduce-scatter kernels
        else:
            grad = self.grad[lo:hi] if self.stage == 1 else self.grad_shard
            self.opt.update("flat", self.buf[lo:hi], grad)
        self.g.all_gather(self.buf, self.flat.sizes)

    def zero_grad(self):
        if self.stage == 1:
            for p in self.flat.params:
                p.grad = None
        else:
            self.grad_shard.zero_()


class _Unit:
    def __init__(self, index, module, params, group, device, dtype):
        self.index, self.module = index, module
        self.flat = FlatLayout(params, group.size, group.rank)
        self.full = torch.empty(self.flat.numel, device=device, dtype=dtype)
        self.nbytes = self.full.untyped_storage().nbytes()
        self.shard = None
        self.grad_shard = torch.zeros(self.flat.hi - self.flat.lo, device=device, dtype=dtype)
        self.gathered = True
        self.pending = None  # all-gather in flight
        self.ready = 0
        self.rs = None  # reduce-scatter in flight
        self.staging = None
        self.fused_acc = False
        self.loose = []
        self.fused = None  # plan for gathering the unit's qkv weight inside its GEMM (FSDP(fuse_gather_gemm=True))
        self.pending_head = None


class FSDP(torch.nn.Module):
    """ZeRO stage 3 over model.units() (for the GPT: embedding, each block, head)."""

    def __init__(self, model, group, optimizer=None, prefetch=True, fuse_gather_gemm=False):
        """fuse_gather_gemm (GPU kernels, bf16 model): in the forward pass a transformer block's qkv weight and
        bias are not gathered ahead of time; the qkv GEMM kernel pulls them from the owners' shards itself while
        it computes (ops.gemm.GatheredLinear), and the rest of the unit arrives on the communication stream
        meanwhile.  Backward gathers whole units as usual."""
        super().__init__()
        self.module, self.g = model, group
        self.fuse = bool(fuse_gather_gemm) and group.fused
        self.opt = optimizer or ShardedAdamW()
        self.prefetch = prefetch
        # The embedding's input needs no gradient, so torch warns that its full
        # backward hook fires on the outputs -- which is when we want it.
        warnings.filterwarnings("ignore", message="Full backward hook is firing when gradients are computed with respect to module outputs")
        self.live = 0  # units whose full parameters exist right now
        self.max_live = 0
        self.units, self.unit_of = [], {}
        taken = set()
        for i, m in enumerate(model.units()):
            ps = [p for p in m.parameters() if p.requires_grad and id(p) not in taken]
            taken.update(id(p) for p in ps)
            if not ps:
                raise ValueError(f"unit {i} has no parameters of its own")
            u = _Unit(i, m, ps, group, ps[0].device, ps[0].dtype)
            with torch.no_grad():
                _flatten_into(u.full, u.flat)
                group.broadcast(u.full, root=0)
                _point_into(u.full, u.flat)
                # every rank allocates the largest shard's size, so heap offsets stay identical across ranks
                u.shard = group.empty(max(u.flat.sizes), u.full.dtype, u.full.device)[:u.flat.hi - u.flat.lo]
                u.shard.copy_(u.full[u.flat.lo:u.flat.hi])
            if self.fuse:
                self._plan_fusion(u, m)
            for p in ps:
                self.unit_of[p] = u
                p.register_post_accumulate_grad_hook(self._on_grad)
            m.register_forward_pre_hook(self._before_forward(u))
            m.register_forward_hook(self._after_forward(u))
            m.register_full_backward_pre_hook(self._before_backward(u))
            self.live += 1
            self._free(u)
            self.units.append(u)
        if len(taken) != sum(1 for p in model.parameters() if p.requires_grad):
            raise ValueError("every parameter must belong to one of model.units()")
        self._queued = False
        self.max_live = 0
        if group.fused and self.units[0].shard.is_cuda:
            group._sym.device_barrier()  # every rank's shards are in place before anyone pulls them

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def _plan_fusion(self, u, m):
        """Marks a unit whose first GEMM can gather its own weight: a block whose qkv weight is bf16, starts
        16-byte aligned in the unit's flat buffer and is followed directly by its bias."""
        qkv = getattr(getattr(m, "attn", None), "qkv", None)
        if qkv is None or qkv.weight.dtype != torch.bfloat16 or not qkv.weight.is_cuda or qkv.bias is None:
            return
        w_off = u.flat.offset[qkv.weight]
        N, K = qkv.weight.shape
        if w_off % 8 or K % 8 or u.flat.offset[qkv.bias] != w_off + N * K:
            return
        u.fused = {"weight": qkv.weight, "w_off": w_off, "end": w_off + N * K + N, "N": N, "K": K, "op": None}

    # ---- a unit's full parameters: gather, wait, free
    def _start_gather(self, u, forward=False):
        if u.gathered or u.pending is not None:
            return
        u.full.untyped_storage().resize_(u.nbytes)
        self.live += 1
        self.max_live = max(self.max_live, self.live)
        if self.fuse and forward and u.fused is not None and torch.is_grad_enabled():
            from ..ops.gemm import GATHERED, GatheredLinear
            from .symm import split_offsets

            f = u.fused
            if f["op"] is None:
                offs = split_offsets(u.flat.numel, self.g.size, u.flat.sizes)
                f["op"] = GatheredLinear(self.g._sym._peers_of(u.shard), offs, self.g.rank, u.full, f["w_off"], f["N"], f["K"],
                                         bias_follows=True)
            sym = self.g._sym
            u.pending_head = sym.gather_shards(u.full, u.shard, u.flat.sizes, lo=0, hi=f["w_off"])
            u.pending = sym.gather_shards(u.full, u.shard, u.flat.sizes, lo=f["end"], hi=u.flat.numel)
            GATHERED[f["weight"].data_ptr()] = (f["op"], u.pending._event)
        elif self.g.fused and u.full.is_cuda:
            # Shards only change inside step(), which is fenced by barriers on both
            # sides, so peers' shards can be pulled with no handshake at all.
            u.pending = self.g._sym.gather_shards(u.full, u.shard, u.flat.sizes)
        else:
            u.full[u.flat.lo:u.flat.hi].copy_(u.shard)
            u.pending = self.g.all_gather(u.full, u.flat.sizes, async_op=True)

    def _gather(self, u, forward=False):
        self._start_gather(u, forward)
        if u.pending_head is not None:
            # fused unit: only what precedes the qkv weight (the first LayerNorm) is awaited here; the qkv GEMM
            # brings its own weight and makes the stream wait for the rest afterwards
            u.pending_head.wait()
            u.pending_head = None
            u.gathered = True
            return
        if u.pending is not None:
            u.pending.wait()
            u.pending = None
            u.gathered = True

    def _free(self, u):
        if u.pending is not None:
            u.pending.wait()
            u.pending = None
        if u.full.untyped_storage().nbytes():
            self.live -= 1
        u.full.untyped_storage().resize_(0)
        u.gathered = False

    # ---- hooks
    def _before_forward(self, u):
        def hook(mod, args):
            self._gather(u, forward=True)
            if self.prefetch and u.index + 1 < len(self.units):
                self._start_gather(self.units[u.index + 1], forward=True)

        return hook

    def _after_forward(self, u):
        def hook(mod, args, out):
            if torch.is_grad_enabled() and u.index == len(self.units) - 1:
                return  # the last unit's backward comes first: keep it
            self._free(u)

        return hook

    def _before_backward(self, u):
        def hook(mod, grad_out):
            if not self._queued:
                self._queued = True
                Variable._execution_engine.queue_callback(self._finish_backward)
            self._gather(u)
            if self.prefetch and u.index > 0:
                self._start_gather(self.units[u.index - 1])

        return hook

    def _on_grad(self, p):
        u = self.unit_of[p]
        if u.staging is None:
            u.staging = self.g.empty(u.flat.numel, p.dtype, p.device, zero=False)
        a, b = u.flat.span(p)
        if p.grad.is_cuda:
            u.loose.append((u.staging[a:b].view_as(p), p.grad))
        else:
            u.staging[a:b].copy_(p.grad.reshape(-1))
        p.grad = None
        u.ready += 1
        if u.ready == len(u.flat.params):
            if u.loose:
                from ..ops import pack_into

                pack_into(u.staging, u.loose)
                u.loose = []
            # Backward through the unit is over: drop its parameters, ship its gradients.
            self._free(u)
            if self.g.fused and u.staging.is_cuda:  # the shard accumulation rides in the kernel's epilogue
                u.rs = self.g.reduce_scatter(u.staging, u.flat.sizes, op="avg", async_op=True, accumulate_into=u.grad_shard)
                u.fused_acc = True
            else:
                u.rs = self.g.reduce_scatter(u.staging, u.flat.sizes, op="avg", async_op=True)
                u.fused_acc = False

    def _finish_backward(self):
        self._queued = False
        incomplete = False
        for u in self.units:
            if u.ready != len(u.flat.params):
                incomplete = True
            if u.rs is not None:
                mine = u.rs.wait()
                if mine.numel() and not u.fused_acc:
                    u.grad_shard.add_(mine)
            if u.staging is not None:
                self.g.release(u.staging)
            u.rs, u.staging, u.ready = None, None, 0
            if u.gathered:
                self._free(u)
        if incomplete:
            raise RuntimeError("tandem_b200 FSDP: every parameter must receive a gradient")

    @torch.no_grad()
    def step(self):
        fence = self.g.fused and self.units[0].shard.is_cuda
        if fence:
            self.g._sym.device_barrier()  # every rank has finished pulling the old shards
        for u in self.units:
            self.opt.update(u.index, u.shard, u.grad_shard)
        if fence:
            self.g._sym.device_barrier(after_current=True)  # the new shards are complete before anyone pulls them

    def zero_grad(self):
        for u in self.units:
            u.grad_shard.zero_()

    @torch.no_grad()
    def full_parameters(self):
        """All parameters gathered into one flat tensor, in units() order (for checkpoints and tests)."""
        out = []
        for u in self.units:
            full = torch.empty(u.flat.numel, device=u.shard.device, dtype=u.shard.dtype)
            full[u.flat.lo:u.flat.hi].copy_(u.shard)
            self.g.all_gather(full, u.flat.sizes)
            out.append(full)
        return torch.cat(out)
