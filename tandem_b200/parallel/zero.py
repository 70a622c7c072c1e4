"""ZeRO stages 1-3: data parallelism that shards optimizer state, then gradients,
then parameters (Rajbhandari et al., 2020).

The user-visible contract and the flat layouts are those of the reference's
tandem/zero.py:29-336, because checkpoints and the bit-equality tests depend on them:
  ZeRO(stage=1|2)  every parameter is a view of one flat buffer (`buf`) in
                   module.parameters() order; rank r owns chunk r of
                   torch.tensor_split(numel, world).  Stage 1 averages slices of a full
                   flat gradient; stage 2 reduce-scatters each slice with per-rank sizes
                   = the overlap of the slice with each shard (often zero) and keeps
                   only `grad_shard`.  step() = sharded AdamW + all-gather of `buf`.
  FSDP             the same per unit of model.units(): a unit's full parameters exist
                   only around its forward and its backward, the neighbouring unit is
                   gathered one step ahead, and a unit's gradients are reduce-scattered
                   as soon as they are complete.  At most three units are whole at once.
Train with: loss = z(x, y); loss.backward(); z.step(); z.zero_grad().

How the data plane is organised here (and why it differs from growing and freeing
storages as the reference does, tandem/zero.py:238-261):

  Fixed memory.  Everything that a collective touches is taken from the group's
  symmetric heap ONCE, at construction: the flat parameter buffer, the full gradient
  (stage 1), a ring of gradient staging slots (stages 2 and 3), each unit's shard, and
  -- stage 3 -- a ring of three unit-sized parameter slots.  Unit i always
  materialises in slot i mod 3 (its neighbours in either direction use the other two),
  so parameter addresses never change: tensors that autograd saved in forward see the
  unit's re-gathered values in backward, nothing is allocated or resized per step, and
  a whole step can be recorded as a CUDA graph (parallel/graph.py).

  Slots carry their own ordering.  A ring slot remembers the collective that last used
  it; taking the slot again first makes the current stream wait for that work (a stream
  dependency on GPUs, a blocking wait on CPU ranks).  That is all the synchronisation
  the schedulers below need besides the order in which hooks fire.

  Gradients.  The gradients autograd hands over are parked until their slice (or unit)
  is complete and then packed into a staging slot by ONE multi-tensor kernel; the
  reduce-scatter reads the peers' staging slots in place, divides operands as it loads
  them and ends in an epilogue instead of a separate pass: accumulate into the gradient
  shard, or (ZeRO(fused_step=True)) the AdamW update itself on the chunk just reduced.

  Parameters (stage 3).  A unit's shards only change inside step(), which is fenced by
  device barriers; gathers therefore need no handshake: each rank pulls the peers'
  shards with one kernel that opens with a system-scope fence, on the communication
  stream, one unit ahead of compute.  With FSDP(fuse_gather_gemm=True) a block's qkv
  weight and bias are not gathered ahead in the forward pass: the rest of the unit is
  pulled around them and the qkv GEMM kernel fetches its own weight from the owners'
  shards while it multiplies (ops.gemm.GatheredLinear).

  Mixed precision.  With 16-bit parameters the optimizer keeps an fp32 master copy of
  each shard next to the moments (ShardedAdamW.master); gradients stay 16-bit on the wire.

On CPU ranks the same classes issue the reference's sequence of collectives and torch
operations, which is what makes them bit-identical to torch DDP + AdamW.
"""

import collections
import warnings

import torch
from torch.autograd import Variable

from .optim import ShardedAdamW


def split_sizes(numel, world):
    """Chunk lengths of torch.tensor_split(numel, world)."""
    base, extra = divmod(numel, world)
    return [base + (1 if r < extra else 0) for r in range(world)]


class FlatLayout:
    """Where each parameter sits inside one flat buffer, and which part each rank owns."""

    def __init__(self, params, world, rank):
        self.params = list(params)
        self.offset = {}
        at = 0
        for p in self.params:
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
        out, start = [], 0
        for size in self.sizes:
            out.append(max(0, min(b, start + size) - max(a, start)))
            start += size
        return out

    @torch.no_grad()
    def gather_into(self, flat):
        """flat <- the parameters' current values, then the parameters become views of flat."""
        for p in self.params:
            a, b = self.span(p)
            flat[a:b].copy_(p.detach().reshape(-1))
        self.alias(flat)

    def alias(self, flat):
        for p in self.params:
            a, b = self.span(p)
            p.data = flat[a:b].view_as(p)


class SlotRing:
    """`count` equally sized flat buffers from the symmetric heap, handed out by index.  Each slot remembers
    the asynchronous work that last used it and what to do with that work's result; `take(i)` first finishes
    that work (a stream dependency on GPUs, a blocking wait on CPU ranks) and hands its result to the
    follow-up, so nobody overwrites data a collective is still reading or a result not yet consumed."""

    def __init__(self, group, count, numel, dtype, device):
        self.slots = [group.empty(numel, dtype, device, zero=False) for _ in range(count)]
        self.busy = [None] * count

    def __len__(self):
        return len(self.slots)

    def _finish(self, i):
        if self.busy[i] is not None:
            work, then = self.busy[i]
            self.busy[i] = None
            result = work.wait()
            if then is not None:
                then(result)

    def take(self, i):
        i %= len(self.slots)
        self._finish(i)
        return self.slots[i]

    def occupy(self, i, work, then=None):
        self.busy[i % len(self.slots)] = (work, then)

    def settle(self):
        for i in range(len(self.slots)):
            self._finish(i)


class _Slice:
    """A contiguous run [a, b) of the flat buffer whose gradients are reduced together (stages 1 and 2)."""

    __slots__ = ("index", "a", "b", "params", "missing", "parked", "flight", "in_kernel")

    def __init__(self, index, a, b, params):
        self.index, self.a, self.b, self.params = index, a, b, params
        self.rearm()

    def rearm(self):
        self.missing = len(self.params)
        self.parked = []      # (offset inside the slice, parameter, gradient) waiting for the slice's one pack
        self.flight = None
        self.in_kernel = False  # the reduce-scatter's epilogue already consumed the reduced chunk


def _park_or_copy(dest, parked):
    """Writes parked gradients into `dest` (a flat staging buffer): one multi-tensor kernel on a GPU."""
    if not parked:
        return
    if dest.is_cuda:
        from ..ops import pack_into

        pack_into(dest, [(dest[at:at + g.numel()].view_as(g), g) for at, g in parked])
    else:
        for at, g in parked:
            dest[at:at + g.numel()].copy_(g.reshape(-1))


class ZeRO(torch.nn.Module):
    """Stages 1 and 2."""

    def __init__(self, module, group, stage=1, optimizer=None, bucket_bytes=25 << 20, fused_step=False, capturable=False):
        """fused_step (stage 2, GPU kernels only): apply the sharded AdamW update inside each slice's
        reduce-scatter kernel, on the freshly reduced gradient chunk, instead of in step().  One pass over
        the gradients instead of three (reduce, accumulate, optimizer); step() then only all-gathers the
        parameters.  Not compatible with accumulating gradients over several backward passes.
        capturable (GPU kernels only): the optimizer's step-dependent constants are computed on the device, so
        that forward + backward + step() can be recorded once as a CUDA graph and replayed."""
        super().__init__()
        if stage not in (1, 2):
            raise ValueError("ZeRO covers stages 1 and 2 (FSDP is stage 3)")
        self.module, self.g, self.stage = module, group, stage
        self.opt = optimizer or ShardedAdamW()
        params = [p for p in module.parameters() if p.requires_grad]
        dev, dtype = params[0].device, params[0].dtype
        if any(p.dtype != dtype or p.device != dev for p in params):
            raise ValueError("ZeRO needs all parameters on one device with one dtype")
        self.flat = FlatLayout(params, group.size, group.rank)
        self.buf = group.empty(self.flat.numel, dtype, dev)
        self.flat.gather_into(self.buf)
        group.broadcast(self.buf, root=0)
        on_kernels = bool(group.fused and dev.type == "cuda")
        self.fused_step = bool(fused_step) and stage == 2 and on_kernels
        self.capturable = bool(capturable) and on_kernels
        if self.capturable:
            self.opt.use_device_scalars(dev)
        # Slices run from the end of the buffer, the order in which backward produces gradients.
        self.slices, self._home = [], {}
        run, size = [], 0
        for p in reversed(params):
            nbytes = p.numel() * p.element_size()
            if run and size + nbytes > bucket_bytes:
                self._cut(run)
                run, size = [], 0
            run.append(p)
            size += nbytes
        if run:
            self._cut(run)
        if stage == 1:
            self.grad = group.empty(self.flat.numel, dtype, dev)
        else:
            self.grad_shard = torch.zeros(self.flat.hi - self.flat.lo, device=dev, dtype=dtype)
            widest = max(s.b - s.a for s in self.slices)
            self._staging = SlotRing(group, min(2, len(self.slices)), widest, dtype, dev)
        self._queue = collections.deque(self.slices)
        self._drain_armed = False
        for p in params:
            p.register_post_accumulate_grad_hook(self._arrived)

    def _cut(self, params):
        a = min(self.flat.offset[p] for p in params)
        b = max(self.flat.offset[p] + p.numel() for p in params)
        piece = _Slice(len(self.slices), a, b, params)
        for p in params:
            self._home[p] = piece
        self.slices.append(piece)

    @property
    def buckets(self):
        return self.slices

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    # ------------------------------------------------------------------ backward
    def _arrived(self, p):
        piece = self._home[p]
        a, b = self.flat.span(p)
        if self.stage == 1:
            home = self.grad[a:b].view_as(p)
            if p.grad.data_ptr() != home.data_ptr():
                home.copy_(p.grad)
                p.grad = home
        else:
            piece.parked.append((a - piece.a, p.grad))
            p.grad = None  # stage 2 keeps no full-size gradient
        if not self._drain_armed:
            self._drain_armed = True
            Variable._execution_engine.queue_callback(self._drain)
        piece.missing -= 1
        while self._queue and self._queue[0].missing == 0:  # in slice order on every rank
            self._send(self._queue.popleft())

    def _send(self, piece):
        if self.stage == 1:
            piece.flight = self.g.all_reduce(self.grad[piece.a:piece.b], op="avg", async_op=True)
            return
        staging = self._staging.take(piece.index)[:piece.b - piece.a]
        _park_or_copy(staging, piece.parked)
        piece.parked = []
        sizes = self.flat.bucket_sizes(piece.a, piece.b)
        mine = sizes[self.g.rank]
        extra = {}
        if mine and self.g.fused and staging.is_cuda:
            at = max(piece.a, self.flat.lo) - self.flat.lo
            if self.fused_step:
                extra["adam"] = self._adam_args(at, mine)
            else:
                extra["accumulate_into"] = self.grad_shard[at:at + mine]
            piece.in_kernel = True
        piece.flight = self.g.reduce_scatter(staging, sizes, op="avg", async_op=True, **extra)
        follow_up = None
        if mine and not piece.in_kernel:  # the reduced chunk sits in the slot: fold it into the shard before the slot moves on
            at = max(piece.a, self.flat.lo) - self.flat.lo
            follow_up = lambda reduced, at=at: self.grad_shard[at:at + reduced.numel()].add_(reduced)
        self._staging.occupy(piece.index, piece.flight, follow_up)

    def _drain(self):
        self._drain_armed = False
        starved = bool(self._queue)
        if self.stage == 2:
            self._staging.settle()
        for piece in self.slices:
            if self.stage == 1 and piece.flight is not None:
                piece.flight.wait()
            piece.rearm()
        self._queue = collections.deque(self.slices)
        if starved:
            raise RuntimeError("tandem_b200 ZeRO: every parameter must receive a gradient")

    def _adam_args(self, at, count):
        """Arguments of the fused update for elements [at, at+count) of this rank's shard, for the step that the
        current backward feeds."""
        from .symm import AdamArgs

        shard = self.buf[self.flat.lo:self.flat.hi]
        _, exp_avg, exp_avg_sq = self.opt.ensure_state("flat", shard)
        master = self.opt.master.get("flat")
        param = (master if master is not None else shard)[at:at + count]
        shadow = shard[at:at + count] if master is not None else None
        moments = exp_avg[at:at + count], exp_avg_sq[at:at + count]
        if self.capturable:
            return AdamArgs.on_device(param, *moments, self.opt.device_scalars(), shadow)
        return AdamArgs.make(param, *moments, self.opt.scalars(self.opt.state["flat"][0] + 1.0), self.opt.weight_decay != 0, shadow)

    # ------------------------------------------------------------------ optimizer
    @torch.no_grad()
    def step(self):
        lo, hi = self.flat.lo, self.flat.hi
        if self.fused_step:
            self.opt.ensure_state("flat", self.buf[lo:hi])[0] += 1.0  # the update itself ran inside the reduce-scatter kernels
        else:
            grad = self.grad[lo:hi] if self.stage == 1 else self.grad_shard
            self.opt.update("flat", self.buf[lo:hi], grad)
        if self.capturable:
            self.opt.advance_on_device()  # the next step's constants
        self.g.all_gather(self.buf, self.flat.sizes)

    def zero_grad(self):
        if self.stage == 1:
            for p in self.flat.params:
                p.grad = None
        else:
            self.grad_shard.zero_()


class _Unit:
    """One element of model.units() under stage 3: its layout, this rank's shard of it, and where it is in its
    cycle of sharded -> gathering -> whole -> sharded."""

    def __init__(self, index, module, layout, home):
        self.index, self.module, self.flat = index, module, layout
        self.full = home[:layout.numel]  # the unit's place in its parameter slot: valid only while `whole`
        self.shard = None
        self.grad_shard = None
        self.whole = False
        self.gather = None       # all-gather in flight
        self.head_gather = None  # fused units: the part that precedes the self-gathering weight
        self.reduce = None       # reduce-scatter in flight
        self.in_kernel = False
        self.missing = len(layout.params)
        self.parked = []
        self.fused = None        # plan for gathering the unit's qkv weight inside its GEMM


class FSDP(torch.nn.Module):
    """ZeRO stage 3 over model.units() (for the GPT: embedding, each block, head)."""

    PARAMETER_SLOTS = 3  # the running unit, the prefetched one, and the head kept from forward to backward

    def __init__(self, model, group, optimizer=None, prefetch=True, fuse_gather_gemm=False, capturable=False):
        """fuse_gather_gemm (GPU kernels, bf16 model): in the forward pass a transformer block's qkv weight and
        bias are not gathered ahead of time; the qkv GEMM kernel pulls them from the owners' shards itself while
        it computes (ops.gemm.GatheredLinear), and the rest of the unit arrives on the communication stream
        meanwhile.  Backward gathers whole units as usual.
        capturable (GPU kernels only): optimizer constants live on the device so that a step can be recorded
        as a CUDA graph."""
        super().__init__()
        self.module, self.g = model, group
        self.opt = optimizer or ShardedAdamW()
        self.prefetch = prefetch
        # The embedding's input needs no gradient, so torch warns that its full
        # backward hook fires on the outputs -- which is exactly when the unit must be whole.
        warnings.filterwarnings("ignore", message="Full backward hook is firing when gradients are computed with respect to module outputs")
        members, claimed = [], set()
        for i, m in enumerate(model.units()):
            own = [p for p in m.parameters() if p.requires_grad and id(p) not in claimed]
            claimed.update(id(p) for p in own)
            if not own:
                raise ValueError(f"unit {i} has no parameters of its own")
            members.append((m, own))
        if len(claimed) != sum(1 for p in model.parameters() if p.requires_grad):
            raise ValueError("every parameter must belong to one of model.units()")
        first = members[0][1][0]
        dev, dtype = first.device, first.dtype
        layouts = [FlatLayout(own, group.size, group.rank) for _, own in members]
        widest = max(l.numel for l in layouts)
        on_kernels = bool(group.fused and dev.type == "cuda")
        self.fuse = bool(fuse_gather_gemm) and on_kernels
        self.capturable = bool(capturable) and on_kernels
        if self.capturable:
            self.opt.use_device_scalars(dev)
        self._homes = SlotRing(group, min(self.PARAMETER_SLOTS, len(members)), widest, dtype, dev)
        self._staging = SlotRing(group, min(2, len(members)), widest, dtype, dev)
        self.live = 0      # units whose full parameters exist right now
        self.max_live = 0
        self.units, self._unit_of = [], {}
        for i, ((m, own), layout) in enumerate(zip(members, layouts)):
            u = _Unit(i, m, layout, self._homes.slots[i % len(self._homes)])
            with torch.no_grad():
                layout.gather_into(u.full)  # parameters become views of the unit's slot, for good
                group.broadcast(u.full, root=0)
                # every rank allocates the largest shard's size, so heap offsets stay identical across ranks
                u.shard = group.empty(max(layout.sizes), dtype, dev)[:layout.hi - layout.lo]
                u.shard.copy_(u.full[layout.lo:layout.hi])
            u.grad_shard = torch.zeros(layout.hi - layout.lo, device=dev, dtype=dtype)
            if self.fuse:
                self._plan_fusion(u)
            for p in own:
                self._unit_of[p] = u
                p.register_post_accumulate_grad_hook(self._arrived)
            m.register_forward_pre_hook(self._before_forward(u))
            m.register_forward_hook(self._after_forward(u))
            m.register_full_backward_pre_hook(self._before_backward(u))
            self.units.append(u)
        self._drain_armed = False
        if on_kernels:
            group._sym.device_barrier()  # every rank's shards are in place before anyone pulls them

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def _plan_fusion(self, u):
        """Marks a unit whose first GEMM can gather its own weight: a block whose qkv weight is bf16, starts
        16-byte aligned in the unit's flat buffer and is followed directly by its bias."""
        qkv = getattr(getattr(u.module, "attn", None), "qkv", None)
        if qkv is None or qkv.weight.dtype != torch.bfloat16 or not qkv.weight.is_cuda or qkv.bias is None:
            return
        start = u.flat.offset[qkv.weight]
        rows, cols = qkv.weight.shape
        if start % 8 or cols % 8 or u.flat.offset[qkv.bias] != start + rows * cols:
            return
        u.fused = {"weight": qkv.weight, "w_off": start, "end": start + rows * cols + rows, "N": rows, "K": cols, "op": None}

    # ------------------------------------------------------------------ a unit's cycle
    def _begin_gather(self, u, forward=False):
        if u.whole or u.gather is not None:
            return
        self._homes.take(u.index)  # orders this stream after whatever last used the slot
        self.live += 1
        self.max_live = max(self.max_live, self.live)
        sym = self.g._sym if self.g.fused and u.full.is_cuda else None
        if sym is not None and self.fuse and forward and u.fused is not None and torch.is_grad_enabled():
            from ..ops.gemm import GATHERED, GatheredLinear
            from .symm import split_offsets

            plan = u.fused
            if plan["op"] is None:
                offs = split_offsets(u.flat.numel, self.g.size, u.flat.sizes)
                plan["op"] = GatheredLinear(sym._peers_of(u.shard), offs, self.g.rank, u.full, plan["w_off"], plan["N"], plan["K"],
                                            bias_follows=True)
            u.head_gather = sym.gather_shards(u.full, u.shard, u.flat.sizes, lo=0, hi=plan["w_off"])
            u.gather = sym.gather_shards(u.full, u.shard, u.flat.sizes, lo=plan["end"], hi=u.flat.numel)
            GATHERED[plan["weight"].data_ptr()] = (plan["op"], u.gather._event)
        elif sym is not None:
            # Shards only change inside step(), which is fenced by barriers on both sides, so the
            # peers' shards can be pulled with no handshake at all.
            u.gather = sym.gather_shards(u.full, u.shard, u.flat.sizes)
        else:
            u.full[u.flat.lo:u.flat.hi].copy_(u.shard)
            u.gather = self.g.all_gather(u.full, u.flat.sizes, async_op=True)

    def _make_whole(self, u, forward=False):
        self._begin_gather(u, forward)
        if u.head_gather is not None:
            # fused unit: only what precedes the qkv weight (the first LayerNorm) is awaited here; the qkv GEMM
            # brings its own weight and makes the stream wait for the rest afterwards
            u.head_gather.wait()
            u.head_gather = None
            u.whole = True
            return
        if u.gather is not None:
            u.gather.wait()
            u.gather = None
        u.whole = True

    def _let_go(self, u):
        """The unit's full parameters are no longer needed: its slot may be taken by another unit."""
        if u.gather is not None:
            u.gather.wait()
            u.gather = None
        if u.whole or u.head_gather is not None:
            self.live -= 1
        u.whole, u.head_gather = False, None

    # ------------------------------------------------------------------ hooks
    def _neighbour(self, u, step):
        j = u.index + step
        return self.units[j] if self.prefetch and 0 <= j < len(self.units) else None

    def _before_forward(self, u):
        def hook(mod, args):
            self._make_whole(u, forward=True)
            ahead = self._neighbour(u, +1)
            if ahead is not None:
                self._begin_gather(ahead, forward=True)

        return hook

    def _after_forward(self, u):
        def hook(mod, args, out):
            keeps = torch.is_grad_enabled() and u.index == len(self.units) - 1  # backward starts with the last unit
            if not keeps:
                self._let_go(u)

        return hook

    def _before_backward(self, u):
        def hook(mod, grad_out):
            if not self._drain_armed:
                self._drain_armed = True
                Variable._execution_engine.queue_callback(self._drain)
            self._make_whole(u)
            ahead = self._neighbour(u, -1)
            if ahead is not None:
                self._begin_gather(ahead)

        return hook

    def _arrived(self, p):
        u = self._unit_of[p]
        u.parked.append((u.flat.offset[p], p.grad))
        p.grad = None
        u.missing -= 1
        if u.missing:
            return
        # Backward through the unit is over: its parameters can go, its gradients ship.
        self._let_go(u)
        staging = self._staging.take(u.index)[:u.flat.numel]
        _park_or_copy(staging, u.parked)
        u.parked = []
        u.in_kernel = bool(self.g.fused and staging.is_cuda)
        extra = {"accumulate_into": u.grad_shard} if u.in_kernel else {}  # the shard accumulation rides in the kernel's epilogue
        u.reduce = self.g.reduce_scatter(staging, u.flat.sizes, op="avg", async_op=True, **extra)
        follow_up = None if u.in_kernel else (lambda reduced, shard=u.grad_shard: shard.add_(reduced) if reduced.numel() else None)
        self._staging.occupy(u.index, u.reduce, follow_up)

    def _drain(self):
        self._drain_armed = False
        starved = False
        self._staging.settle()
        for u in self.units:
            starved |= u.missing != 0
            u.reduce, u.missing, u.parked = None, len(u.flat.params), []
            if u.whole or u.gather is not None:
                self._let_go(u)
        if starved:
            raise RuntimeError("tandem_b200 FSDP: every parameter must receive a gradient")

    # ------------------------------------------------------------------ optimizer
    @torch.no_grad()
    def step(self):
        fenced = self.g.fused and self.units[0].shard.is_cuda
        if fenced:
            self.g._sym.device_barrier()  # every rank has finished pulling the old shards
        for u in self.units:
            self.opt.update(u.index, u.shard, u.grad_shard)
        if self.capturable:
            self.opt.advance_on_device()
        if fenced:
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
