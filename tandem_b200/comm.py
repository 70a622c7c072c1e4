"""Collectives between the ranks of one machine: `Group`, `Work`, `launch`.

Public surface and semantics follow the reference's tandem/comm.py:55-547
(`CommError`, `Work`, `Group` with all_reduce / reduce_scatter / all_gather /
broadcast / send / recv / sendrecv / barrier / submit / close, and `launch`).
The machinery underneath is different:

  CPU ranks   the native host runtime (tandem_b200/csrc): one progress thread
              per rank, every rank's staging window mapped by every other rank,
              two-shot all-reduce by direct reads of the peers' windows.
  GPU ranks   one kernel per collective on a high-priority stream.  Buffers live
              in symmetric memory (each rank's allocation mapped into every
              peer through CUDA IPC); kernels load from and store to the peers'
              copies over NVLink and synchronise through flag words, with the
              gradient-averaging divide fused into the loads.  `Work.wait()`
              makes the caller's stream wait on an event; the host never blocks.
              transport="host" stages through pinned memory and the CPU runtime
              instead (for machines without peer access).

Point-to-point transfers between GPU ranks use NCCL send/recv through
torch.distributed, started lazily.
"""

import os
import threading
import time
import uuid

import torch
import torch.multiprocessing as mp

DEFAULT_SLOT_BYTES = 4 << 20
DEFAULT_SLOTS = 2
DEFAULT_TIMEOUT = float(os.environ.get("TANDEM_TIMEOUT", "600"))
DEFAULT_TRANSPORT = os.environ.get("TANDEM_TRANSPORT", "device")
DEFAULT_PRIORITY = int(os.environ.get("TANDEM_PRIORITY", "-1"))  # lower is more urgent
DEFAULT_BACKEND = os.environ.get("TANDEM_BACKEND", "native")
_BACKENDS = ("native", "cpp", "python")  # the reference's two names select the same native engine

DTYPE_CODE = {torch.float32: 0, torch.float64: 1, torch.bfloat16: 2, torch.float16: 3, torch.int64: 4,
              torch.int32: 5, torch.int16: 6, torch.int8: 7, torch.uint8: 8, torch.bool: 8}


class CommError(RuntimeError):
    pass


class Work:
    """A collective in flight.  `wait()` returns `result` (the tensor, or the
    reduced chunk for reduce_scatter); while `group.tracing` is on it also
    records how long the caller was blocked (tandem/comm.py:59-81)."""

    def __init__(self, name, group=None, handle=None, result=None, nbytes=0, keep=()):
        self.name = name
        self._group = group
        self._handle = handle
        self.result = result
        self._nbytes = nbytes
        self._keep = keep  # tensors the engine is reading or writing
        self._recorded = False
        self._error = None  # an exception raised by a Python job on the progress thread

    def wait(self):
        g, h = self._group, self._handle
        if h is None:
            return self.result
        t0 = time.perf_counter() if g is not None and g.tracing and not h.done() else None
        try:
            h.wait()
        except Exception as e:
            raise CommError(f"{self.name} failed: {e}") from e
        if t0 is not None:
            g.waits.append((self.name, t0, time.perf_counter()))
        if g is not None and g.tracing and not self._recorded:
            g.trace.append((self.name, h.started, h.finished, self._nbytes))
        self._recorded = True
        self._keep = ()
        if self._error is not None:
            raise CommError(f"{self.name} failed: {self._error}") from self._error
        return self.result

    def is_completed(self):
        return self._handle is None or self._handle.done()


class _StreamWork(Work):
    """A collective queued on the communication stream of a GPU rank: waiting
    is a stream dependency, not a host block (tandem/csrc/collectives.cpp:56-66)."""

    def __init__(self, name, group, event, result, nbytes, start_event=None):
        super().__init__(name, group, None, result, nbytes)
        self._event, self._start = event, start_event

    def wait(self):
        g = self._group
        torch.cuda.current_stream(g.device).wait_event(self._event)
        if g.tracing and not self._recorded and self._start is not None:
            g._pending_spans.append((self.name, self._start, self._event, self._nbytes))
        self._recorded = True
        g.check()
        return self.result

    def is_completed(self):
        return self._event.query()


class Group:
    """One rank's handle on the group."""

    def __init__(self, rank, size, device="cpu", sync=None, queues=None, slot_bytes=DEFAULT_SLOT_BYTES,
                 slots=DEFAULT_SLOTS, timeout=DEFAULT_TIMEOUT, transport=None, priority=None,
                 backend=None, job=None):
        self.rank, self.size = int(rank), int(size)
        self.device = torch.device(device)
        self.slot_bytes, self.slots, self.timeout = int(slot_bytes), int(slots), float(timeout)
        self.transport = transport or DEFAULT_TRANSPORT
        self.priority = DEFAULT_PRIORITY if priority is None else priority
        self.backend = backend or DEFAULT_BACKEND
        if self.transport not in ("device", "host"):
            raise CommError(f"unknown transport {self.transport}")
        if self.backend not in _BACKENDS:
            raise CommError(f"unknown backend {self.backend}")
        if job is None:
            raise CommError("a group needs a job name shared by its ranks (launch() and Group.from_env() make one)")
        self.job = job
        self.trace = []  # (name, start, end, bytes) per collective, on time.perf_counter's clock
        self.waits = []  # (name, start, end): time a caller spent blocked on a collective
        self.tracing = False
        self._pending_spans = []
        self._closed = False
        self._sym = None
        self._nccl = None
        from .engine import lib

        try:
            self._engine = lib().Engine(job, self.rank, self.size, self.slots, self.slot_bytes, self.timeout)
            self._engine.connect()
        except Exception as e:
            raise CommError(f"could not join group {job}: {e}") from e
        if self.device.type == "cuda":
            if self.device.index is None:
                self.device = torch.device("cuda", torch.cuda.current_device())
            if self.transport == "device" and self._ranks_share_a_gpu():
                # Collective kernels of different ranks wait on one another; as separate processes on ONE GPU
                # nothing guarantees that they run at the same time.  Such groups (the reference's
                # launch(gpus=[0, 0])) stage through the host engine instead.
                self.transport = "host"
            if self.transport == "device":
                from .parallel.symm import SymmetricComm

                self._sym = SymmetricComm(self)
        self.barrier()

    def _ranks_share_a_gpu(self):
        if self.size == 1:
            return False
        ids = torch.zeros(self.size, dtype=torch.int64)
        import hashlib

        props = torch.cuda.get_device_properties(self.device)
        name = f"{getattr(props, 'uuid', '')}/{getattr(props, 'pci_bus_id', self.device.index)}/{self.device.index}"
        ids[self.rank] = int(hashlib.sha1(name.encode()).hexdigest()[:15], 16)
        self._engine.all_gather(ids.data_ptr(), ids.numel(), 4, [1] * self.size).wait()
        return len(set(ids.tolist())) < self.size

    # ------------------------------------------------------------------ construction helpers
    @staticmethod
    def make_sync(ctx, size, slots):
        """Kept for signature parity (tandem/comm.py:175): the native runtime
        creates its own shared-memory synchronisation, so there is nothing to
        inherit from the launcher."""
        return None

    @classmethod
    def from_env(cls, device=None, **kw):
        """A group for a process started by torchrun (RANK / WORLD_SIZE /
        LOCAL_RANK / MASTER_PORT).  The job name is agreed through
        torch.distributed when a process group exists, else derived from the
        rendezvous port and TANDEM_JOB."""
        rank = int(os.environ.get("RANK", "0"))
        size = int(os.environ.get("WORLD_SIZE", "1"))
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        if device == "cuda":
            local = int(os.environ.get("LOCAL_RANK", str(rank)))
            torch.cuda.set_device(local)
            device = torch.device("cuda", local)
        job = os.environ.get("TANDEM_JOB")
        if job is None:
            import torch.distributed as dist

            if dist.is_available() and dist.is_initialized():
                box = [uuid.uuid4().hex[:12] if rank == 0 else None]
                dist.broadcast_object_list(box, src=0)
                job = box[0]
            elif size == 1:
                job = uuid.uuid4().hex[:12]
            else:
                # the launcher process (torchrun's agent) is the same parent for every rank of one run
                job = f"env{os.environ.get('MASTER_PORT', '0')}-{os.getppid()}"
        return cls(rank, size, device, job=job, **kw)

    # ------------------------------------------------------------------ plumbing
    def _native(self, name, start, result, nbytes, async_op, keep=()):
        if self._closed:
            raise CommError("group is closed")
        try:
            handle = start()
        except (ValueError, RuntimeError, TypeError) as e:
            raise CommError(f"{name}: {e}") from e
        work = Work(name, self, handle, result, nbytes, keep)
        return work if async_op else work.wait()

    def submit(self, name, fn, ready=None, nbytes=0, async_op=False):
        """Runs fn on the progress thread, in order with the collectives, after
        `ready` (a CUDA event) completes (tandem/comm.py:235-242)."""
        if self._closed:
            raise CommError("group is closed")
        work = Work(name, self, None, None, nbytes)

        def job():
            try:
                if ready is not None:
                    ready.synchronize()
                work.result = fn()
            except BaseException as e:  # reported to whoever waits
                work._error = e

        work._handle = self._engine.submit(job)
        return work if async_op else work.wait()

    @staticmethod
    def _flat(t):
        if not t.is_contiguous():
            raise CommError("collectives need contiguous tensors")
        return t.reshape(-1)

    def _code(self, t):
        try:
            return DTYPE_CODE[t.dtype]
        except KeyError:
            raise CommError(f"unsupported dtype {t.dtype}") from None

    def _chunks(self, flat, sizes):
        if sizes is None:
            return list(torch.tensor_split(flat, self.size))
        if len(sizes) != self.size or sum(sizes) != flat.numel() or any(s < 0 for s in sizes):
            raise CommError(f"chunk sizes {list(sizes)} do not partition {flat.numel()} elements")
        return list(torch.split(flat, list(sizes)))

    def _on_host(self, t):
        return self.device.type == "cpu" or t.device.type == "cpu"

    def _staged(self, name, flat, run, result_of, nbytes, async_op):
        """GPU tensor through pinned host memory and the CPU runtime (transport="host"): three jobs queued on
        the progress thread, which runs them in order -- copy to the host, the CPU collective, copy back."""
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(self.device))
        host = torch.empty(flat.shape, dtype=flat.dtype, pin_memory=True)
        dev = self.device

        def stage_in():
            ready.synchronize()
            with torch.cuda.device(dev):
                host.copy_(flat)
                torch.cuda.current_stream(dev).synchronize()

        self.submit(name + ":stage", stage_in, None, 0, True)
        inner = run(host)  # queued behind stage_in

        def stage_out():
            inner.wait()  # it ran before this job on the same thread: returns at once, or raises its error
            with torch.cuda.device(dev):
                flat.copy_(host)
                torch.cuda.current_stream(dev).synchronize()
            return result_of()

        return self.submit(name, stage_out, None, nbytes, async_op)

    def empty(self, numel, dtype, device=None, zero=True):
        """A flat tensor for communication buffers.  On GPU ranks it comes from
        the symmetric heap (mapped by every peer), which makes collectives on it
        zero-copy; every rank must make the same sequence of empty()/release()
        calls.  Elsewhere it is an ordinary tensor."""
        device = torch.device(device) if device is not None else self.device
        if self._sym is not None and device.type == "cuda":
            return self._sym.alloc(numel, dtype, zero)
        return (torch.zeros if zero else torch.empty)(numel, dtype=dtype, device=device)

    def release(self, t):
        """Returns a tensor from empty() to the symmetric heap."""
        if self._sym is not None and t.is_cuda:
            self._sym.free(t)

    def check(self):
        """Raises CommError if a GPU collective gave up waiting for a peer."""
        if self._sym is not None:
            self._sym.check()

    def _drain_spans(self):
        """Turns finished (start, end) CUDA-event pairs into host-clock spans."""
        if self._sym is None or not self._pending_spans:
            return
        self._sym.resolve_spans(self._pending_spans, self.trace)
        self._pending_spans = []

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, t, op="sum", async_op=False):
        """In place: every rank ends with the sum (or mean) of all ranks' `t`."""
        if op not in ("sum", "avg"):
            raise CommError(f"unknown op {op}")
        flat = self._flat(t)
        nbytes = t.numel() * t.element_size()
        code = self._code(flat)
        if op == "avg" and not flat.is_floating_point():
            raise CommError("avg needs a floating-point tensor")
        if not self._on_host(flat):
            if self._sym is not None:
                return self._sym.all_reduce(flat, op == "avg", t, nbytes, async_op)
            return self._staged("all_reduce", flat,
                                lambda h: self._engine.all_reduce(h.data_ptr(), h.numel(), code, op == "avg"),
                                lambda: t, nbytes, async_op)
        return self._native("all_reduce", lambda: self._engine.all_reduce(flat.data_ptr(), flat.numel(), code, op == "avg"),
                            t, nbytes, async_op, (flat,))

    @property
    def fused(self):
        """True when collectives run as GPU kernels that accept fused epilogues
        (reduce_scatter's accumulate_into= / adam=) and sync-free shard gathers."""
        return self._sym is not None and os.environ.get("TANDEM_FUSED", "1") != "0"

    def reduce_scatter(self, t, sizes=None, op="sum", async_op=False, accumulate_into=None, adam=None):
        """Sums `t` across ranks; rank r's chunk (chunk r of torch.tensor_split,
        or of `sizes`) ends reduced in place and is returned as a view.  The
        other chunks' contents afterwards are unspecified.
        GPU kernels only (`group.fused`): accumulate_into, a tensor shaped like
        the chunk, also receives `+= chunk` inside the kernel; adam, a
        parallel.symm.AdamArgs, applies a fused AdamW step with the chunk as
        the gradient."""
        if op not in ("sum", "avg"):
            raise CommError(f"unknown op {op}")
        flat = self._flat(t)
        nbytes = t.numel() * t.element_size()
        code = self._code(flat)
        mine = self._chunks(flat, sizes)[self.rank]
        szs = [] if sizes is None else [int(s) for s in sizes]
        if op == "avg" and not flat.is_floating_point():
            raise CommError("avg needs a floating-point tensor")
        if not self._on_host(flat):
            if self._sym is not None:
                return self._sym.reduce_scatter(flat, sizes, op == "avg", mine, nbytes, async_op, accumulate_into, adam)
        if accumulate_into is not None or adam is not None:
            raise CommError("fused reduce_scatter epilogues need GPU ranks with transport='device'")
        if not self._on_host(flat):
            return self._staged("reduce_scatter", flat,
                                lambda h: self._engine.reduce_scatter(h.data_ptr(), h.numel(), code, szs, op == "avg"),
                                lambda: mine, nbytes, async_op)
        return self._native("reduce_scatter",
                            lambda: self._engine.reduce_scatter(flat.data_ptr(), flat.numel(), code, szs, op == "avg"),
                            mine, nbytes, async_op, (flat,))

    def all_gather(self, t, sizes=None, async_op=False):
        """Rank r's chunk of `t` is valid on entry; fills in everyone else's."""
        flat = self._flat(t)
        nbytes = t.numel() * t.element_size()
        code = self._code(flat)
        self._chunks(flat, sizes)
        szs = [] if sizes is None else [int(s) for s in sizes]
        if not self._on_host(flat):
            if self._sym is not None:
                return self._sym.all_gather(flat, sizes, t, nbytes, async_op)
            return self._staged("all_gather", flat, lambda h: self._engine.all_gather(h.data_ptr(), h.numel(), code, szs),
                                lambda: t, nbytes, async_op)
        return self._native("all_gather", lambda: self._engine.all_gather(flat.data_ptr(), flat.numel(), code, szs),
                            t, nbytes, async_op, (flat,))

    def broadcast(self, t, root=0, async_op=False):
        flat = self._flat(t)
        nbytes = t.numel() * t.element_size()
        code = self._code(flat)
        if not 0 <= root < self.size:
            raise CommError(f"broadcast root {root} is not a rank of this group")
        if not self._on_host(flat):
            if self._sym is not None:
                return self._sym.broadcast(flat, root, t, nbytes, async_op)
            return self._staged("broadcast", flat, lambda h: self._engine.broadcast(h.data_ptr(), h.numel(), code, root),
                                lambda: t, nbytes, async_op)
        return self._native("broadcast", lambda: self._engine.broadcast(flat.data_ptr(), flat.numel(), code, root),
                            t, nbytes, async_op, (flat,))

    # ------------------------------------------------------------------ point to point
    def _p2p(self):
        if self._nccl is None:
            from .parallel.p2p import NcclP2P

            self._nccl = NcclP2P(self)
        return self._nccl

    def send(self, t, dst, async_op=False):
        flat = self._flat(t)
        nbytes = t.numel() * t.element_size()
        if not self._on_host(flat):
            return self._p2p().send(flat, dst, t, nbytes, async_op)
        return self._native(f"send->{dst}", lambda: self._engine.send(flat.data_ptr(), nbytes, dst), t, nbytes,
                            async_op, (flat,))

    def recv(self, t, src, async_op=False):
        flat = self._flat(t)
        nbytes = t.numel() * t.element_size()
        if not self._on_host(flat):
            return self._p2p().recv(flat, src, t, nbytes, async_op)
        return self._native(f"recv<-{src}", lambda: self._engine.recv(flat.data_ptr(), nbytes, src), t, nbytes,
                            async_op, (flat,))

    def sendrecv(self, send, dst, recv, src, async_op=False):
        """Sends one tensor while receiving another (pipeline parallelism's paired transfers)."""
        sf, rf = self._flat(send), self._flat(recv)
        sb, rb = sf.numel() * sf.element_size(), rf.numel() * rf.element_size()
        if not self._on_host(sf):
            return self._p2p().sendrecv(sf, dst, rf, src, recv, sb + rb, async_op)
        return self._native(f"sendrecv->{dst}<-{src}",
                            lambda: self._engine.sendrecv(sf.data_ptr(), sb, dst, rf.data_ptr(), rb, src),
                            recv, sb + rb, async_op, (sf, rf))

    def barrier(self):
        """Returns once every rank has called it; ordered after this rank's earlier collectives."""
        if self._sym is not None:
            self._sym.quiesce()
        return self._native("barrier", self._engine.barrier, None, 0, False)

    def abort(self):
        """Marks the job failed so that every rank blocked in a collective raises promptly."""
        try:
            self._engine.abort()
        except Exception:
            pass

    def close(self):
        if self._closed:
            return
        self.barrier()  # no rank unmaps memory a peer may still be reading
        if self._nccl is not None:
            self._nccl.close()
            self._nccl = None
        if self._sym is not None:
            self._sym.close()
            self._sym = None
            self.barrier()
        self._closed = True
        self._engine.close()
        self._engine = None


def _worker(rank, size, fn, args, device, slot_bytes, slots, transport, priority, backend, job, gpus, results):
    if device == "cuda":
        index = gpus[rank] if gpus else rank
        torch.cuda.set_device(index)
        dev = torch.device("cuda", index)
    else:
        dev = torch.device("cpu")
        torch.set_num_threads(max(1, int(os.environ.get("TANDEM_CPU_THREADS", "1"))))
    g = Group(rank, size, dev, slot_bytes=slot_bytes, slots=slots, transport=transport, priority=priority,
              backend=backend, job=job)
    try:
        out = fn(g, *args)
        g.close()
    except BaseException as e:
        # Say what went wrong before waking the peers: they fail a moment later
        # with "rank r failed", and launch() reports the first cause, not those.
        if not isinstance(e, CommError) or "failed while this rank waited" not in str(e):
            import traceback

            with open(os.path.join(results, f"error-rank{rank}.txt"), "w") as f:
                f.write(traceback.format_exc())
        g.abort()  # peers blocked on this rank fail now, not after the timeout
        g._closed = True
        raise
    if out is not None:
        torch.save(out, os.path.join(results, f"rank{rank}.pt"))


def launch(fn, size, *args, device="cpu", slot_bytes=DEFAULT_SLOT_BYTES, slots=DEFAULT_SLOTS,
           transport=None, priority=None, backend=None, gpus=None):
    """Runs fn(group, *args) on `size` processes (one per GPU with device="cuda")
    and returns each rank's return value in rank order (tandem/comm.py:517-547).
    `gpus` gives the GPU index of each rank (default: rank r on GPU r).  Return
    values travel back through files, so keep them small."""
    import tempfile

    from .engine import lib

    lib()  # build once in the parent, not in every rank at the same time
    if device == "cuda":
        from .parallel.symm import cuda_lib

        cuda_lib()
    job = uuid.uuid4().hex[:12]
    with tempfile.TemporaryDirectory(prefix="tandem-") as results:
        try:
            mp.spawn(_worker, args=(size, fn, args, device, slot_bytes, slots, transport, priority, backend, job,
                                    gpus, results), nprocs=size, join=True)
        except Exception as e:
            causes = []
            for r in range(size):
                path = os.path.join(results, f"error-rank{r}.txt")
                if os.path.exists(path):
                    with open(path) as f:
                        causes.append(f"rank {r} failed:\n{f.read()}")
            if causes:
                raise CommError("\n".join(causes)) from e
            raise
        out = []
        for r in range(size):
            path = os.path.join(results, f"rank{r}.pt")
            out.append(torch.load(path, weights_only=False) if os.path.exists(path) else None)
    return out
