"""Point-to-point transfers between GPU ranks: NCCL send/recv through
torch.distributed, started on first use.  Pipeline stages exchange activations
and gradients with these (the reference moves them through its own slot
transport: tandem/comm.py:411-448, tandem/csrc/collectives.cpp:350-379).
Transfers are ordered after the caller's stream, and `wait()` is a stream
dependency, so a stage can queue compute behind a receive without blocking
the host."""

import os
import tempfile

import torch


class _NcclWork:
    def __init__(self, name, group, works, result, nbytes, keep):
        self.name, self._group, self._works, self.result, self._nbytes, self._keep = name, group, works, result, nbytes, keep

    def wait(self):
        for w in self._works:
            w.wait()
        self._keep = ()
        return self.result

    def is_completed(self):
        return all(w.is_completed() for w in self._works)


class NcclP2P:
    def __init__(self, group):
        import torch.distributed as dist

        self.dist, self.g = dist, group
        self._own = False
        if dist.is_initialized():
            if dist.get_world_size() != group.size or dist.get_rank() != group.rank:
                raise RuntimeError("the torch.distributed process group does not match this Group")
        else:
            path = os.path.join(tempfile.gettempdir(), f"tb2-nccl-{group.job}")
            dist.init_process_group("nccl", init_method=f"file://{path}", rank=group.rank, world_size=group.size,
                                    device_id=group.device)
            self._own = True

    # ---- lanes for pipeline stages
    # Activations travel down the pipeline on one communicator, gradients travel up on another.  Each (pair of
    # stages, lane) then carries one direction only, so a receive can be posted long before its data exists without
    # ever standing in front of a send to the same peer on the same NCCL stream (which is how early receives
    # deadlock when both directions share a communicator).
    def lane(self, name):
        if not hasattr(self, "_lanes"):
            self._lanes = {"act": None}  # None: the default process group
            self._lanes["grad"] = self.dist.new_group(list(range(self.g.size)), backend="nccl")  # collective: every rank calls it
            self._side = torch.cuda.Stream(self.g.device)
            self._connect_neighbours()
        return self._lanes[name]

    def _connect_neighbours(self):
        """NCCL sets up the connection between two ranks at their first transfer on a communicator, and that set-up
        is a host-side rendezvous of both.  A receive posted ahead of time would sit in it until the sender reaches
        its first send -- which may itself depend on this rank's progress.  So every pair of neighbouring stages
        exchanges one element in both directions on both lanes here, symmetrically, before any real traffic."""
        r, n = self.g.rank, self.g.size
        for group in self._lanes.values():
            ops, keep = [], []
            for peer in (r - 1, r + 1):
                if 0 <= peer < n:
                    out = torch.zeros(1, device=self.g.device)
                    inp = torch.zeros(1, device=self.g.device)
                    keep += [out, inp]
                    ops.append(self.dist.P2POp(self.dist.isend, out, peer, group=group))
                    ops.append(self.dist.P2POp(self.dist.irecv, inp, peer, group=group))
            if ops:
                for w in self.dist.batch_isend_irecv(ops):
                    w.wait()
        torch.cuda.synchronize(self.g.device)

    def post_recv(self, shape, dtype, src, lane):
        """Starts a receive into a fresh buffer, independent of whatever is queued on the caller's stream.
        Returns (work, buffer); the buffer is usable on the caller's stream after work.wait()."""
        group = self.lane(lane)
        with torch.cuda.stream(self._side):
            buf = torch.empty(shape, device=self.g.device, dtype=dtype)
            work = self.dist.irecv(buf, src, group=group)
        return work, buf

    def claim(self, work, buf):
        """Orders the caller's stream after a posted receive and hands the buffer over to it."""
        work.wait()
        buf.record_stream(torch.cuda.current_stream(self.g.device))
        return buf

    def post_send(self, tensor, dst, lane):
        """Starts a send ordered after the caller's stream; the caller keeps (work, tensor) until the step ends."""
        return self.dist.isend(tensor, dst, group=self.lane(lane)), tensor

    def exchange(self, sends, recvs, shape, dtype):
        """One grouped NCCL call on the default communicator: every (tensor, dst) of `sends` and one fresh buffer per
        source in `recvs`, ordered after the caller's stream.  Returns (work, tensors to keep alive, received buffers);
        the buffers are usable on the caller's stream after claim(work, buffer)."""
        received = [torch.empty(shape, device=self.g.device, dtype=dtype) for _ in recvs]
        ops = [self.dist.P2POp(self.dist.isend, t, dst) for t, dst in sends]
        ops += [self.dist.P2POp(self.dist.irecv, buf, src) for buf, src in zip(received, recvs)]
        works = self.dist.batch_isend_irecv(ops)
        return _NcclWork("exchange", self.g, works, None, 0, ()), [t for t, _ in sends] + received, received

    def _done(self, name, works, result, nbytes, async_op, keep):
        work = _NcclWork(name, self.g, works, result, nbytes, keep)
        return work if async_op else work.wait()

    def send(self, flat, dst, result, nbytes, async_op):
        return self._done(f"send->{dst}", [self.dist.isend(flat, dst)], result, nbytes, async_op, (flat,))

    def recv(self, flat, src, result, nbytes, async_op):
        return self._done(f"recv<-{src}", [self.dist.irecv(flat, src)], result, nbytes, async_op, (flat,))

    def sendrecv(self, sf, dst, rf, src, result, nbytes, async_op):
        ops = [self.dist.P2POp(self.dist.isend, sf, dst), self.dist.P2POp(self.dist.irecv, rf, src)]
        return self._done(f"sendrecv->{dst}<-{src}", self.dist.batch_isend_irecv(ops), result, nbytes, async_op, (sf, rf))

    def close(self):
        if self._own and self.dist.is_initialized():
            torch.cuda.synchronize(self.g.device)
            self.dist.destroy_process_group()
            self._own = False
