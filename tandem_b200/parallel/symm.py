"""Symmetric memory and the GPU collectives built on it.

Each rank cudaMalloc's heap segments and exports them through CUDA IPC; every
rank maps every peer's segments, so the same (segment, offset) names a buffer
on all ranks.  The allocator is deterministic: ranks that make the same
sequence of alloc()/free() calls get the same offsets, with no communication
per allocation.  Collectives are single kernels from libtb200_cuda.so
(tandem_b200/cuda/collectives.cu) launched on one high-priority stream.

A tensor that lives in the heap (DDP buckets, ZeRO flat buffers, FSDP shards,
anything from Group.empty()) is reduced or gathered in place, zero-copy.  Any
other CUDA tensor is staged through a symmetric scratch area inside the same
kernel (copy-in, collective, copy-out fused), in pieces if it is larger.

This replaces the reference's per-peer slot arrays, interprocess events and
host-driven piece loop (tandem/csrc/cuda_links.cpp:43-160).
"""

import ctypes
import functools
import os
import time

import numpy as np
import torch

MAX_RANKS = 8
MAX_BLOCKS = 128
ALIGN = 256
FLAG_BYTES = MAX_BLOCKS * MAX_RANKS * 4
ALGO = {"auto": 0, "oneshot": 1, "twoshot": 2, "nvls": 3}


class AdamArgs(ctypes.Structure):
    _fields_ = [("param", ctypes.c_void_p), ("exp_avg", ctypes.c_void_p), ("exp_avg_sq", ctypes.c_void_p),
                ("shadow", ctypes.c_void_p), ("decay", ctypes.c_float), ("w1", ctypes.c_float), ("b2", ctypes.c_float),
                ("w2", ctypes.c_float), ("inv_bias2_sqrt", ctypes.c_float), ("eps", ctypes.c_float),
                ("neg_step", ctypes.c_float), ("do_decay", ctypes.c_int), ("scalars_dev", ctypes.c_void_p)]

    @staticmethod
    def _check(param, exp_avg, exp_avg_sq, shadow):
        # The kernel addresses param / exp_avg / exp_avg_sq as float and shadow as bf16: anything else would make it
        # read and write past the arrays.
        for name, t in (("param", param), ("exp_avg", exp_avg), ("exp_avg_sq", exp_avg_sq)):
            if t.dtype != torch.float32:
                raise TypeError(f"AdamArgs: {name} must be float32 (got {t.dtype}); 16-bit shards are stepped through their fp32 master")
        if shadow is not None and shadow.dtype != torch.bfloat16:
            raise TypeError(f"AdamArgs: shadow must be bfloat16 (got {shadow.dtype})")
        if not (param.numel() == exp_avg.numel() == exp_avg_sq.numel()) or (shadow is not None and shadow.numel() != param.numel()):
            raise ValueError("AdamArgs: param, moments and shadow must have the same number of elements")

    @classmethod
    def on_device(cls, param, exp_avg, exp_avg_sq, scalars_dev, shadow=None):
        """The step's constants are read by the kernel from `scalars_dev` (eight floats written on the device by
        ops.elementwise.adam_prepare) instead of being baked into the launch: for steps replayed as a CUDA graph."""
        cls._check(param, exp_avg, exp_avg_sq, shadow)
        if scalars_dev.dtype != torch.float32 or scalars_dev.numel() < 8 or not scalars_dev.is_cuda:
            raise TypeError("AdamArgs.on_device: scalars_dev must be a CUDA float32 tensor of 8 elements")
        return cls(param.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), shadow.data_ptr() if shadow is not None else None,
                   0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0, scalars_dev.data_ptr())

    @classmethod
    def make(cls, param, exp_avg, exp_avg_sq, scalars, do_decay, shadow=None):
        cls._check(param, exp_avg, exp_avg_sq, shadow)
        decay, w1, b2, w2, bias2_sqrt, eps, neg_step = scalars
        inv = float(np.float32(1.0) / np.float32(bias2_sqrt))
        return cls(param.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(),
                   shadow.data_ptr() if shadow is not None else None, decay, w1, b2, w2, inv, eps, neg_step, int(do_decay), None)


@functools.cache
def cuda_lib():
    """libtb200_cuda.so through ctypes, built in-tree if it is missing or stale."""
    from ..utils import build

    path = build.build_cuda(verbose=os.environ.get("TANDEM_BUILD_VERBOSE") == "1")
    if path is None or not os.path.exists(path):
        raise RuntimeError("libtb200_cuda.so is missing and could not be built (is nvcc installed?)")
    lib = ctypes.CDLL(path)
    vp, i, ll, d, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_double, ctypes.c_float
    pp = ctypes.POINTER(ctypes.c_void_p)
    pll = ctypes.POINTER(ctypes.c_longlong)
    sig = {
        "tb_last_error": ([], ctypes.c_char_p),
        "tb_error_string": ([i], ctypes.c_char_p),
        "tb_launch_count": ([i], ll),
        "tb_malloc": ([pp, ctypes.c_size_t], i),
        "tb_free": ([vp], i),
        "tb_ipc_export": ([vp, vp], i),
        "tb_ipc_open": ([vp, pp], i),
        "tb_ipc_close": ([vp], i),
        "tb_enable_peer": ([i], i),
        "tb_can_access_peer": ([i, i], i),
        "tb_status_alloc": ([pp, pp, ctypes.c_size_t], i),
        "tb_status_free": ([vp], i),
        "tb_memset_async": ([vp, i, ctypes.c_size_t, vp], i),
        "tb_memcpy_async": ([vp, vp, ctypes.c_size_t, vp], i),
        "tb_device_sync": ([], i),
        "tb_comm_create": ([i, i, i, pp, pp, vp, d, i], vp),
        "tb_comm_destroy": ([vp], None),
        "tb_comm_set_timeout": ([vp, d], None),
        "tb_comm_set_max_blocks": ([vp, i], None),
        "tb_barrier": ([vp, vp], i),
        "tb_all_reduce": ([vp, pp, pp, pp, ll, i, i, i, i, vp], i),
        "tb_all_reduce_nvls": ([vp, vp, ll, i, i, vp], i),
        "tb_all_gather_nvls": ([vp, vp, vp, ll, ll, ll, vp], i),
        "tb_reduce_scatter_nvls": ([vp, vp, vp, ll, pll, i, i, vp, ctypes.POINTER(AdamArgs), vp], i),
        "tb_broadcast_nvls": ([vp, vp, vp, ll, i, vp], i),
        "tb_reduce_scatter": ([vp, pp, pp, ll, pll, i, i, i, pp, ctypes.POINTER(AdamArgs), vp], i),
        "tb_gather_pull": ([vp, pp, pp, pll, pll, pll, pp, i, ll, vp], i),
        "tb_adamw": ([vp, vp, i, vp, vp, vp, ll, ctypes.POINTER(f), i, f, vp], i),
        "tb_multi_copy": ([pp, pp, pll, i, vp], i),
        "tb_adam_prepare": ([vp, d, d, d, d, d, vp, vp], i),
        "tb_adamw_dev": ([vp, vp, i, vp, vp, vp, ll, vp, vp], i),
    }
    for name, (argtypes, restype) in sig.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = argtypes, restype
    ull = ctypes.c_ulonglong
    pi = ctypes.POINTER(i)
    pull = ctypes.POINTER(ull)
    for name, (argtypes, restype) in {
        "tb_vmm_last_error": ([], ctypes.c_char_p),
        "tb_vmm_probe": ([i, pi], i),
        "tb_vmm_granularity": ([i, i, ll], ll),
        "tb_vmm_create": ([ll, ll, i, pp, pi, pull], i),
        "tb_vmm_import": ([i, ll, ll, i, pp, pull], i),
        "tb_vmm_release": ([vp, ll, ull], i),
        "tb_mc_create": ([ll, i, pi, pull], i),
        "tb_mc_import": ([i, pull], i),
        "tb_mc_add_device": ([ull, i], i),
        "tb_mc_bind_and_map": ([ull, ull, ll, ll, i, pp], i),
        "tb_mc_release": ([ull, vp, ll, i], i),
        "tb_close_fd": ([i], i),
    }.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = argtypes, restype
    # TANDEM_PDL=0: launch the compute kernels without programmatic dependent launch (for A/B measurements)
    lib.tb_set_pdl.argtypes, lib.tb_set_pdl.restype = [i], None
    lib.tb_set_pdl(0 if os.environ.get("TANDEM_PDL", "1") == "0" else 1)
    return lib


def check_rc(rc, what):
    if rc != 0:
        lib = cuda_lib()
        msg = lib.tb_error_string(rc).decode() if rc > 0 else f"code {rc}"
        raise RuntimeError(f"{what} failed: {msg} ({lib.tb_last_error().decode()})")


def _ptr_array(values, n=None):
    n = n or len(values)
    arr = (ctypes.c_void_p * n)()
    for k, v in enumerate(values):
        arr[k] = v
    return arr


def _ll_array(values):
    return (ctypes.c_longlong * len(values))(*values)


class _Raw:
    """A device address range exposed through the CUDA array interface."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def tensor_at(ptr, numel, dtype, device):
    """A tensor over memory this library owns (it does not free it)."""
    nbytes = max(numel, 1) * torch.empty(0, dtype=dtype).element_size()
    t = torch.as_tensor(_Raw(ptr, nbytes), device=device)
    return t.view(dtype)[:numel]


def split_offsets(numel, n, sizes=None):
    """Element offsets [o_0 .. o_n] of the rank chunks (torch.tensor_split, or explicit sizes)."""
    if sizes is None:
        base, extra = divmod(numel, n)
        sizes = [base + (1 if r < extra else 0) for r in range(n)]
    offs = [0]
    for s in sizes:
        offs.append(offs[-1] + int(s))
    return offs


class Heap:
    """Deterministic first-fit allocator over equally sized segments on every rank."""

    def __init__(self):
        self.segments = []  # [(bytes, [base pointer per rank])]
        self.multicast = []  # per segment: NVSwitch multicast address of the segment, or 0
        self.free = []  # [(segment, offset, bytes)], sorted
        self.used = {}  # (segment, offset) -> bytes

    def add_segment(self, nbytes, bases, multicast=0):
        self.segments.append((nbytes, bases))
        self.multicast.append(int(multicast or 0))
        self.free.append((len(self.segments) - 1, 0, nbytes))

    def take(self, nbytes):
        nbytes = (max(nbytes, 1) + ALIGN - 1) // ALIGN * ALIGN
        for k, (seg, off, size) in enumerate(self.free):
            if size >= nbytes:
                if size == nbytes:
                    self.free.pop(k)
                else:
                    self.free[k] = (seg, off + nbytes, size - nbytes)
                self.used[(seg, off)] = nbytes
                return seg, off
        return None

    def give(self, seg, off):
        nbytes = self.used.pop((seg, off))
        self.free.append((seg, off, nbytes))
        self.free.sort()
        merged = []
        for s, o, b in self.free:
            if merged and merged[-1][0] == s and merged[-1][1] + merged[-1][2] == o:
                merged[-1] = (s, merged[-1][1], merged[-1][2] + b)
            else:
                merged.append((s, o, b))
        self.free = merged

    def locate(self, rank, ptr, nbytes):
        for seg, (size, bases) in enumerate(self.segments):
            base = bases[rank]
            if base <= ptr and ptr + nbytes <= base + size:
                return seg, ptr - base
        return None

    def peers(self, seg, off):
        return [b + off for b in self.segments[seg][1]]


def swap_fds(job, tag, rank, n, barrier, timeout, mine=None, root=None):
    """File descriptors between the ranks of a job over abstract Unix datagram sockets (SCM_RIGHTS).
    root None: every rank sends `mine` to every other rank; returns {rank: fd} with the own entry = mine.
    root given: only the root sends `mine`; the others return {root: fd}.  `barrier` is a host barrier over the
    same ranks.  The received descriptors are new ones in this process; the caller closes them."""
    import array
    import socket
    import struct

    def address(q):
        return b"\0tb2-" + job.encode() + b"-" + tag.encode() + b"-" + str(q).encode()

    sock = socket.socket(socket.AF_UNIX, socket.SOCK_DGRAM)
    try:
        sock.bind(address(rank))
        sock.settimeout(timeout)
        barrier()  # every rank's socket exists
        got = {}
        if root is None or root == rank:
            rights = [(socket.SOL_SOCKET, socket.SCM_RIGHTS, array.array("i", [mine]))]
            for q in range(n):
                if q != rank:
                    sock.sendmsg([struct.pack("i", rank)], rights, 0, address(q))
            got[rank] = mine
        expect = n if root is None else 1
        while len(got) < expect:
            msg, fds, _flags, _addr = socket.recv_fds(sock, 16, 1)
            got[struct.unpack("i", msg[:4])[0]] = fds[0]
        barrier()  # nobody closes a socket a peer may still be sending to
        return got
    finally:
        sock.close()


class SymmetricComm:
    """The GPU side of a Group (one process per GPU)."""

    def __init__(self, group):
        from ..comm import DTYPE_CODE, CommError

        self._codes, self._error = DTYPE_CODE, CommError
        self.g = group
        self.lib = cuda_lib()
        self.n, self.rank, self.device = group.size, group.rank, group.device
        if self.n > MAX_RANKS:
            raise CommError(f"the GPU collectives support at most {MAX_RANKS} ranks")
        torch.cuda.set_device(self.device)
        torch.cuda.current_stream(self.device).synchronize()  # make sure a context exists
        self.stream = torch.cuda.Stream(self.device, priority=group.priority)
        self.segment_bytes = int(os.environ.get("TANDEM_SYMM_BYTES", str(1 << 30)))
        self.heap = Heap()
        self._torch_segments = []  # segments that came from torch's symmetric-memory allocator (kept alive here)
        self._vmm_segments = []  # segments created through the driver's virtual-memory API (own, imported, multicast)
        self._nvls_error = None
        self._owned = []  # this rank's cudaMalloc'd segments
        self._opened = []  # peers' segments mapped here
        self._add_segment(max(self.segment_bytes, 4 << 20))
        # control block: flags in the heap (peers write them), barrier counters private
        seg, off = self.heap.take(FLAG_BYTES)
        flags = self.heap.peers(seg, off)
        self._epoch = ctypes.c_void_p()
        check_rc(self.lib.tb_malloc(ctypes.byref(self._epoch), MAX_BLOCKS * 4), "cudaMalloc")
        host, dev = ctypes.c_void_p(), ctypes.c_void_p()
        check_rc(self.lib.tb_status_alloc(ctypes.byref(host), ctypes.byref(dev), 64), "cudaHostAlloc")
        self._status_host = host
        self._status = (ctypes.c_uint32 * 16).from_address(host.value)
        self.device_timeout = float(os.environ.get("TANDEM_DEVICE_TIMEOUT", str(min(group.timeout, 30.0))))
        self.max_blocks = int(os.environ.get("TANDEM_COMM_BLOCKS", "128"))
        epochs = [self._epoch.value if q == self.rank else None for q in range(self.n)]
        self.comm = self.lib.tb_comm_create(self.n, self.rank, 0, _ptr_array(flags), _ptr_array(epochs), dev,
                                            self.device_timeout, self.max_blocks)
        # A second, independent set of flags and counters for blocking calls, which run in line on the
        # caller's stream: kernels of the two channels may overlap on the GPU without sharing barrier state.
        # (All blocking collectives of a rank must come from one stream at a time.)
        seg2, off2 = self.heap.take(FLAG_BYTES)
        self._epoch2 = ctypes.c_void_p()
        check_rc(self.lib.tb_malloc(ctypes.byref(self._epoch2), MAX_BLOCKS * 4), "cudaMalloc")
        epochs2 = [self._epoch2.value if q == self.rank else None for q in range(self.n)]
        self.comm_inline = self.lib.tb_comm_create(self.n, self.rank, 0, _ptr_array(self.heap.peers(seg2, off2)),
                                                   _ptr_array(epochs2), dev, self.device_timeout, self.max_blocks)
        self._launch_comm = self.comm
        self.scratch_half = int(os.environ.get("TANDEM_SCRATCH_BYTES", str(32 << 20)))
        self._scratch = [self._take(self.scratch_half) for _ in range(2)]
        self._half = 0
        self._launch_stream = self.stream
        self._ptr_cache = {}
        self.exact16 = os.environ.get("TANDEM_EXACT16", "0") == "1"
        self.nvls_min_bytes = int(os.environ.get("TANDEM_NVLS_MIN_BYTES", str(1 << 20)))
        # Measured: with 2 ranks the peer-to-peer two-shot kernel is faster than going through the switch's
        # reduction (530 vs 396 GB/s bus at 256 MB); the switch pays off as the peer count grows.
        self.nvls_min_ranks = int(os.environ.get("TANDEM_NVLS_MIN_RANKS", "4"))
        self.algo = ALGO[os.environ.get("TANDEM_ALLREDUCE", "auto")]
        # clock calibration for traces: device event time -> host perf_counter
        self._t0_event = torch.cuda.Event(enable_timing=True)
        self._t0_event.record(self.stream)
        self._t0_event.synchronize()
        self._t0_host = time.perf_counter()

    # ------------------------------------------------------------------ heap
    def _add_segment(self, nbytes):
        """Collective: every rank allocates a segment and maps everyone else's.  First choice is this library's own
        path (cuMemCreate, descriptors over Unix sockets, its own multicast binding for the multimem kernels;
        TANDEM_VMM=0 skips it).  If the ranks do not all succeed: torch's symmetric-memory allocator when a
        torch.distributed NCCL group is in place (and TANDEM_NVLS != 0), else cudaMalloc + CUDA IPC (no multicast)."""
        if self.n > 1 and os.environ.get("TANDEM_VMM", "1") != "0" and self._add_segment_vmm(nbytes):
            return
        if self.n > 1 and os.environ.get("TANDEM_NVLS", "1") != "0" and self._add_segment_multicast(nbytes):
            return
        mine = ctypes.c_void_p()
        check_rc(self.lib.tb_malloc(ctypes.byref(mine), nbytes), f"cudaMalloc of a {nbytes >> 20} MiB symmetric segment")
        self._owned.append(mine.value)
        handle = (ctypes.c_ubyte * 64)()
        check_rc(self.lib.tb_ipc_export(mine, handle), "cudaIpcGetMemHandle")
        table = torch.zeros(self.n, 64, dtype=torch.uint8)
        table[self.rank] = torch.frombuffer(bytearray(handle), dtype=torch.uint8)
        self.g._native("handles", lambda: self.g._engine.all_gather(table.data_ptr(), table.numel(), 8, [64] * self.n),
                       None, 0, False, (table,))
        bases = []
        for q in range(self.n):
            if q == self.rank:
                bases.append(mine.value)
                continue
            raw = (ctypes.c_ubyte * 64)(*table[q].tolist())
            out = ctypes.c_void_p()
            check_rc(self.lib.tb_ipc_open(raw, ctypes.byref(out)), f"cudaIpcOpenMemHandle of rank {q}'s segment")
            self._opened.append(out.value)
            bases.append(out.value)
        self.heap.add_segment(nbytes, bases)

    # ---- segments created through the driver's virtual-memory API, with this library's own multicast binding
    def _agree(self, ok):
        """True if every rank says ok (an all-gather over the host control plane)."""
        votes = torch.zeros(self.n, dtype=torch.int64)
        votes[self.rank] = 1 if ok else 0
        self.g._native("agree", lambda: self.g._engine.all_gather(votes.data_ptr(), votes.numel(), 4, [1] * self.n), None, 0, False, (votes,))
        return bool(votes.min().item() == 1)

    def _host_barrier(self):
        self.g._native("barrier", self.g._engine.barrier, None, 0, False)

    def _swap_fds(self, tag, mine=None, root=None):
        return swap_fds(self.g.job, tag, self.rank, self.n, self._host_barrier, max(5.0, min(self.g.timeout, 120.0)), mine, root)

    def _add_segment_vmm(self, nbytes):
        """cuMemCreate + POSIX-fd exchange + mapping of every peer's segment; if the GPUs support it (and TANDEM_NVLS
        is not 0), the segments are also bound to one multicast object whose mapping serves the multimem kernels.
        Every step ends in an agreement between the ranks, so either all ranks use this segment or none does."""
        lib, dev = self.lib, self.device.index
        caps = (ctypes.c_int * 2)()
        ok = lib.tb_vmm_probe(dev, caps) == 0 and caps[0] == 1
        if not self._agree(ok):
            self._nvls_error = "the driver cannot export device memory as file descriptors on every rank"
            return False
        want_mc = self._agree(caps[1] == 1) and os.environ.get("TANDEM_NVLS", "1") != "0"
        gran = lib.tb_vmm_granularity(dev, self.n if want_mc else 1, nbytes)
        sizes = torch.zeros(self.n, dtype=torch.int64)
        sizes[self.rank] = gran
        self.g._native("sizes", lambda: self.g._engine.all_gather(sizes.data_ptr(), sizes.numel(), 4, [1] * self.n), None, 0, False, (sizes,))
        gran = int(sizes.max().item())
        if gran <= 0:
            return False
        size = (nbytes + gran - 1) // gran * gran
        ptr, fd, handle = ctypes.c_void_p(), ctypes.c_int(-1), ctypes.c_ulonglong(0)
        created = lib.tb_vmm_create(size, gran, dev, ctypes.byref(ptr), ctypes.byref(fd), ctypes.byref(handle)) == 0
        if not self._agree(created):
            if created:
                lib.tb_close_fd(fd.value)
                lib.tb_vmm_release(ptr, size, handle.value)
            self._nvls_error = lib.tb_vmm_last_error().decode()
            return False
        self._seg_count = getattr(self, "_seg_count", 0) + 1
        tag = f"s{self._seg_count}"
        fds = self._swap_fds(tag, fd.value)
        bases, imported, good = [], [], True
        for q in range(self.n):
            if q == self.rank:
                bases.append(ptr.value)
                continue
            p, h = ctypes.c_void_p(), ctypes.c_ulonglong(0)
            if good and lib.tb_vmm_import(fds[q], size, gran, dev, ctypes.byref(p), ctypes.byref(h)) == 0:
                imported.append((p.value, h.value))
                bases.append(p.value)
            else:
                good = False
            lib.tb_close_fd(fds[q])
        lib.tb_close_fd(fd.value)

        def undo():
            for p, h in imported:
                lib.tb_vmm_release(p, size, h)
            self._host_barrier()  # nobody still maps this rank's memory
            lib.tb_vmm_release(ptr, size, handle.value)

        if not self._agree(good):
            self._nvls_error = lib.tb_vmm_last_error().decode()
            undo()
            return False
        mc_handle, mc_ptr = 0, 0
        if want_mc:
            mc_handle, mc_ptr = self._bind_multicast(tag, size, gran, handle.value)
        self._vmm_segments.append({"size": size, "own": (ptr.value, handle.value), "imported": imported, "mc": (mc_handle, mc_ptr)})
        self.heap.add_segment(size, bases, mc_ptr)
        return True

    def _bind_multicast(self, tag, size, gran, mem_handle):
        """(multicast handle, multicast address) or (0, 0) when the object cannot be set up on every rank."""
        lib, dev = self.lib, self.device.index
        mc, fd = ctypes.c_ulonglong(0), ctypes.c_int(-1)
        ok = True
        if self.rank == 0:
            ok = lib.tb_mc_create(size, self.n, ctypes.byref(fd), ctypes.byref(mc)) == 0
        if not self._agree(ok):
            self._nvls_error = lib.tb_vmm_last_error().decode()
            return 0, 0
        got = self._swap_fds(tag + "m", fd.value if self.rank == 0 else None, root=0)
        if self.rank != 0:
            ok = lib.tb_mc_import(got[0], ctypes.byref(mc)) == 0
            lib.tb_close_fd(got[0])
        else:
            lib.tb_close_fd(fd.value)
        ok = ok and lib.tb_mc_add_device(mc.value, dev) == 0
        if not self._agree(ok):  # agreement doubles as "every device has joined"
            self._nvls_error = lib.tb_vmm_last_error().decode()
            return 0, 0
        mapped = ctypes.c_void_p()
        ok = lib.tb_mc_bind_and_map(mc.value, mem_handle, size, gran, dev, ctypes.byref(mapped)) == 0
        if not self._agree(ok):
            self._nvls_error = lib.tb_vmm_last_error().decode()
            if ok:
                lib.tb_mc_release(mc.value, mapped, size, dev)
            return 0, 0
        return mc.value, mapped.value

    def _add_segment_multicast(self, nbytes):
        try:
            import torch.distributed as dist

            if not (dist.is_available() and dist.is_initialized() and dist.get_backend() == "nccl"
                    and dist.get_world_size() == self.n and dist.get_rank() == self.rank):
                return False
            import torch.distributed._symmetric_memory as symm_mem

            t = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
            handle = symm_mem.rendezvous(t, dist.group.WORLD)
            bases = [int(p) for p in handle.buffer_ptrs]
            mc = int(handle.multicast_ptr or 0)  # 0 when the machine has no NVSwitch multicast
        except Exception as e:  # no multicast on this machine / torch build: fall back to CUDA IPC
            self._nvls_error = repr(e)
            return False
        t.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier()
        self._torch_segments.append((t, handle))
        self.heap.add_segment(nbytes, bases, mc)
        return True

    def _take(self, nbytes):
        where = self.heap.take(nbytes)
        if where is None:
            self._add_segment(max(self.segment_bytes, (nbytes + ALIGN - 1) // ALIGN * ALIGN))
            where = self.heap.take(nbytes)
        return where

    def alloc(self, numel, dtype, zero=True):
        esz = torch.empty(0, dtype=dtype).element_size()
        seg, off = self._take(numel * esz)
        t = tensor_at(self.heap.segments[seg][1][self.rank] + off, numel, dtype, self.device)
        if zero:
            t.zero_()
        return t

    def free(self, t):
        self._ptr_cache.clear()
        where = self.heap.locate(self.rank, t.data_ptr(), 1)
        if where is not None and where in self.heap.used:
            self.heap.give(*where)

    def _peers_of(self, t):
        """Peer addresses of a tensor that lives in the heap, else None."""
        ptr = t.data_ptr()
        nbytes = max(t.numel() * t.element_size(), 1)
        hit = self._ptr_cache.get(ptr)
        if hit is not None and hit[0] >= nbytes:
            return hit[1]
        where = self.heap.locate(self.rank, ptr, nbytes)
        if where is None:
            return None
        peers = self.heap.peers(*where)
        if len(self._ptr_cache) > 4096:
            self._ptr_cache.clear()
        self._ptr_cache[ptr] = (nbytes, peers)
        return peers

    def _multicast_of(self, t):
        """NVSwitch multicast address of a heap tensor, or 0."""
        where = self.heap.locate(self.rank, t.data_ptr(), max(t.numel() * t.element_size(), 1))
        if where is None or not self.heap.multicast[where[0]]:
            return 0
        return self.heap.multicast[where[0]] + where[1]

    @property
    def nvls(self):
        """True when the heap is bound to an NVSwitch multicast object (multimem kernels available)."""
        return any(self.heap.multicast)

    # ------------------------------------------------------------------ launching
    def _begin(self, name, tensors, async_op=True):
        """Picks the stream for this collective and orders it after the caller's work.  A blocking
        call runs on the caller's own stream (no events, no stream hop); an async one on the
        high-priority communication stream.  Returns the timing start event or None."""
        cur = torch.cuda.current_stream(self.device)
        registered = all(t is None or self._peers_of(t) is not None for t in tensors[:1])
        if not async_op and not self.g.tracing and registered:
            self._launch_stream, self._launch_comm = cur, self.comm_inline
            return None
        self._launch_stream, self._launch_comm = self.stream, self.comm
        ready = torch.cuda.Event()
        ready.record(cur)
        self.stream.wait_event(ready)
        for t in tensors:
            if t is not None and t.is_cuda and self._peers_of(t) is None:
                t.record_stream(self.stream)  # the caching allocator must not recycle it under the kernel
        if self.g.tracing:
            start = torch.cuda.Event(enable_timing=True)
            start.record(self.stream)
            return start
        return None

    def _end(self, name, start, result, nbytes, async_op):
        from ..comm import _StreamWork

        if self._launch_stream is not self.stream:  # ran in line on the caller's stream: already ordered
            if self._status[0] != 0:
                self.check()
            return result
        done = torch.cuda.Event(enable_timing=start is not None)
        done.record(self.stream)
        work = _StreamWork(name, self.g, done, result, nbytes, start)
        if async_op:
            return work
        return work.wait()

    def _next_scratch(self):
        self._half ^= 1
        return self.heap.peers(*self._scratch[self._half])

    def _wide_scratch(self, nbytes, stream):
        """Peer addresses of one staging block of at least nbytes, kept for later calls.  Every rank makes the same
        calls in the same order, so all ranks grow it together.  Unlike the two alternating halves there is only one
        such block per call kind: a barrier launch keeps this rank from overwriting what a slower peer still reads from the
        previous call."""
        if not hasattr(self, "_wide"):
            self._wide = {}
        lane = 0 if self._launch_comm is self.comm else 1  # blocking and asynchronous calls never share a block
        held = self._wide.get(lane)
        if held is None or held[1] < nbytes:
            if held is not None:
                torch.cuda.synchronize(self.device)
                self._ptr_cache.clear()
                self.heap.give(*held[0])
            size = (nbytes + (8 << 20) - 1) // (8 << 20) * (8 << 20)
            self._wide[lane] = held = (self._take(size), size)
        check_rc(self.lib.tb_barrier(self._launch_comm, stream), "barrier")
        return self.heap.peers(*held[0])

    def check(self):
        if self._status[0] != 0:
            code, rank, peer, epoch, block = (int(self._status[k]) for k in range(5))
            raise self._error(f"GPU collective gave up after {self.device_timeout:.1f}s: rank {rank} block {block} "
                              f"never saw rank {peer}'s signal for barrier {epoch} (code {code})")

    def resolve_spans(self, pending, out):
        for name, start, end, nbytes in pending:
            end.synchronize()
            t0 = self._t0_host + self._t0_event.elapsed_time(start) / 1e3
            t1 = self._t0_host + self._t0_event.elapsed_time(end) / 1e3
            out.append((name, t0, t1, nbytes))

    def quiesce(self):
        self.stream.synchronize()
        self.check()

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, flat, average, result, nbytes, async_op, algo=None):
        start = self._begin("all_reduce", [flat], async_op)
        code = self._codes[flat.dtype]
        algo = self.algo if algo is None else ALGO[algo]
        s = self._launch_stream.cuda_stream
        peers = self._peers_of(flat)
        if flat.numel() and self.n > 1:  # a group of one: the buffer already holds its own sum (and mean)
            mc = self._multicast_of(flat) if peers is not None and flat.dtype in (torch.float32, torch.bfloat16) else 0
            nbytes_ = flat.numel() * flat.element_size()
            want_nvls = algo == ALGO["nvls"] or (algo == ALGO["auto"] and self.n >= self.nvls_min_ranks and nbytes_ >= self.nvls_min_bytes and not self.exact16
                                                 and not torch.are_deterministic_algorithms_enabled())
            if mc and want_nvls and nbytes_ % 16 == 0 and mc % 16 == 0:
                check_rc(self.lib.tb_all_reduce_nvls(self._launch_comm, mc, flat.numel(), code, int(average), s), "all_reduce (NVLS)")
            elif peers is not None:
                check_rc(self.lib.tb_all_reduce(self._launch_comm, _ptr_array(peers), None, None, flat.numel(), code, int(average),
                                                int(self.exact16), algo, s), "all_reduce")
            else:
                # Not in the heap: copy each piece into this rank's scratch, reduce the scratch in place, copy
                # it back.  (The copies are separate launches on purpose: a block of the collective may only
                # assume that the peers' matching block has run, not that their whole grid has.)
                esz = flat.element_size()
                step = self.scratch_half // esz
                for lo in range(0, flat.numel(), step):
                    piece = flat[lo:lo + step]
                    scratch = self._next_scratch()
                    pbytes = piece.numel() * esz
                    check_rc(self.lib.tb_memcpy_async(scratch[self.rank], piece.data_ptr(), pbytes, s), "memcpy")
                    check_rc(self.lib.tb_all_reduce(self._launch_comm, _ptr_array(scratch), None, None, piece.numel(),
                                                    code, int(average), int(self.exact16), algo, s), "all_reduce")
                    check_rc(self.lib.tb_memcpy_async(piece.data_ptr(), scratch[self.rank], pbytes, s), "memcpy")
        return self._end("all_reduce", start, result, nbytes, async_op)

    def reduce_scatter(self, flat, sizes, average, result, nbytes, async_op, accumulate_into=None, adam=None):
        """Chunk r of `flat` summed over ranks into rank r's `flat` (in place).
        accumulate_into: a tensor shaped like the chunk that also receives `+= chunk`.
        adam: AdamArgs for a fused AdamW step with the chunk as the gradient."""
        start = self._begin("reduce_scatter", [flat, accumulate_into], async_op)
        code = self._codes[flat.dtype]
        offs = split_offsets(flat.numel(), self.n, sizes)
        s = self._launch_stream.cuda_stream
        peers = self._peers_of(flat)
        acc = _ptr_array([accumulate_into.data_ptr()]) if accumulate_into is not None and accumulate_into.numel() else None
        adam_p = ctypes.pointer(adam) if adam is not None and offs[self.rank + 1] > offs[self.rank] else None
        if flat.numel():
            esz = flat.element_size()
            nbytes_ = flat.numel() * esz
            mc = self._multicast_of(flat) if peers is not None and self.n > 1 and flat.dtype in (torch.float32, torch.bfloat16) else 0
            want_nvls = self.algo == ALGO["nvls"] or (self.algo == ALGO["auto"] and self.n >= self.nvls_min_ranks
                                                      and nbytes_ >= self.nvls_min_bytes and not self.exact16
                                                      and not torch.are_deterministic_algorithms_enabled())
            if mc and want_nvls and mc % 16 == 0 and flat.data_ptr() % 16 == 0 and all((o * esz) % 16 == 0 for o in offs):
                # the switch adds the ranks' copies of this rank's chunk (multimem.ld_reduce); same epilogues
                one = accumulate_into.data_ptr() if accumulate_into is not None and accumulate_into.numel() else None
                check_rc(self.lib.tb_reduce_scatter_nvls(self._launch_comm, mc, flat.data_ptr(), flat.numel(), _ll_array(offs), code,
                                                         int(average), one, adam_p, s), "reduce_scatter (NVLS)")
            elif peers is not None:
                check_rc(self.lib.tb_reduce_scatter(self._launch_comm, _ptr_array(peers), None, flat.numel(), _ll_array(offs), code,
                                                    int(average), int(self.exact16), acc, adam_p, s), "reduce_scatter")
            else:
                # not in the heap: through the scratch area, or through a staging block that grows to the largest
                # such call (the kernel needs the whole operand of every rank at once, so it cannot go piecewise)
                scratch = self._next_scratch() if nbytes_ <= self.scratch_half else self._wide_scratch(nbytes_, s)
                check_rc(self.lib.tb_memcpy_async(scratch[self.rank], flat.data_ptr(), flat.numel() * flat.element_size(), s), "memcpy")
                check_rc(self.lib.tb_reduce_scatter(self._launch_comm, _ptr_array(scratch), None,
                                                    flat.numel(), _ll_array(offs), code, int(average), int(self.exact16),
                                                    acc, adam_p, s), "reduce_scatter")
                lo, hi = offs[self.rank], offs[self.rank + 1]
                if hi > lo:  # the reduced chunk sits in the scratch: bring it home
                    esz = flat.element_size()
                    check_rc(self.lib.tb_memcpy_async(flat.data_ptr() + lo * esz, scratch[self.rank] + lo * esz,
                                                      (hi - lo) * esz, s), "memcpy")
        return self._end("reduce_scatter", start, result, nbytes, async_op)

    def _pull(self, srcs, dst, src_off, dst_off, lens, stage, sync, grid_bytes=0):
        """stage: address of this rank's piece to publish first (copied to srcs[rank] + src_off[rank] by a
        separate launch, so that it is complete before any peer's block can pass the barrier)."""
        s = self._launch_stream.cuda_stream
        if stage is not None and lens[self.rank] > 0:
            check_rc(self.lib.tb_memcpy_async(srcs[self.rank] + src_off[self.rank], stage, lens[self.rank], s), "memcpy")
        check_rc(self.lib.tb_gather_pull(self._launch_comm, _ptr_array(srcs), _ptr_array([dst]), _ll_array(src_off), _ll_array(dst_off),
                                         _ll_array(lens), None, int(sync), grid_bytes, s), "gather")

    def all_gather(self, flat, sizes, result, nbytes, async_op):
        start = self._begin("all_gather", [flat], async_op)
        esz = flat.element_size()
        offs = [o * esz for o in split_offsets(flat.numel(), self.n, sizes)]
        lens = [offs[q + 1] - offs[q] for q in range(self.n)]
        peers = self._peers_of(flat)
        if flat.numel() and self.n > 1:
            mc = self._multicast_of(flat) if peers is not None else 0
            # measured at 8 ranks: multicasting wins or ties up to 64 MB in total (1 MB: 25 us vs 38 us pulled),
            # loses beyond (256 MB: 656 us vs 404 us)
            total = offs[-1]
            want_nvls = self.algo == ALGO["nvls"] or (self.algo == ALGO["auto"] and self.n >= self.nvls_min_ranks
                                                      and self.nvls_min_bytes <= total <= (32 << 20))
            if mc and want_nvls and mc % 16 == 0 and flat.data_ptr() % 16 == 0 and all(o % 16 == 0 for o in offs):
                # each rank multicasts its own chunk through the switch (multimem.st)
                check_rc(self.lib.tb_all_gather_nvls(self._launch_comm, flat.data_ptr(), mc, offs[self.rank], lens[self.rank], max(lens),
                                                     self._launch_stream.cuda_stream), "all_gather (NVLS)")
            elif peers is not None:
                self._pull(peers, flat.data_ptr(), offs[:-1], offs[:-1], lens, None, True)
            else:
                step = self.scratch_half
                for lo in range(0, max(lens), step):  # piece k of every rank's chunk per launch
                    plen = [max(0, min(l - lo, step)) for l in lens]
                    mine = flat.data_ptr() + offs[self.rank] + lo if plen[self.rank] else None
                    self._pull(self._next_scratch(), flat.data_ptr(), [0] * self.n, [offs[q] + lo for q in range(self.n)],
                               plen, mine, True)
        return self._end("all_gather", start, result, nbytes, async_op)

    def gather_shards(self, full, shard, sizes, async_op=True, lo=None, hi=None):
        """full[off_q : off_q + sizes[q]] = rank q's `shard`, for every q, with no
        handshake between ranks: `shard` is a heap tensor allocated identically on
        every rank whose contents only change between barriers (parameter shards
        between optimizer steps).  The kernel still opens with a system-scope fence:
        measured on B200, without it loads of a peer's memory can return lines from
        before the peer's last update even though a barrier kernel ran in between."""
        start = self._begin("all_gather", [full], async_op)
        esz = full.element_size()
        offs = [o * esz for o in split_offsets(full.numel(), self.n, sizes)]
        lens = [offs[q + 1] - offs[q] for q in range(self.n)]
        peers = self._peers_of(shard)
        if peers is None:
            raise self._error("gather_shards needs a shard allocated with Group.empty()")
        src_off, dst_off = [0] * self.n, offs[:-1]
        if lo is not None:  # only the elements [lo, hi) of the flat buffer: each rank's shard clipped to that range
            a, b = lo * esz, hi * esz
            starts = [max(offs[q], a) for q in range(self.n)]
            lens = [max(0, min(offs[q + 1], b) - starts[q]) for q in range(self.n)]
            src_off = [starts[q] - offs[q] if lens[q] else 0 for q in range(self.n)]
            dst_off = [starts[q] if lens[q] else 0 for q in range(self.n)]
        self._pull(peers, full.data_ptr(), src_off, dst_off, lens, None, 2, max(max(lens), 1))  # 2: fence, no handshake
        return self._end("all_gather", start, full, sum(lens), async_op)

    def broadcast(self, flat, root, result, nbytes, async_op):
        start = self._begin("broadcast", [flat], async_op)
        total = flat.numel() * flat.element_size()
        peers = self._peers_of(flat)
        if total and self.n > 1:
            mc = self._multicast_of(flat) if peers is not None else 0
            want_nvls = self.algo == ALGO["nvls"] or (self.algo == ALGO["auto"] and self.n >= self.nvls_min_ranks
                                                      and total >= self.nvls_min_bytes)
            if mc and want_nvls and total % 16 == 0 and mc % 16 == 0 and flat.data_ptr() % 16 == 0:
                # the root writes once to the multicast address; the switch replicates into every rank's copy
                check_rc(self.lib.tb_broadcast_nvls(self._launch_comm, flat.data_ptr(), mc, total, root,
                                                    self._launch_stream.cuda_stream), "broadcast (NVLS)")
            elif peers is not None:
                if total >= (1 << 20) and self.n > 2:
                    # scatter + all-gather: rank q pulls slice q from the root, then everyone pulls the other
                    # slices from their new holders, so the root sends each byte once instead of n-1 times.
                    cut = [(total * q // self.n) // 16 * 16 for q in range(self.n)] + [total]
                    lens = [cut[self.rank + 1] - cut[self.rank] if q == root else 0 for q in range(self.n)]
                    widest = max(cut[q + 1] - cut[q] for q in range(self.n))  # the same on every rank: grids must match
                    self._pull(peers, flat.data_ptr(), [cut[self.rank]] * self.n, [cut[self.rank]] * self.n, lens, None, True, widest)
                    lens = [0 if self.rank == root or q == self.rank else cut[q + 1] - cut[q] for q in range(self.n)]
                    self._pull(peers, flat.data_ptr(), cut[:-1], cut[:-1], lens, None, True, widest)
                else:
                    lens = [total if q == root else 0 for q in range(self.n)]
                    self._pull(peers, flat.data_ptr(), [0] * self.n, [0] * self.n, lens, None, True, total)
            else:
                step = self.scratch_half
                for lo in range(0, total, step):
                    plen = min(step, total - lo)
                    lens = [plen if q == root else 0 for q in range(self.n)]
                    stage = flat.data_ptr() + lo if self.rank == root else None
                    self._pull(self._next_scratch(), flat.data_ptr(), [0] * self.n, [lo] * self.n, lens, stage, True, plen)
        return self._end("broadcast", start, result, nbytes, async_op)

    def device_barrier(self, after_current=False):
        """A barrier on the communication stream (ranks meet on the device, the host does not block).
        The caller's stream waits for it either way; it also waits for the caller's earlier work."""
        start = self._begin("barrier", [], True)
        check_rc(self.lib.tb_barrier(self.comm, self.stream.cuda_stream), "barrier")
        return self._end("barrier", start, None, 0, False)

    def close(self):
        torch.cuda.synchronize(self.device)
        self.g._native("barrier", self.g._engine.barrier, None, 0, False)  # nobody is still reading our memory
        for p in self._opened:
            self.lib.tb_ipc_close(p)
        self._opened = []
        for seg in self._vmm_segments:  # multicast mappings and bindings go first, then the peers' mappings
            mc, mc_ptr = seg["mc"]
            if mc:
                self.lib.tb_mc_release(mc, mc_ptr, seg["size"], self.device.index)
            for p, h in seg["imported"]:
                self.lib.tb_vmm_release(p, seg["size"], h)
        self.g._native("barrier", self.g._engine.barrier, None, 0, False)  # everyone has unmapped
        for seg in self._vmm_segments:
            self.lib.tb_vmm_release(seg["own"][0], seg["size"], seg["own"][1])
        self._vmm_segments = []
        for p in self._owned:
            self.lib.tb_free(p)
        self._owned = []
        self.lib.tb_free(self._epoch)
        self.lib.tb_free(self._epoch2)
        self.lib.tb_comm_destroy(self.comm_inline)
        self.lib.tb_status_free(self._status_host)
        self.lib.tb_comm_destroy(self.comm)
        self.comm = None


class EmulatedRanks:
    """All ranks of a group on ONE GPU, driven by one process: every collective is
    a single cooperative launch whose blockIdx.y is the rank, so blocks that wait
    on one another are resident together.  For testing the kernels' multi-rank
    logic where only one GPU is available; not a transport."""

    def __init__(self, n, device="cuda:0", timeout_s=2.0, max_blocks=16):
        self.lib = cuda_lib()
        self.n = n
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self._flags = [torch.zeros(FLAG_BYTES // 4, dtype=torch.int32, device=self.device) for _ in range(n)]
        self._epochs = [torch.zeros(MAX_BLOCKS, dtype=torch.int32, device=self.device) for _ in range(n)]
        host, dev = ctypes.c_void_p(), ctypes.c_void_p()
        check_rc(self.lib.tb_status_alloc(ctypes.byref(host), ctypes.byref(dev), 64), "cudaHostAlloc")
        self._status_host = host
        self.status = (ctypes.c_uint32 * 16).from_address(host.value)
        self.comm = self.lib.tb_comm_create(n, 0, 1, _ptr_array([t.data_ptr() for t in self._flags]),
                                            _ptr_array([t.data_ptr() for t in self._epochs]), dev, timeout_s, max_blocks)

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def all_reduce(self, bufs, average=False, exact=False, algo="auto"):
        """bufs: one symmetric buffer per rank, reduced in place."""
        code = {torch.float32: 0, torch.float64: 1, torch.bfloat16: 2, torch.float16: 3, torch.int64: 4, torch.int32: 5}[bufs[0].dtype]
        numel = bufs[0].numel()
        check_rc(self.lib.tb_all_reduce(self.comm, _ptr_array([b.data_ptr() for b in bufs]), None, None, numel, code,
                                        int(average), int(exact), ALGO[algo], self._stream()), "all_reduce")

    def reduce_scatter(self, bufs, sizes=None, average=False, exact=False, accumulate_into=None, adam=None):
        code = {torch.float32: 0, torch.float64: 1, torch.bfloat16: 2, torch.float16: 3, torch.int64: 4, torch.int32: 5}[bufs[0].dtype]
        numel = bufs[0].numel()
        offs = split_offsets(numel, self.n, sizes)
        acc = _ptr_array([t.data_ptr() for t in accumulate_into]) if accumulate_into else None
        ad = (AdamArgs * self.n)(*adam) if adam else None
        check_rc(self.lib.tb_reduce_scatter(self.comm, _ptr_array([b.data_ptr() for b in bufs]), None, numel, _ll_array(offs),
                                            code, int(average), int(exact), acc, ad, self._stream()), "reduce_scatter")
        return offs

    def gather(self, srcs, dsts, src_off, dst_off, lens, stage=None, sync=True):
        st = _ptr_array([t.data_ptr() if t is not None else None for t in stage]) if stage else None
        check_rc(self.lib.tb_gather_pull(self.comm, _ptr_array([t.data_ptr() for t in srcs]), _ptr_array([t.data_ptr() for t in dsts]),
                                         _ll_array(src_off), _ll_array(dst_off), _ll_array(lens), st, int(sync), 0,
                                         self._stream()), "gather")

    def barrier(self):
        check_rc(self.lib.tb_barrier(self.comm, self._stream()), "barrier")

    def close(self):
        torch.cuda.synchronize(self.device)
        self.lib.tb_comm_destroy(self.comm)
        self.lib.tb_status_free(self._status_host)
