"""Linear layers on the tcgen05 GEMM (tandem_b200/cuda/gemm.cu).

`linear` and `mlp` are autograd functions whose forward and both backward
products (dX, dW) run on the same kernel with different operand layouts, and
whose element-wise work rides in the GEMM epilogues: bias add, exact GELU
(which also saves GELU's derivative at each pre-activation, so that backward
only multiplies by it), and the residual add that follows the projection.
The reference computes these with nn.Linear / F.gelu / `+` (tandem/model.py:36-58)."""

import os

import torch

from ._lib import check_rc, empty_padded, lib, need_bf16, pad8, stream

BIAS, GELU, RESIDUAL, DGELU, ACCUMULATE, OUT_F32 = 1, 2, 4, 8, 16, 32


def _rows(t):
    """(2-D view, leading dimension) of a tensor whose last dim is contiguous and rows evenly strided."""
    t2 = t.reshape(-1, t.shape[-1]) if t.dim() != 2 else t
    if t2.stride(1) != 1 or (t2.shape[0] > 1 and t2.stride(0) % 8) or t2.data_ptr() % 16:
        t2 = _repack(t2)
    return t2, (t2.stride(0) if t2.shape[0] > 1 else pad8(t2.shape[1]))


def _repack(t2):
    out = empty_padded(t2.shape[0], t2.shape[1], t2.dtype, t2.device)
    out.copy_(t2)
    return out


def gemm(a, b, M, N, K, lda, ldb, a_mn, b_mn, flags=0, bias=None, aux_in=None, aux_out=None, out=None, out_dtype=torch.bfloat16,
         workspace=None):
    """out[M, N] = op(a) . op(b) (+ epilogue).  Returns a [M, N] view with a 16-byte-aligned row stride.
    workspace: a uint8 tensor of at least lib().tb_gemm_workspace_bytes(M, N, K) bytes, for callers that launch on another stream
    than the one their memory belongs to (else it is allocated here)."""
    if out is None:
        out = empty_padded(M, N, out_dtype, a.device)
    ldc = out.stride(0) if M > 1 else pad8(N)
    if aux_in is not None and (aux_in.stride(0) if M > 1 else ldc) != ldc:
        raise ValueError("aux_in must share the output's row stride")
    if out.dtype == torch.float32:
        flags |= OUT_F32
    # Problems with too few output tiles for the SMs (weight gradients, small per-rank batches) are computed with the
    # reduction cut into parts inside the one kernel; it parks partial tiles in this workspace.
    need = lib().tb_gemm_workspace_bytes(M, N, K)
    if need and (workspace is None or workspace.numel() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=a.device)
    if not need:
        workspace = None
    rc = lib().tb_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, lda, ldb, ldc, int(a_mn), int(b_mn), flags,
                            bias.data_ptr() if bias is not None else None,
                            aux_in.data_ptr() if aux_in is not None else None,
                            aux_out.data_ptr() if aux_out is not None else None, 0,
                            workspace.data_ptr() if workspace is not None else None, need, stream(a))
    if rc in (-11, -12):
        raise RuntimeError(f"gemm: operand not addressable by TMA (M={M} N={N} K={K} lda={lda} ldb={ldb} a_mn={a_mn} b_mn={b_mn} "
                           f"a={a.data_ptr():#x} b={b.data_ptr():#x}): {lib().tb_gemm_last_error().decode()}")
    check_rc(rc, "gemm")
    return out


def _forward(x2, ldx, w, bias, flags, aux_in=None, aux_out=None):
    M, K = x2.shape
    N = w.shape[0]
    if bias is not None:
        flags |= BIAS
    return gemm(x2, w, M, N, K, ldx, w.stride(0), False, False, flags, bias, aux_in, aux_out)


def _grad_input(dy2, ldy, w, flags=0, aux_in=None):
    """dX[M, K] = dY[M, N] . W[N, K]   (reduction over N; W read as an MN-major operand)"""
    M, N = dy2.shape
    K = w.shape[1]
    return gemm(dy2, w, M, K, N, ldy, w.stride(0), False, True, flags, None, aux_in)


def _grad_weight(dy2, ldy, x2, ldx, dtype):
    """dW[N, K] = dY[M, N]^T . X[M, K]   (reduction over the M tokens; both operands MN-major)"""
    M, N = dy2.shape
    K = x2.shape[1]
    return gemm(dy2, x2, N, K, M, ldy, ldx, True, True, 0, out_dtype=dtype).contiguous()


def _grad_bias(dy2, ldy):
    M, N = dy2.shape
    out = torch.empty(N, dtype=torch.bfloat16, device=dy2.device)
    scratch = torch.empty(32 * N, dtype=torch.float32, device=dy2.device)
    check_rc(lib().tb_col_sum(dy2.data_ptr(), M, N, ldy, out.data_ptr(), scratch.data_ptr(), stream(dy2)), "col_sum")
    return out


# The two products of a layer's backward that share dY -- the weight (and bias) gradient and the input gradient --
# do not depend on each other.  With few tokens per rank neither fills the GPU (48-144 CTAs for 148 SMs), so the
# parameter gradients run on a second stream beside the input gradient; the streams fork and join inside one backward
# call, which a CUDA-graph capture records as two branches.  Everything the side stream touches is allocated on the
# caller's stream beforehand and outlives the join, so the caching allocator's per-stream pools never see a block
# used by a stream it does not know about.
# with more tokens each product fills the SMs by itself and the fork only adds two event waits (TANDEM_SIDE_TOKENS=0: never fork)
SIDE_BELOW_TOKENS = int(os.environ.get("TANDEM_SIDE_TOKENS", "4096"))
_side_streams = {}


def _parameter_grads_beside(dy2, ldy, x2, ldx, dtype, want_w, want_b):
    """(dW, dB, join): starts dW = dY^T . X and dB = column sums of dY on the side stream when the problem is small;
    join() makes the caller's stream wait for them (call it after queuing the input gradient)."""
    M, N = dy2.shape
    K = x2.shape[1]
    if not (want_w or want_b):
        return None, None, lambda: None
    if M >= SIDE_BELOW_TOKENS or not dy2.is_cuda:
        dw = _grad_weight(dy2, ldy, x2, ldx, dtype) if want_w else None
        db = _grad_bias(dy2, ldy) if want_b else None
        return dw, db, lambda: None
    dev = dy2.device
    main = torch.cuda.current_stream(dev)
    side = _side_streams.get(dev.index)
    if side is None:
        side = _side_streams[dev.index] = torch.cuda.Stream(dev)
    dw = db = scratch = workspace = None
    if want_w:
        if pad8(K) != K:  # a padded product needs a compaction copy afterwards: keep that case on one stream
            dw = _grad_weight(dy2, ldy, x2, ldx, dtype)
            want_w = False
        else:
            dw = torch.empty(N, K, dtype=dtype, device=dev)
            need = lib().tb_gemm_workspace_bytes(N, K, M)
            workspace = torch.empty(need, dtype=torch.uint8, device=dev) if need else None
    if want_b:
        db = torch.empty(N, dtype=torch.bfloat16, device=dev)
        scratch = torch.empty(32 * N, dtype=torch.float32, device=dev)
    side.wait_stream(main)
    with torch.cuda.stream(side):
        if want_w:
            gemm(dy2, x2, N, K, M, ldy, ldx, True, True, 0, out=dw, workspace=workspace)
        if want_b:
            check_rc(lib().tb_col_sum(dy2.data_ptr(), M, N, ldy, db.data_ptr(), scratch.data_ptr(), side.cuda_stream), "col_sum")
    keep = (scratch, workspace)  # released by the caller's frame, after the join

    def join():
        main.wait_stream(side)
        return keep

    return dw, db, join


# Weights whose all-gather the next forward GEMM performs itself: data_ptr of the weight's place in the local flat
# buffer -> (GatheredLinear, event to wait for afterwards or None).  ZeRO-3 fills it when it starts a unit's gather.
GATHERED = {}


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, residual):
        need_bf16(x, w, bias, residual)
        x2, ldx = _rows(x)
        fused = GATHERED.pop(w.data_ptr(), None) if GATHERED and residual is None else None
        if fused is not None:
            op, after = fused
            y = op(x2, None if op.tail else bias)
            if after is not None:  # the rest of the unit's parameters, pulled meanwhile on the communication stream
                torch.cuda.current_stream(x.device).wait_event(after)
            ctx.save_for_backward(x2, w)
            ctx.ldx, ctx.has_bias, ctx.has_res = ldx, bias is not None, False
            ctx.in_shape = x.shape
            return y.view(*x.shape[:-1], w.shape[0])
        res2 = None
        if residual is not None:
            res2 = residual.reshape(-1, residual.shape[-1])
            if pad8(w.shape[0]) != w.shape[0] or not res2.is_contiguous():
                raise ValueError("a fused residual needs a contiguous tensor whose width is a multiple of 8")
        y = _forward(x2, ldx, w, bias, RESIDUAL if res2 is not None else 0, res2)
        ctx.save_for_backward(x2, w)
        ctx.ldx, ctx.has_bias, ctx.has_res = ldx, bias is not None, residual is not None
        ctx.in_shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0]) if y.is_contiguous() else y.unflatten(0, x.shape[:-1])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2, ldy = _rows(dy)
        dx = dres = None
        dw, db, join = _parameter_grads_beside(dy2, ldy, x2, ctx.ldx, w.dtype, ctx.needs_input_grad[1],
                                                ctx.has_bias and ctx.needs_input_grad[2])
        if ctx.needs_input_grad[0]:
            dx = _grad_input(dy2, ldy, w)
            dx = dx.view(ctx.in_shape) if dx.is_contiguous() else dx.unflatten(0, ctx.in_shape[:-1])
        join()
        if ctx.has_res and ctx.needs_input_grad[3]:
            dres = dy
        return dx, dw, db, dres


class _MLP(torch.autograd.Function):
    """out = residual + W2 . gelu(W1 . x + b1) + b2, with both element-wise stages in GEMM epilogues."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual):
        need_bf16(x, w1, b1, w2, b2, residual)
        if residual is None:
            raise ValueError("ops.mlp adds its input stream: pass the residual tensor")
        if w1.shape[0] % 8 or w2.shape[0] % 8:
            raise ValueError("ops.mlp needs hidden and output widths that are multiples of 8 (16-byte rows)")
        x2, ldx = _rows(x)
        M = x2.shape[0]
        slope = empty_padded(M, w1.shape[0], torch.bfloat16, x.device)  # gelu'(W1 . x + b1), written by the same epilogue
        h = _forward(x2, ldx, w1, b1, GELU, None, slope)
        res2 = residual.reshape(-1, residual.shape[-1])
        y = _forward(h, h.stride(0), w2, b2, RESIDUAL, res2)
        ctx.save_for_backward(x2, w1, w2, slope, h)
        ctx.ldx, ctx.in_shape = ldx, x.shape
        return y.view(*x.shape[:-1], w2.shape[0]) if y.is_contiguous() else y.unflatten(0, x.shape[:-1])

    @staticmethod
    def backward(ctx, dy):
        x2, w1, w2, slope, h = ctx.saved_tensors
        need = ctx.needs_input_grad
        dy2, ldy = _rows(dy)
        dw2, db2, join2 = _parameter_grads_beside(dy2, ldy, h, h.stride(0), w2.dtype, need[3], need[4])
        dpre = _grad_input(dy2, ldy, w2, DGELU, slope)  # (dY . W2) * gelu'(pre)
        join2()
        ldp = dpre.stride(0)
        dw1, db1, join1 = _parameter_grads_beside(dpre, ldp, x2, ctx.ldx, w1.dtype, need[1], need[2])
        dx = None
        if need[0]:
            dx = _grad_input(dpre, ldp, w1)
            dx = dx.view(ctx.in_shape) if dx.is_contiguous() else dx.unflatten(0, ctx.in_shape[:-1])
        join1()
        return dx, dw1, db1, dw2, db2, (dy if need[5] else None)


def linear(x, weight, bias=None, gelu=False, residual=None):
    if gelu:
        raise ValueError("use ops.mlp for the GELU MLP (its backward fuses GELU's derivative into a GEMM epilogue)")
    return _Linear.apply(x, weight, bias, residual)


def mlp(x, w1, b1, w2, b2, residual):
    return _MLP.apply(x, w1, b1, w2, b2, residual)


def gemm_error():
    """True once any GEMM gave up on a wait (results since then are invalid)."""
    return bool(lib().tb_gemm_error())


class GatheredLinear:
    """y = x . W^T (+ bias) where W is one parameter inside a sharded flat buffer (a ZeRO-3 unit): the
    all-gather of W is fused into the GEMM.  Extra warps of the GEMM kernel pull W's bytes from the owners'
    shards (peer pointers into symmetric memory) into `full`, this rank's copy of the flat buffer, and the
    kernel's TMA producer consumes each weight panel as soon as its chunks have landed.

    shard_ptrs[q]: address (in this process) of rank q's shard; shard q holds flat elements
    [offsets[q], offsets[q+1]).  w_offset: W's first element in the flat buffer; W is [N, K] row-major.
    Forward only (the backward of a ZeRO-3 unit re-gathers with the ordinary pull)."""

    CHUNK = 32 << 10

    def __init__(self, shard_ptrs, offsets, rank, full, w_offset, N, K, bias_follows=False):
        """bias_follows: the layer's bias (N elements) lies right behind W in the flat buffer (the parameter order of
        nn.Linear) and is fetched and applied by the same kernel."""
        esz = 2
        self.tail = N * esz if bias_follows else 0
        self.ptrs, self.rank, self.full = list(shard_ptrs), rank, full
        self.lo = [o * esz for o in offsets[:-1]]
        self.hi = [o * esz for o in offsets[1:]]
        self.w_off, self.N, self.K = w_offset * esz, N, K
        if self.w_off % 16 or K % 8:
            raise ValueError("the gathered weight must start 16-byte aligned in the flat buffer and K must be a multiple of 8")
        nchunks = (N * K * esz + self.tail + self.CHUNK - 1) // self.CHUNK
        self.ready = torch.zeros(nchunks, dtype=torch.int32, device=full.device)
        self.epoch = 0
        # visit first the panel fed by this rank's own shard (it arrives without crossing NVLink)
        own = max(self.lo[rank], self.w_off) - self.w_off
        own = own if self.lo[rank] < self.w_off + N * K * esz and self.hi[rank] > self.w_off else 0
        self.n_start = (own // (K * esz)) // 256

    def __call__(self, x, bias=None):
        import ctypes

        need_bf16(x, bias)
        x2, ldx = _rows(x)
        M = x2.shape[0]
        out = empty_padded(M, self.N, torch.bfloat16, x.device)
        self.epoch += 1
        n = len(self.ptrs)
        ptrs = (ctypes.c_void_p * n)(*self.ptrs)
        lo = (ctypes.c_longlong * n)(*self.lo)
        hi = (ctypes.c_longlong * n)(*self.hi)
        if self.tail:
            bias_ptr = self.full.data_ptr() + self.w_off + self.N * self.K * 2
        else:
            bias_ptr = bias.data_ptr() if bias is not None else None
        check_rc(lib().tb_gemm_gathered(x2.data_ptr(), out.data_ptr(), M, self.N, self.K, ldx, out.stride(0), BIAS if bias_ptr else 0,
                                        bias_ptr, None, None, ptrs, lo, hi, n, self.full.data_ptr(), self.w_off, self.tail,
                                        self.ready.data_ptr(), self.epoch, self.CHUNK, self.n_start, stream(x)), "gathered gemm")
        return out.view(*x.shape[:-1], self.N)
