"""Causal self-attention over a packed qkv tensor [B, T, 3*dim], on the hand-written
tcgen05 kernels (tandem_b200/cuda/attention.cu): forward keeps only the output and one
log-sum-exp per row; backward recomputes the probabilities tile by tile in two kernels
(dQ, then dK and dV), deterministically and without scratch beyond one float per row.  Shapes the
kernels do not cover (T not a multiple of 128, head dim other than 64 / 128, non-bf16)
raise rather than fall back silently.  The reference calls torch's
scaled_dot_product_attention (tandem/model.py:43)."""

import ctypes
import functools

import torch

from ._lib import check_rc, lib, need_bf16, stream


@functools.cache
def _fns():
    L = lib()
    vp, i = ctypes.c_void_p, ctypes.c_int
    L.tb_attn_fwd.argtypes = [vp, vp, vp, i, i, i, i, vp]
    L.tb_attn_fwd.restype = i
    L.tb_attn_bwd.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i, vp]
    L.tb_attn_bwd.restype = i
    L.tb_attn_error.argtypes = []
    L.tb_attn_error.restype = i
    return L


class _CausalAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, heads):
        need_bf16(qkv)
        B, T, d3 = qkv.shape
        d = d3 // 3
        hd = d // heads
        if T % 128 or hd not in (64, 128):
            raise ValueError(f"causal_attention kernels need T % 128 == 0 and head dim 64 or 128 (got T={T}, head dim {hd})")
        qkv = qkv.contiguous()
        out = torch.empty(B, T, d, dtype=torch.bfloat16, device=qkv.device)
        lse = torch.empty(B, heads, T, dtype=torch.float32, device=qkv.device)
        check_rc(_fns().tb_attn_fwd(qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), B, T, heads, hd, stream(qkv)), "attention forward")
        ctx.save_for_backward(qkv, out, lse)
        ctx.heads = heads
        return out

    @staticmethod
    def backward(ctx, d_out):
        qkv, out, lse = ctx.saved_tensors
        B, T, d3 = qkv.shape
        d = d3 // 3
        heads = ctx.heads
        d_out = d_out.contiguous()
        dqkv = torch.empty_like(qkv)
        delta = torch.empty(B * heads * T, dtype=torch.float32, device=qkv.device)
        check_rc(_fns().tb_attn_bwd(qkv.data_ptr(), out.data_ptr(), d_out.data_ptr(), lse.data_ptr(), dqkv.data_ptr(), delta.data_ptr(),
                                    B, T, heads, d // heads, stream(qkv)), "attention backward")
        return dqkv, None


def causal_attention(qkv, heads):
    """Returns [B, T, dim]."""
    return _CausalAttention.apply(qkv, heads)


def attention_error():
    """True once any attention kernel gave up on a wait (results since then are invalid)."""
    return bool(_fns().tb_attn_error())
