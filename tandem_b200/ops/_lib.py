"""ctypes signatures of the compute kernels in libtb200_cuda.so."""

import ctypes
import functools

import torch

from ..parallel.symm import check_rc, cuda_lib  # noqa: F401


@functools.cache
def lib():
    L = cuda_lib()
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    sig = {
        "tb_gemm_error": ([], i),
        "tb_gemm_last_error": ([], ctypes.c_char_p),
        "tb_gemm_force_tile": ([i], None),
        "tb_gemm_tma_store": ([i], None),
        "tb_gemm_gathered": ([vp, vp, i, i, i, i, i, i, vp, vp, vp, ctypes.POINTER(vp), ctypes.POINTER(ctypes.c_longlong),
                              ctypes.POINTER(ctypes.c_longlong), i, vp, ctypes.c_longlong, ctypes.c_longlong, vp, ctypes.c_uint, i, i, vp], i),
        "tb_gemm_bf16": ([vp, vp, vp, i, i, i, i, i, i, i, i, i, vp, vp, vp, i, vp, ctypes.c_longlong, vp], i),
        "tb_gemm_workspace_bytes": ([i, i, i], ctypes.c_longlong),
        "tb_gemm_plan": ([i, i, i, ctypes.POINTER(ctypes.c_int)], None),
        "tb_gemm_force_splits": ([i], None),
        "tb_layernorm_fwd": ([vp, vp, vp, vp, vp, vp, i, i, f, vp], i),
        "tb_layernorm_bwd_blocks": ([i], i),
        "tb_layernorm_bwd": ([vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, vp], i),
        "tb_layernorm_bwd_add": ([vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, vp], i),
        "tb_col_sum": ([vp, i, i, i, vp, vp, vp], i),
        "tb_xent_fwd": ([vp, vp, vp, vp, vp, i, i, i, vp], i),
        "tb_xent_bwd": ([vp, vp, vp, vp, i, i, i, i, vp], i),
        "tb_embed_fwd": ([vp, vp, vp, vp, i, i, i, vp], i),
        "tb_embed_bwd": ([vp, vp, vp, vp, vp, i, i, i, i, vp], i),
    }
    for name, (argtypes, restype) in sig.items():
        if not hasattr(L, name):
            continue
        fn = getattr(L, name)
        fn.argtypes, fn.restype = argtypes, restype
    return L


def stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def pad8(n):
    return (n + 7) // 8 * 8


def empty_padded(rows, cols, dtype, device):
    """A [rows, cols] view of [rows, pad8(cols)] storage: every row starts 16-byte aligned."""
    ld = pad8(cols)
    return torch.empty(rows, ld, dtype=dtype, device=device)[:, :cols]


def need_bf16(*tensors):
    for t in tensors:
        if t is not None and (not t.is_cuda or t.dtype != torch.bfloat16):
            raise TypeError("the sm_100a operators take bf16 CUDA tensors (cast the model with .bfloat16())")
