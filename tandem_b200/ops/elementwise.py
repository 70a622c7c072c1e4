"""Launchers for the fused element-wise kernels (tandem_b200/cuda/elementwise.cu)."""

import ctypes

import torch

from ..parallel.symm import _ll_array, _ptr_array, check_rc, cuda_lib


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def multi_copy(flat, pairs):
    """dst.copy_(src) for every (dst, src) pair in one launch per 48 tensors.
    Pairs whose dtypes differ or that are not contiguous fall back to copy_."""
    srcs, dsts, sizes = [], [], []
    for dst, src in pairs:
        if src.dtype != dst.dtype or not src.is_contiguous() or not dst.is_contiguous() or src.device != dst.device:
            dst.copy_(src)
            continue
        srcs.append(src.data_ptr())
        dsts.append(dst.data_ptr())
        sizes.append(src.numel() * src.element_size())
    if srcs:
        check_rc(cuda_lib().tb_multi_copy(_ptr_array(srcs), _ptr_array(dsts), _ll_array(sizes), len(srcs), _stream(flat)),
                 "multi_copy")


def adamw_step(param, grad, exp_avg, exp_avg_sq, scalars, decay, shadow=None, grad_scale=1.0):
    """One fused AdamW step on fp32 {param, exp_avg, exp_avg_sq}; grad is fp32 or
    bf16; `shadow` (bf16) receives a copy of the new parameter."""
    if not (param.is_cuda and param.dtype == torch.float32 and param.is_contiguous()):
        raise ValueError("the fused AdamW kernel needs contiguous fp32 CUDA parameters")
    if grad.dtype not in (torch.float32, torch.bfloat16) or grad.numel() != param.numel():
        raise ValueError("gradient must be fp32 or bf16 and match the parameter")
    if shadow is not None and (shadow.dtype != torch.bfloat16 or shadow.numel() != param.numel()):
        raise ValueError("shadow must be a bf16 tensor of the parameter's size")
    sc = (ctypes.c_float * 7)(*scalars)
    check_rc(cuda_lib().tb_adamw(param.data_ptr(), grad.contiguous().data_ptr(), int(grad.dtype == torch.bfloat16),
                                 exp_avg.data_ptr(), exp_avg_sq.data_ptr(), shadow.data_ptr() if shadow is not None else None,
                                 param.numel(), sc, int(decay), float(grad_scale), _stream(param)), "adamw")


def adam_prepare(step_counter, hyper, scalars):
    """step_counter (1 double on the device) += 1; `scalars` (8 floats on the device) <- that step's constants."""
    lr, (b1, b2), eps, wd = hyper
    check_rc(cuda_lib().tb_adam_prepare(step_counter.data_ptr(), lr, b1, b2, eps, wd, scalars.data_ptr(), _stream(scalars)),
             "adam_prepare")


def adamw_step_dev(param, grad, exp_avg, exp_avg_sq, scalars, shadow=None):
    """adamw_step with the step's constants read from device memory (safe inside a CUDA graph)."""
    check_rc(cuda_lib().tb_adamw_dev(param.data_ptr(), grad.data_ptr(), int(grad.dtype == torch.bfloat16), exp_avg.data_ptr(),
                                     exp_avg_sq.data_ptr(), shadow.data_ptr() if shadow is not None else None, param.numel(),
                                     scalars.data_ptr(), _stream(param)), "adamw")
