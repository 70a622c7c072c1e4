"""Hand-written sm_100a operators and their autograd wrappers.

Each function here launches kernels from libtb200_cuda.so (tandem_b200/cuda);
on CPU tensors the few that strategies call unconditionally (`pack_into`) fall
back to torch ops.  A CUDA tensor with the library missing is an error, never a
silent fallback."""

import torch


def pack_into(flat, pairs):
    """Copies each `src` into its `view` of the bucket `flat`.  `pairs` is
    [(view, src)].  One multi-tensor kernel per call on a GPU (the reference
    issues one copy per parameter: tandem/ddp.py:92-94)."""
    if not pairs:
        return
    if flat.is_cuda:
        from .elementwise import multi_copy

        multi_copy(flat, pairs)
        return
    for view, src in pairs:
        view.copy_(src)


def fused_adamw(param, grad, exp_avg, exp_avg_sq, scalars, decay, shadow=None):
    from .elementwise import adamw_step

    adamw_step(param, grad, exp_avg, exp_avg_sq, scalars, decay, shadow)


def linear(x, weight, bias=None, gelu=False, residual=None):
    from .gemm import linear as f

    return f(x, weight, bias, gelu, residual)


def mlp(x, w1, b1, w2, b2, residual):
    from .gemm import mlp as f

    return f(x, w1, b1, w2, b2, residual)


def layer_norm(x, weight, bias, eps=1e-5):
    from .norm import layer_norm as f

    return f(x, weight, bias, eps)


def residual_layer_norm(x, weight, bias, eps=1e-5):
    from .norm import residual_layer_norm as f

    return f(x, weight, bias, eps)


def causal_attention(qkv, heads):
    from .attention import causal_attention as f

    return f(qkv, heads)


def embedding(idx, tok, pos):
    from .embed import embedding as f

    return f(idx, tok, pos)


def cross_entropy(logits, targets):
    from .xent import cross_entropy as f

    return f(logits, targets)
