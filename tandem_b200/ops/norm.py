"""LayerNorm on the fused kernels (tandem_b200/cuda/layers.cu): one pass forward
saving mean and 1/std per row; one pass backward producing dx plus per-block
partial sums of the weight and bias gradients, reduced in a fixed order."""

import torch

from ._lib import check_rc, lib, need_bf16, stream


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps):
        need_bf16(x, w, b)
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        M, D = x2.shape
        y = torch.empty_like(x2)
        mean = torch.empty(M, dtype=torch.float32, device=x.device)
        rstd = torch.empty(M, dtype=torch.float32, device=x.device)
        check_rc(lib().tb_layernorm_fwd(x2.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                        M, D, eps, stream(x)), "layernorm forward")
        ctx.save_for_backward(x2, w, mean, rstd)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, mean, rstd = ctx.saved_tensors
        M, D = x2.shape
        dy2 = dy.reshape(-1, D).contiguous()
        dx = torch.empty_like(x2)
        dw = torch.empty_like(w)
        db = torch.empty_like(w)
        blocks = lib().tb_layernorm_bwd_blocks(M)
        scratch = torch.empty(blocks * 2 * D, dtype=torch.float32, device=x2.device)
        check_rc(lib().tb_layernorm_bwd(dy2.data_ptr(), x2.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                        dw.data_ptr(), db.data_ptr(), scratch.data_ptr(), M, D, stream(x2)), "layernorm backward")
        return dx.view(dy.shape), dw, db, None


def layer_norm(x, weight, bias, eps=1e-5):
    return _LayerNorm.apply(x, weight, bias, eps)


class _ResidualLayerNorm(torch.autograd.Function):
    """(x, LayerNorm(x)): the input is handed through for the residual connection, so that backward receives
    both gradients of x -- the residual branch's and the normalised branch's -- and the LayerNorm backward kernel
    sums them in fp32 while it writes dx, instead of autograd adding them in a pass of its own."""

    @staticmethod
    def forward(ctx, x, w, b, eps):
        need_bf16(x, w, b)
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        M, D = x2.shape
        y = torch.empty_like(x2)
        mean = torch.empty(M, dtype=torch.float32, device=x.device)
        rstd = torch.empty(M, dtype=torch.float32, device=x.device)
        check_rc(lib().tb_layernorm_fwd(x2.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                        M, D, eps, stream(x)), "layernorm forward")
        ctx.save_for_backward(x2, w, mean, rstd)
        return x.view_as(x), y.view(x.shape)

    @staticmethod
    def backward(ctx, dres, dy):
        x2, w, mean, rstd = ctx.saved_tensors
        M, D = x2.shape
        if dy is None:
            return dres, None, None, None
        dy2 = dy.reshape(-1, D).contiguous()
        add = None if dres is None else dres.reshape(-1, D).contiguous()
        dx = torch.empty_like(x2)
        dw = torch.empty_like(w)
        db = torch.empty_like(w)
        blocks = lib().tb_layernorm_bwd_blocks(M)
        scratch = torch.empty(blocks * 2 * D, dtype=torch.float32, device=x2.device)
        check_rc(lib().tb_layernorm_bwd_add(dy2.data_ptr(), x2.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                            None if add is None else add.data_ptr(), dx.data_ptr(), dw.data_ptr(), db.data_ptr(),
                                            scratch.data_ptr(), M, D, stream(x2)), "layernorm backward")
        return dx.view(dy.shape), dw, db, None


def residual_layer_norm(x, weight, bias, eps=1e-5):
    """Returns (x, LayerNorm(x)); use the returned x for the residual connection."""
    return _ResidualLayerNorm.apply(x, weight, bias, eps)
