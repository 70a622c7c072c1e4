"""Token + position embedding in one gather kernel; backward scatters token
gradients with fp32 atomics and sums position gradients over the batch in a
fixed order (tandem_b200/cuda/layers.cu)."""

import torch

from ._lib import check_rc, lib, need_bf16, stream


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, tok, pos):
        need_bf16(tok, pos)
        B, T = idx.shape
        D = tok.shape[1]
        idx = idx.contiguous()
        out = torch.empty(B, T, D, dtype=torch.bfloat16, device=tok.device)
        check_rc(lib().tb_embed_fwd(idx.data_ptr(), tok.data_ptr(), pos.data_ptr(), out.data_ptr(), B * T, T, D, stream(tok)),
                 "embedding forward")
        ctx.save_for_backward(idx)
        ctx.shapes = (tok.shape, pos.shape)
        return out

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        (V, D), (S, _) = ctx.shapes
        B, T = idx.shape
        dy = dy.contiguous()
        dtok32 = torch.zeros(V, D, dtype=torch.float32, device=dy.device)
        dtok = torch.empty(V, D, dtype=torch.bfloat16, device=dy.device)
        dpos = torch.zeros(S, D, dtype=torch.bfloat16, device=dy.device)
        check_rc(lib().tb_embed_bwd(idx.data_ptr(), dy.data_ptr(), dtok32.data_ptr(), dtok.data_ptr(), dpos.data_ptr(), B, T, D, V,
                                    stream(dy)), "embedding backward")
        return None, dtok, dpos


def embedding(idx, tok, pos):
    return _Embedding.apply(idx, tok, pos)
