"""Softmax cross-entropy (mean over rows) on the fused kernels: forward reads the
logits once for the row maximum and once for the sum; backward overwrites the
logits buffer with (softmax - onehot) * grad / rows, so no second [rows, vocab]
tensor is ever allocated (tandem_b200/cuda/layers.cu)."""

import torch

from ._lib import check_rc, lib, need_bf16, stream


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        need_bf16(logits)
        rows, V = logits.shape
        if logits.stride(1) != 1:
            logits = logits.contiguous()
        ld = logits.stride(0) if rows > 1 else V
        targets = targets.contiguous()
        lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
        row_loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        loss = torch.empty((), dtype=torch.float32, device=logits.device)
        check_rc(lib().tb_xent_fwd(logits.data_ptr(), targets.data_ptr(), lse.data_ptr(), row_loss.data_ptr(), loss.data_ptr(),
                                   rows, V, ld, stream(logits)), "cross-entropy forward")
        ctx.save_for_backward(logits, targets, lse)
        ctx.ld = ld
        return loss

    @staticmethod
    def backward(ctx, grad):
        logits, targets, lse = ctx.saved_tensors
        rows, V = logits.shape
        scale = grad.detach().reshape(1).float().contiguous()
        # In place: the saved logits become their own gradient (they are not needed again).
        ld = ctx.ld
        width = ld if ld - V < 8 and _owns_padding(logits, ld) else V
        check_rc(lib().tb_xent_bwd(logits.data_ptr(), targets.data_ptr(), lse.data_ptr(), scale.data_ptr(), rows, V, ld, width,
                                   stream(logits)), "cross-entropy backward")
        return logits, None


def _owns_padding(logits, width):
    """True when the columns [V, width) of each row belong to this tensor's storage (a padded allocation)."""
    need = (logits.shape[0] - 1) * logits.stride(0) + width
    return logits.storage_offset() + need <= logits.untyped_storage().nbytes() // logits.element_size()


def cross_entropy(logits, targets):
    return _CrossEntropy.apply(logits, targets)
