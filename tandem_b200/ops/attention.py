"""Causal self-attention over a packed qkv tensor [B, T, 3*dim]."""

import torch
import torch.nn.functional as F


def causal_attention(qkv, heads):
    """Returns [B, T, dim].  Placeholder dispatch: the fused flash kernel from
    torch (a library call) until the hand-written sm_100a kernel lands here."""
    b, t, d3 = qkv.shape
    d = d3 // 3
    q, k, v = qkv.split(d, dim=2)
    q, k, v = (z.view(b, t, heads, d // heads).transpose(1, 2) for z in (q, k, v))
    y = F.scaled_dot_product_attention(q, k, v, is_causal=True)
    return y.transpose(1, 2).reshape(b, t, d)
