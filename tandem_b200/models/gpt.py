"""Decoder-only GPT: the model every strategy trains.

Module tree, parameter names and unit boundaries follow the reference's
tandem/model.py:14-120 so that state dicts are interchangeable:
embed.{tok,pos}.weight, blocks.{i}.{ln1,attn.qkv,attn.proj,ln2,fc,out}.*,
head.{ln,lm}.*; units() = [embed, *blocks, head]; the LM head is untied.

Two compute paths share those parameters:
  kernels="torch"  torch.nn.functional ops (cuBLAS / SDPA); the oracle and the
                   path the deterministic bit-for-bit checks use.
  kernels="b200"   the hand-written sm_100a kernels in tandem_b200.ops
                   (tcgen05 GEMM with fused bias / GELU / residual epilogues,
                   fused LayerNorm, causal attention, fused softmax-cross-entropy).
"""

import math
import os
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class Config:
    vocab: int = 256
    seq: int = 128
    layers: int = 4
    heads: int = 4
    dim: int = 128
    kernels: str = "torch"  # or "b200"

    @staticmethod
    def preset(name):
        presets = {
            "tiny": dict(),
            "verify": dict(seq=128, layers=4, heads=4, dim=256),  # 3.3M with vocab 256
            "small": dict(seq=256, layers=6, heads=6, dim=384),  # 11M
            "medium": dict(seq=512, layers=12, heads=12, dim=768),  # 85.8M
            "large": dict(seq=512, layers=24, heads=16, dim=1024),  # 302M
            "pp24": dict(vocab=50304, seq=1024, layers=24, heads=16, dim=1024),  # 406M, pipeline config
            "1.3b": dict(vocab=50304, seq=2048, layers=24, heads=16, dim=2048),  # 1.42B (untied head)
        }
        return Config(**presets[name])


# Pre-LayerNorm blocks sum the residual branch's gradient inside the LayerNorm backward kernel (TANDEM_RESIDUAL_LN=0:
# leave that addition to autograd).
RESIDUAL_LN = os.environ.get("TANDEM_RESIDUAL_LN", "0") != "0"


def _b200():
    from .. import ops

    return ops


class Attention(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.heads, self.kernels = c.heads, c.kernels
        self.qkv = nn.Linear(c.dim, 3 * c.dim)
        self.proj = nn.Linear(c.dim, c.dim)

    def forward(self, x, residual=None):
        b, t, d = x.shape
        if self.kernels == "b200" and x.is_cuda:
            ops = _b200()
            qkv = ops.linear(x, self.qkv.weight, self.qkv.bias)
            y = ops.causal_attention(qkv, self.heads)
            return ops.linear(y, self.proj.weight, self.proj.bias, residual=residual)
        q, k, v = self.qkv(x).split(d, dim=2)
        q, k, v = (z.view(b, t, self.heads, d // self.heads).transpose(1, 2) for z in (q, k, v))
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        y = self.proj(y.transpose(1, 2).reshape(b, t, d))
        return y if residual is None else residual + y


class Block(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.kernels = c.kernels
        self.ln1 = nn.LayerNorm(c.dim)
        self.attn = Attention(c)
        self.ln2 = nn.LayerNorm(c.dim)
        self.fc = nn.Linear(c.dim, 4 * c.dim)
        self.out = nn.Linear(4 * c.dim, c.dim)

    def forward(self, x):
        if self.kernels == "b200" and x.is_cuda:
            ops = _b200()
            if not RESIDUAL_LN:
                x = self.attn(ops.layer_norm(x, self.ln1.weight, self.ln1.bias, self.ln1.eps), residual=x)
                return ops.mlp(ops.layer_norm(x, self.ln2.weight, self.ln2.bias, self.ln2.eps), self.fc.weight, self.fc.bias,
                               self.out.weight, self.out.bias, residual=x)
            # residual_layer_norm hands x through, so both gradients of x meet in the LayerNorm backward kernel
            x, n = ops.residual_layer_norm(x, self.ln1.weight, self.ln1.bias, self.ln1.eps)
            x = self.attn(n, residual=x)
            x, n = ops.residual_layer_norm(x, self.ln2.weight, self.ln2.bias, self.ln2.eps)
            return ops.mlp(n, self.fc.weight, self.fc.bias, self.out.weight, self.out.bias, residual=x)
        x = x + self.attn(self.ln1(x))
        return x + self.out(F.gelu(self.fc(self.ln2(x))))


class Embed(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.kernels = c.kernels
        self.tok = nn.Embedding(c.vocab, c.dim)
        self.pos = nn.Embedding(c.seq, c.dim)

    def forward(self, idx):
        if self.kernels == "b200" and idx.is_cuda:
            return _b200().embedding(idx, self.tok.weight, self.pos.weight)
        return self.tok(idx) + self.pos(torch.arange(idx.shape[1], device=idx.device))


class Head(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.kernels = c.kernels
        self.ln = nn.LayerNorm(c.dim)
        self.lm = nn.Linear(c.dim, c.vocab, bias=False)

    def forward(self, x):
        if self.kernels == "b200" and x.is_cuda:
            ops = _b200()
            return ops.linear(ops.layer_norm(x, self.ln.weight, self.ln.bias, self.ln.eps), self.lm.weight, None)
        return self.lm(self.ln(x))


class GPT(nn.Module):
    def __init__(self, c):
        super().__init__()
        if c.dim % c.heads:
            raise ValueError("dim must be a multiple of heads")
        self.config = c
        self.embed = Embed(c)
        self.blocks = nn.ModuleList(Block(c) for _ in range(c.layers))
        self.head = Head(c)
        self.apply(self._init)
        for b in self.blocks:  # residual projections start smaller, as in GPT-2
            for lin in (b.attn.proj, b.out):
                nn.init.normal_(lin.weight, std=0.02 / math.sqrt(2 * c.layers))

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
        if isinstance(m, nn.Linear) and m.bias is not None:
            nn.init.zeros_(m.bias)

    def units(self):
        """The model as the sequence of modules that ZeRO-3 shards one at a time
        and pipeline parallelism deals out to stages."""
        return [self.embed, *self.blocks, self.head]

    def forward(self, idx, targets=None):
        x = self.embed(idx)
        for b in self.blocks:
            x = b(x)
        logits = self.head(x)
        if targets is None:
            return logits
        return loss_fn(logits, targets, self.config.kernels)


def loss_fn(logits, targets, kernels="torch"):
    if kernels == "b200" and logits.is_cuda:
        return _b200().cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1))
    return F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), targets.reshape(-1))


def count_params(model):
    return sum(p.numel() for p in model.parameters())
