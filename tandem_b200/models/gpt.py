"""Decoder-only GPT: the model every strategy trains.

Module tree, parameter names and unit boundaries follow the reference's
tandem/model.py:14-120 so that state dicts are interchangeable:
embed.{tok,pos}.weight, blocks.{i}.{ln1,attn.qkv,attn.proj,ln2,fc,out}.*,
head.{ln,lm}.*; units() = [embed, *blocks, head]; the LM head is untied.
Modules are created, and their weights drawn, in that same order, so a seed
gives the same initial weights as the reference.

Every module has two forward paths over the same parameters, chosen by
Config.kernels and by where the input lives:
  "torch"  torch.nn.functional ops (cuBLAS / SDPA): the oracle, and the path the
           deterministic bit-for-bit checks use; also taken for CPU tensors.
  "b200"   the hand-written sm_100a kernels in tandem_b200.ops (tcgen05 GEMM with
           fused bias / GELU / residual epilogues, LayerNorm, causal attention,
           fused softmax-cross-entropy).
"""

import math
import os
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

# name -> fields that differ from the defaults (parameter counts with the default vocabulary of 256 unless given)
PRESETS = {
    "tiny": {},
    "verify": {"dim": 256},                                                       # 3.3M
    "small": {"seq": 256, "layers": 6, "heads": 6, "dim": 384},                    # 11M
    "medium": {"seq": 512, "layers": 12, "heads": 12, "dim": 768},                 # 85.8M
    "large": {"seq": 512, "layers": 24, "heads": 16, "dim": 1024},                 # 302M
    "pp24": {"vocab": 50304, "seq": 1024, "layers": 24, "heads": 16, "dim": 1024},  # 406M, the pipeline configuration
    "1.3b": {"vocab": 50304, "seq": 2048, "layers": 24, "heads": 16, "dim": 2048},  # 1.42B (untied head)
}


@dataclass
class Config:
    vocab: int = 256
    seq: int = 128
    layers: int = 4
    heads: int = 4
    dim: int = 128
    kernels: str = "torch"  # or "b200"

    @classmethod
    def preset(cls, name):
        return cls(**PRESETS[name])


# Pre-LayerNorm blocks sum the residual branch's gradient inside the LayerNorm backward kernel instead of leaving
# that addition to autograd (one element-wise kernel less per LayerNorm and one pass less over the activations).
# TANDEM_RESIDUAL_LN=0 switches back to autograd's addition.
RESIDUAL_LN = os.environ.get("TANDEM_RESIDUAL_LN", "1") != "0"


def _ops():
    from .. import ops

    return ops


def _on_kernels(module, tensor):
    return module.kernels == "b200" and tensor.is_cuda


def _norm(ops, ln, x):
    return ops.layer_norm(x, ln.weight, ln.bias, ln.eps)


class Attention(nn.Module):
    """Fused qkv projection, causal multi-head attention, output projection (+ the residual when given)."""

    def __init__(self, c):
        super().__init__()
        width = c.dim
        self.heads = c.heads
        self.kernels = c.kernels
        self.qkv = nn.Linear(width, 3 * width)
        self.proj = nn.Linear(width, width)

    def forward(self, x, residual=None):
        if _on_kernels(self, x):
            ops = _ops()
            qkv = ops.linear(x, self.qkv.weight, self.qkv.bias)
            y = ops.causal_attention(qkv, self.heads)
            return ops.linear(y, self.proj.weight, self.proj.bias, residual=residual)
        batch, steps, width = x.shape
        per_head = (batch, steps, self.heads, width // self.heads)
        q, k, v = (part.view(per_head).transpose(1, 2) for part in self.qkv(x).split(width, dim=2))
        mixed = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        y = self.proj(mixed.transpose(1, 2).reshape(batch, steps, width))
        return y if residual is None else residual + y


class Block(nn.Module):
    """x + attn(ln1(x)), then x + out(gelu(fc(ln2(x))))."""

    def __init__(self, c):
        super().__init__()
        width = c.dim
        self.kernels = c.kernels
        self.ln1 = nn.LayerNorm(width)
        self.attn = Attention(c)
        self.ln2 = nn.LayerNorm(width)
        self.fc = nn.Linear(width, 4 * width)
        self.out = nn.Linear(4 * width, width)

    def _mlp_weights(self):
        return self.fc.weight, self.fc.bias, self.out.weight, self.out.bias

    def forward(self, x):
        if not _on_kernels(self, x):
            x = x + self.attn(self.ln1(x))
            hidden = F.gelu(self.fc(self.ln2(x)))
            return x + self.out(hidden)
        ops = _ops()
        if RESIDUAL_LN:
            # residual_layer_norm hands x through, so both gradients of x meet in the LayerNorm backward kernel
            x, normed = ops.residual_layer_norm(x, self.ln1.weight, self.ln1.bias, self.ln1.eps)
            x = self.attn(normed, residual=x)
            x, normed = ops.residual_layer_norm(x, self.ln2.weight, self.ln2.bias, self.ln2.eps)
            return ops.mlp(normed, *self._mlp_weights(), residual=x)
        x = self.attn(_norm(ops, self.ln1, x), residual=x)
        return ops.mlp(_norm(ops, self.ln2, x), *self._mlp_weights(), residual=x)


class Embed(nn.Module):
    """Token embedding plus a learned position embedding."""

    def __init__(self, c):
        super().__init__()
        self.kernels = c.kernels
        self.tok = nn.Embedding(c.vocab, c.dim)
        self.pos = nn.Embedding(c.seq, c.dim)

    def forward(self, idx):
        if _on_kernels(self, idx):
            return _ops().embedding(idx, self.tok.weight, self.pos.weight)
        positions = torch.arange(idx.shape[1], device=idx.device)
        return self.tok(idx) + self.pos(positions)


class Head(nn.Module):
    """Final LayerNorm and the (untied, bias-free) projection to the vocabulary."""

    def __init__(self, c):
        super().__init__()
        self.kernels = c.kernels
        self.ln = nn.LayerNorm(c.dim)
        self.lm = nn.Linear(c.dim, c.vocab, bias=False)

    def forward(self, x):
        if _on_kernels(self, x):
            ops = _ops()
            return ops.linear(_norm(ops, self.ln, x), self.lm.weight, None)
        return self.lm(self.ln(x))


def _draw_weights(module):
    """N(0, 0.02) weights, zero biases (LayerNorms keep their ones and zeros)."""
    if isinstance(module, (nn.Linear, nn.Embedding)):
        nn.init.normal_(module.weight, std=0.02)
        if getattr(module, "bias", None) is not None:
            nn.init.zeros_(module.bias)


class GPT(nn.Module):
    def __init__(self, c):
        super().__init__()
        if c.dim % c.heads:
            raise ValueError("dim must be a multiple of heads")
        self.config = c
        self.embed = Embed(c)
        self.blocks = nn.ModuleList([Block(c) for _ in range(c.layers)])
        self.head = Head(c)
        self.apply(_draw_weights)
        shrunk = 0.02 / math.sqrt(2 * c.layers)  # the projections that feed the residual stream start smaller (GPT-2)
        for block in self.blocks:
            nn.init.normal_(block.attn.proj.weight, std=shrunk)
            nn.init.normal_(block.out.weight, std=shrunk)

    def units(self):
        """The model as the sequence of modules that ZeRO-3 shards one at a time
        and pipeline parallelism deals out to stages."""
        return [self.embed] + list(self.blocks) + [self.head]

    def forward(self, idx, targets=None):
        x = self.embed(idx)
        for block in self.blocks:
            x = block(x)
        logits = self.head(x)
        return logits if targets is None else loss_fn(logits, targets, self.config.kernels)


def loss_fn(logits, targets, kernels="torch"):
    """Mean cross-entropy over every position."""
    flat_logits = logits.reshape(-1, logits.shape[-1])
    flat_targets = targets.reshape(-1)
    if kernels == "b200" and logits.is_cuda:
        return _ops().cross_entropy(flat_logits, flat_targets)
    return F.cross_entropy(flat_logits.float(), flat_targets)


def count_params(model):
    return sum(p.numel() for p in model.parameters())
