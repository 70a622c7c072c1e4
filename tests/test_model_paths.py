"""The GPT's two forward paths are wired the same way: with the kernel library replaced by plain torch functions
of the same signatures, the kernels="b200" path must give exactly the losses, logits and gradients of the
kernels="torch" path.  (What the real kernels compute is checked on a GPU; this runs anywhere and catches a
swapped argument, a forgotten residual or a bias that is not passed.)"""

import types

import pytest
import torch
import torch.nn.functional as F

import tandem_b200.models.gpt as gpt


def stand_in_ops():
    def linear(x, weight, bias=None, gelu=False, residual=None):
        y = F.linear(x, weight, bias)
        return y if residual is None else residual + y

    def layer_norm(x, weight, bias, eps=1e-5):
        return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)

    def residual_layer_norm(x, weight, bias, eps=1e-5):
        return x, layer_norm(x, weight, bias, eps)

    def causal_attention(qkv, heads):
        batch, steps, three_d = qkv.shape
        d = three_d // 3
        q, k, v = (part.view(batch, steps, heads, d // heads).transpose(1, 2) for part in qkv.split(d, dim=2))
        return F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(batch, steps, d)

    def mlp(x, w1, b1, w2, b2, residual):
        return residual + F.linear(F.gelu(F.linear(x, w1, b1)), w2, b2)

    def embedding(idx, tok, pos):
        return tok[idx] + pos[torch.arange(idx.shape[1])]

    def cross_entropy(logits, targets):
        return F.cross_entropy(logits.float(), targets)

    return types.SimpleNamespace(linear=linear, layer_norm=layer_norm, residual_layer_norm=residual_layer_norm,
                                 causal_attention=causal_attention, mlp=mlp, embedding=embedding, cross_entropy=cross_entropy)


@pytest.mark.parametrize("residual_ln", [False, True])
def test_kernel_path_is_wired_like_the_torch_path(monkeypatch, residual_ln):
    monkeypatch.setattr(gpt, "_ops", stand_in_ops)
    monkeypatch.setattr(gpt, "_on_kernels", lambda module, tensor: module.kernels == "b200")  # also for CPU tensors
    monkeypatch.setattr(gpt, "RESIDUAL_LN", residual_ln)
    models = []
    for kernels in ("torch", "b200"):
        torch.manual_seed(0)
        models.append(gpt.GPT(gpt.Config(seq=32, layers=2, heads=2, dim=32, kernels=kernels)))
    oracle, wired = models
    tokens, targets = torch.randint(0, 256, (2, 32)), torch.randint(0, 256, (2, 32))
    assert torch.equal(oracle(tokens), wired(tokens))
    losses = [m(tokens, targets) for m in models]
    assert losses[0].item() == losses[1].item()
    for loss in losses:
        loss.backward()
    for (name, p), q in zip(oracle.named_parameters(), wired.parameters()):
        assert torch.equal(p.grad, q.grad), name
