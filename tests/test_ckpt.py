"""Checkpoint / resume: train k steps, save, keep training -> A; in fresh ranks load
the file and train the same further steps -> B; A and B must be bit-identical, for
every strategy, and a checkpoint written by one strategy must load into another."""

import os
import tempfile

import pytest
import torch

from tandem_b200 import ckpt, launch
from tandem_b200.data import synthetic
from tandem_b200.ddp import DDP
from tandem_b200.model import GPT, Config
from tandem_b200.optim import ShardedAdamW
from tandem_b200.zero import FSDP, ZeRO

CFG = Config(seq=32, layers=2, heads=2, dim=32)


def build(g, strategy, dtype=torch.float32):
    torch.manual_seed(0)
    model = GPT(CFG).to(dtype)
    if strategy == "ddp":
        w = DDP(model, g, bucket_bytes=32 << 10)
        opt = torch.optim.AdamW(model.parameters(), lr=3e-3, weight_decay=0.1, foreach=False)
        return w, opt, lambda: (opt.step(), opt.zero_grad())
    if strategy == "ddp-sharded-adamw":
        from tandem_b200.ddp import ShardedBucketAdamW

        w = DDP(model, g, bucket_bytes=32 << 10, rebuild=False)
        opt = ShardedBucketAdamW(w, lr=3e-3, weight_decay=0.1)
        return w, opt, lambda: (opt.step(), opt.zero_grad())
    if strategy in ("ddp-bucket-adamw", "ddp-bucket-adamw-during-backward"):
        from tandem_b200.ddp import BucketAdamW

        w = DDP(model, g, bucket_bytes=32 << 10, rebuild=False)
        opt = BucketAdamW(w, lr=3e-3, weight_decay=0.1, during_backward=strategy.endswith("during-backward"))
        return w, opt, lambda: (opt.step(), opt.zero_grad())
    opt = ShardedAdamW(lr=3e-3, weight_decay=0.1)
    w = ZeRO(model, g, int(strategy[-1]), opt, 8 << 10) if strategy != "zero3" else FSDP(model, g, opt)
    return w, opt, lambda: (w.step(), w.zero_grad())


def steps(g, w, finish, first, count):
    text = synthetic(20_000)
    losses = []
    for step in range(first, first + count):
        x, y = text.batch(step, 8, CFG.seq, rank=g.rank, world=g.size)
        loss = w(x, y)
        loss.backward()
        finish()
        losses.append(loss.item())
    return losses


def weights(w):
    sd = ckpt.full_state_dict(w)
    return torch.cat([sd[k].reshape(-1) for k in sorted(sd)])


def run_and_save(g, strategy, path, dtype=torch.float32):
    w, opt, finish = build(g, strategy, dtype)
    steps(g, w, finish, 0, 3)
    ckpt.save(path, w, opt, extra={"next_step": 3})
    more = steps(g, w, finish, 3, 3)
    return more, weights(w)


def resume(g, strategy, path, dtype=torch.float32, stale_steps=0):
    w, opt, finish = build(g, strategy, dtype)
    if stale_steps:  # the optimizer has already stepped (and built its own master weights) before the load
        steps(g, w, finish, 100, stale_steps)
    extra = ckpt.load(path, w, opt)
    more = steps(g, w, finish, extra["next_step"], 3)
    return more, weights(w)


@pytest.mark.parametrize("strategy", ["ddp", "ddp-sharded-adamw", "ddp-bucket-adamw", "ddp-bucket-adamw-during-backward", "zero1", "zero2", "zero3"])
def test_resume_is_bit_identical(strategy):
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "ck.pt")
        a = launch(run_and_save, 2, strategy, path)
        b = launch(resume, 2, strategy, path)
        blob = torch.load(path, weights_only=False)
    assert a[0][0] == b[0][0] and a[1][0] == b[1][0]
    assert torch.equal(a[0][1], b[0][1])
    keys = set(blob["model"])
    assert "module.embed.tok.weight" in keys and "module.blocks.1.attn.qkv.bias" in keys and "module.head.lm.weight" in keys


def test_checkpoint_moves_between_strategies():
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "ck.pt")
        a = launch(run_and_save, 2, "zero2", path)
        b = launch(resume, 2, "zero3", path)
    assert a[0][0] == b[0][0]
    assert torch.equal(a[0][1], b[0][1])


@pytest.mark.parametrize("strategy", ["zero1", "zero2", "zero3"])
def test_bf16_resume_restores_the_fp32_master_weights(strategy):
    """16-bit parameters: the optimizer's fp32 master copy and fp32 moments are part of the checkpoint.  A resumed
    run continues bit-identically, also when the loading optimizer had stepped before and holds a stale master."""
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "ck.pt")
        a = launch(run_and_save, 2, strategy, path, torch.bfloat16)
        b = launch(resume, 2, strategy, path, torch.bfloat16)
        c = launch(resume, 2, strategy, path, torch.bfloat16, 2)
        blob = torch.load(path, weights_only=False)
    assert blob["optim"]["master"] and all(t.dtype == torch.float32 for t in blob["optim"]["master"].values())
    assert all(t.dtype == torch.float32 for t in blob["optim"]["exp_avg"].values())
    for other in (b, c):
        assert a[0][0] == other[0][0] and a[1][0] == other[1][0]
        assert torch.equal(a[0][1], other[0][1])


def _load_then_inspect(g, path):
    w, opt, finish = build(g, "zero2", torch.bfloat16)
    steps(g, w, finish, 0, 2)
    ckpt.save(path, w, opt)
    w2, opt2, _ = build(g, "zero2", torch.bfloat16)
    ckpt.load(path, w2, opt2)
    _, m, v = opt2.state["flat"]
    return (m.dtype, v.dtype, opt2.master["flat"].dtype, torch.equal(opt2.master["flat"], opt.master["flat"]),
            torch.equal(m, opt.state["flat"][1]))


def test_bf16_master_survives_a_load(tmp_path):
    """After load() the optimizer steps fp32 master weights with fp32 moments, never the bf16 shard itself."""
    for m_dt, v_dt, w_dt, same_master, same_m in launch(_load_then_inspect, 2, str(tmp_path / "ck.pt")):
        assert m_dt == v_dt == w_dt == torch.float32
        assert same_master and same_m


def test_adam_args_refuse_sixteen_bit_arrays():
    from tandem_b200.parallel.symm import AdamArgs

    sc = ShardedAdamW().scalars(1.0)
    f32 = torch.zeros(8)
    b16 = torch.zeros(8, dtype=torch.bfloat16)
    AdamArgs.make(f32, f32, f32, sc, True, b16)
    with pytest.raises(TypeError):
        AdamArgs.make(b16, f32, f32, sc, True)
    with pytest.raises(TypeError):
        AdamArgs.make(f32, b16, b16, sc, True)
    with pytest.raises(TypeError):
        AdamArgs.make(f32, f32, f32, sc, True, f32)
