"""Verification and benchmark driver (the counterpart of the reference's bench/run.py).

  python -m tandem_b200.run verify     [--device cpu|cuda] [--ranks 2]
        A small GPT, deterministic kernels, 20 steps: losses and weights of DDP, ZeRO-1/2/3 against
        torch DDP (gloo on CPU, NCCL on GPUs), and GPipe / 1F1B against one process accumulating
        gradients.  Bit-for-bit at 2 ranks ((a/2)+(b/2) is order-independent).
  python -m tandem_b200.run allreduce  [--device cpu|cuda] [--ranks 2]
        All-reduce by size against torch.distributed (gloo / NCCL): time, algorithm and bus bandwidth.
        (The full GPU sweep over every collective is `python -m tandem_b200.bench_collectives`.)
  python -m tandem_b200.run contention [--ranks 2]                      (GPUs only)
        A 64 MB all-reduce alone and while the GPU runs GEMMs it does not depend on.
  python -m tandem_b200.run bench      [--device cpu|cuda] [--ranks 2] [--model medium] [--steps 12]
        Step time, tokens/s and peak memory per strategy, with the share of communication hidden
        behind compute (profile of the last step) and an optional Chrome trace (--trace out.json).

One JSON line per measurement, also appended to --out.  On GPUs every time is device time from
CUDA events, reduced as the maximum over ranks; bus bandwidth = algorithm bandwidth x 2(n-1)/n.
"""

import argparse
import json
import os
import statistics
import tempfile
import time

import torch
import torch.multiprocessing as mp

from . import launch
from .data import synthetic, uniform_tokens
from .ddp import DDP
from .model import GPT, Config, count_params, loss_fn
from .optim import ShardedAdamW
from .pipeline import Pipeline
from .profile import Timeline, chrome_trace, summarize
from .zero import FSDP, ZeRO

LR, WD = 3e-4, 0.1
OUT = None


def emit(row):
    line = json.dumps(row)
    print(line, flush=True)
    if OUT:
        with open(OUT, "a") as f:
            f.write(line + "\n")


def setup(device, index, deterministic):
    if device == "cuda":
        torch.cuda.set_device(index)
        if deterministic:
            os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
            torch.use_deterministic_algorithms(True)
            torch.backends.cuda.enable_flash_sdp(False)
            torch.backends.cuda.enable_mem_efficient_sdp(False)
        return torch.device("cuda", index)
    torch.set_num_threads(1)
    return torch.device("cpu")


def flat_weights(params):
    return torch.cat([p.detach().reshape(-1).float().cpu() for p in params])


class StepTimer:
    """Wall time on CPU ranks, CUDA events on GPU ranks."""

    def __init__(self, dev):
        self.dev, self.times = dev, []

    def __enter__(self):
        if self.dev.type == "cuda":
            self.a, self.b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.a.record()
        else:
            self.t0 = time.perf_counter()

    def __exit__(self, *exc):
        if self.dev.type == "cuda":
            self.b.record()
            self.b.synchronize()
            self.times.append(self.a.elapsed_time(self.b) / 1e3)
        else:
            self.times.append(time.perf_counter() - self.t0)


# ------------------------------------------------------------------------------------------ ranks
def ours_rank(g, strategy, cfg, steps, batch, micro, deterministic, want_weights, profile):
    dev = setup(g.device.type, g.device.index or 0, deterministic)
    torch.manual_seed(0)
    text = synthetic(200_000)
    model = GPT(cfg).to(dev)
    tl = Timeline(enabled=profile, device=dev)
    world, rank = g.size, g.rank
    pipe = None
    if strategy.startswith("ddp"):
        wrapped = DDP(model, g, overlap=strategy != "ddp-nooverlap")
        opt = torch.optim.AdamW(model.parameters(), lr=LR, weight_decay=WD, foreach=False)
    elif strategy in ("zero1", "zero2"):
        wrapped = ZeRO(model, g, int(strategy[-1]), ShardedAdamW(lr=LR, weight_decay=WD, fused=False if deterministic else None))
    elif strategy == "zero3":
        wrapped = FSDP(model, g, ShardedAdamW(lr=LR, weight_decay=WD, fused=False if deterministic else None))
    else:
        pipe = Pipeline(model, g, micro, strategy[3:], timeline=tl)
        opt = torch.optim.AdamW(pipe.parameters(), lr=LR, weight_decay=WD, foreach=False)
        world, rank = 1, 0
    losses, timer = [], StepTimer(dev)
    if dev.type == "cuda":
        torch.cuda.reset_peak_memory_stats(dev)
    for step in range(steps):
        x, y = text.batch(step, batch, cfg.seq, rank=rank, world=world, device=dev)
        if profile and step == steps - 1:
            g.trace.clear()
            g.waits.clear()
            g.tracing = True
            tl.spans.clear()
        with timer:
            if pipe is not None:
                loss = pipe.train_step(x, y)
                opt.step()
                opt.zero_grad()
            else:
                with tl.span("forward"):
                    loss = wrapped(x, y)
                with tl.span("backward"):
                    loss.backward()
                with tl.span("optimizer"):
                    if strategy.startswith("ddp"):
                        opt.step()
                        opt.zero_grad()
                    else:
                        wrapped.step()
                        wrapped.zero_grad()
        losses.append(None if loss is None else loss.item())
    g.tracing = False
    g._drain_spans()
    out = {"losses": losses, "times": timer.times,
           "peak_mem": torch.cuda.max_memory_allocated(dev) if dev.type == "cuda" else None}
    if profile:
        comm = [s for s in g.trace if s[0] != "barrier"]
        out["profile"] = summarize(tl.spans, comm, list(g.waits), timer.times[-1])
        out["trace"] = (tl.spans, comm)
    if want_weights:
        if strategy == "zero3":
            out["weights"] = wrapped.full_parameters().float().cpu()
        elif pipe is not None:
            out["weights"] = flat_weights(pipe.parameters())
        else:
            out["weights"] = flat_weights(model.parameters())
    return out


def torch_rank(rank, world, init, out, device, strategy, cfg, steps, batch, deterministic, want_weights):
    import torch.distributed as dist

    dev = setup(device, rank, deterministic)
    dist.init_process_group("nccl" if device == "cuda" else "gloo", init_method=f"file://{init}", rank=rank, world_size=world)
    torch.manual_seed(0)
    text = synthetic(200_000)
    model = GPT(cfg).to(dev)
    if strategy == "torch-ddp":
        from torch.nn.parallel import DistributedDataParallel

        wrapped = DistributedDataParallel(model, device_ids=[rank] if device == "cuda" else None)
    else:
        from torch.distributed.fsdp import FullyShardedDataParallel, ShardingStrategy
        from torch.distributed.fsdp.wrap import ModuleWrapPolicy

        from .model import Block, Embed, Head

        wrapped = FullyShardedDataParallel(model, auto_wrap_policy=ModuleWrapPolicy({Embed, Block, Head}),
                                           sharding_strategy=ShardingStrategy.FULL_SHARD,
                                           device_id=dev if device == "cuda" else None, use_orig_params=True)
    opt = torch.optim.AdamW(wrapped.parameters(), lr=LR, weight_decay=WD, foreach=False)
    losses, timer = [], StepTimer(dev)
    if dev.type == "cuda":
        torch.cuda.reset_peak_memory_stats(dev)
    for step in range(steps):
        x, y = text.batch(step, batch, cfg.seq, rank=rank, world=world, device=dev)
        with timer:
            loss = wrapped(x, y)
            loss.backward()
            opt.step()
            opt.zero_grad()
        losses.append(loss.item())
    res = {"losses": losses, "times": timer.times,
           "peak_mem": torch.cuda.max_memory_allocated(dev) if dev.type == "cuda" else None}
    if want_weights:
        if strategy == "torch-fsdp":
            from torch.distributed.fsdp import FullyShardedDataParallel

            with FullyShardedDataParallel.summon_full_params(wrapped):
                res["weights"] = flat_weights(model.parameters())
        else:
            res["weights"] = flat_weights(model.parameters())
    torch.save(res, f"{out}.{rank}")
    dist.destroy_process_group()


def run_torch(strategy, device, world, cfg, steps, batch, deterministic=False, want_weights=False):
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(torch_rank, args=(world, os.path.join(d, "init"), os.path.join(d, "out"), device, strategy, cfg, steps, batch,
                                   deterministic, want_weights), nprocs=world)
        return [torch.load(os.path.join(d, f"out.{r}"), weights_only=False) for r in range(world)]


def run_ours(strategy, device, world, cfg, steps, batch, micro=4, deterministic=False, want_weights=False, profile=False):
    return launch(ours_rank, world, strategy, cfg, steps, batch, micro, deterministic, want_weights, profile, device=device)


def single_rank(_, device, cfg, steps, batch, micro, deterministic, out):
    dev = setup(device, 0, deterministic)
    torch.manual_seed(0)
    text = synthetic(200_000)
    model = GPT(cfg).to(dev)
    opt = torch.optim.AdamW(model.parameters(), lr=LR, weight_decay=WD, foreach=False)
    losses, timer = [], StepTimer(dev)
    for step in range(steps):
        x, y = text.batch(step, batch, cfg.seq, device=dev)
        with timer:
            total = 0
            for xb, yb in zip(x.chunk(micro), y.chunk(micro)):
                loss = loss_fn(model(xb), yb) / micro
                loss.backward()
                total = total + loss.detach()
            opt.step()
            opt.zero_grad()
        losses.append(total.item())
    torch.save({"losses": losses, "times": timer.times, "weights": flat_weights(model.parameters()),
                "unit_sizes": [sum(p.numel() for p in u.parameters()) for u in model.units()],
                "peak_mem": torch.cuda.max_memory_allocated(dev) if dev.type == "cuda" else None}, out)


def run_single(device, cfg, steps, batch, micro, deterministic=False):
    with tempfile.TemporaryDirectory() as d:
        out = os.path.join(d, "single.pt")
        mp.spawn(single_rank, args=(device, cfg, steps, batch, micro, deterministic, out), nprocs=1)
        return torch.load(out, weights_only=False)


# ------------------------------------------------------------------------------------------ sections
def compare(name, ours, ref, ref_name):
    a, b = ours[0], ref[0]
    emit({"section": "verify", "strategy": name, "against": ref_name, "losses_equal": a["losses"] == b["losses"],
          "weights_equal": bool(torch.equal(a["weights"], b["weights"])),
          "max_weight_diff": float((a["weights"] - b["weights"]).abs().max()), "steps": len(b["losses"]),
          "final_loss": a["losses"][-1]})


def verify(device, world):
    cfg = Config(seq=128, layers=4, heads=4, dim=256)
    kw = dict(cfg=cfg, steps=20, batch=16, deterministic=True, want_weights=True)
    ref = run_torch("torch-ddp", device, world, **kw)
    emit({"section": "verify", "model_params": count_params(GPT(cfg)), "device": device, "ranks": world, "torch": torch.__version__})
    try:
        compare("torch-fsdp", run_torch("torch-fsdp", device, world, **kw), ref, "torch-ddp")
    except Exception as e:
        emit({"section": "verify", "strategy": "torch-fsdp", "error": repr(e)[:300]})
    for s in ("ddp", "zero1", "zero2", "zero3"):
        compare(s, run_ours(s, device, world, **kw), ref, "torch-ddp")
    single = run_single(device, cfg, 20, 16, 4, deterministic=True)
    for s in ("pp-gpipe", "pp-1f1b"):
        ours = run_ours(s, device, world, micro=4, **kw)
        stages = torch.cat([o["weights"] for o in ours])
        emit({"section": "verify", "strategy": s, "against": "single-process accumulation", "stages": world,
              "losses_equal": ours[-1]["losses"] == single["losses"], "weights_equal": bool(torch.equal(stages, single["weights"])),
              "max_weight_diff": float((stages - single["weights"]).abs().max())})


def ar_ours(g, sizes, reps):
    dev = setup(g.device.type, g.device.index or 0, False)
    out = {}
    for mb in sizes:
        x = g.empty(mb * (1 << 20) // 4, torch.float32, dev)
        x.fill_(1.0)
        g.all_reduce(x)
        ts = []
        for _ in range(reps):
            g.barrier()
            timer = StepTimer(dev)
            with timer:
                g.all_reduce(x)
            ts.append(timer.times[0])
        out[mb] = statistics.median(ts)
        g.release(x)
    return out


def ar_torch(rank, world, init, out, device, sizes, reps):
    import torch.distributed as dist

    dev = setup(device, rank, False)
    dist.init_process_group("nccl" if device == "cuda" else "gloo", init_method=f"file://{init}", rank=rank, world_size=world)
    res = {}
    for mb in sizes:
        x = torch.ones(mb * (1 << 20) // 4, device=dev)
        dist.all_reduce(x)
        ts = []
        for _ in range(reps):
            dist.barrier()
            timer = StepTimer(dev)
            with timer:
                dist.all_reduce(x)
            ts.append(timer.times[0])
        res[mb] = statistics.median(ts)
    torch.save(res, f"{out}.{rank}")
    dist.destroy_process_group()


def allreduce(device, world):
    sizes, reps = [1, 4, 16, 64, 256], 10
    ours = launch(ar_ours, world, sizes, reps, device=device)
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(ar_torch, args=(world, os.path.join(d, "init"), os.path.join(d, "o"), device, sizes, reps), nprocs=world)
        ref = [torch.load(os.path.join(d, f"o.{r}")) for r in range(world)]
    base = "nccl" if device == "cuda" else "gloo"
    bus = 2 * (world - 1) / world
    for mb in sizes:
        t_ours, t_ref = max(o[mb] for o in ours), max(o[mb] for o in ref)
        emit({"section": "allreduce", "MB": mb, "ranks": world, "ours_ms": t_ours * 1e3, f"{base}_ms": t_ref * 1e3,
              "ours_GBps": mb / 1024 / t_ours, f"{base}_GBps": mb / 1024 / t_ref, "ours_bus_GBps": mb / 1024 / t_ours * bus,
              f"{base}_bus_GBps": mb / 1024 / t_ref * bus})


def contention_rank(g, mb, reps, gemms):
    """Device time of a 64 MB all-reduce alone, then while the default stream runs GEMMs it does not depend on."""
    dev = setup("cuda", g.device.index or 0, False)
    x = g.empty(mb * (1 << 20) // 4, torch.float32, dev)
    a = torch.randn(4096, 4096, device=dev).bfloat16()
    g.all_reduce(x)
    a @ a
    torch.cuda.synchronize()

    def once(busy):
        g.barrier()
        x.fill_(1.0)
        g.trace.clear()
        g.tracing = True
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        w = g.all_reduce(x, async_op=True)
        for _ in range(gemms if busy else 0):
            a @ a
        w.wait()
        t1.record()
        torch.cuda.synchronize()
        g.tracing = False
        g._drain_spans()
        _, s, e, _ = g.trace[-1]
        assert torch.equal(x, torch.full_like(x, float(g.size))), "wrong all-reduce result"
        return e - s, t0.elapsed_time(t1) / 1e3

    def gemm_alone():
        timer = StepTimer(dev)
        with timer:
            for _ in range(gemms):
                a @ a
        return timer.times[0]

    alone = statistics.median(once(False)[0] for _ in range(reps))
    busy = [once(True) for _ in range(reps)]
    return {"comm_alone_ms": alone * 1e3, "comm_busy_ms": statistics.median(c for c, _ in busy) * 1e3,
            "gemms_ms": statistics.median(gemm_alone() for _ in range(reps)) * 1e3,
            "gemms_plus_comm_ms": statistics.median(t for _, t in busy) * 1e3}


def contention(world):
    emit({"section": "contention", "gpu": torch.cuda.get_device_name(0), "ranks": world})
    for priority in (0, -1):
        r = launch(contention_rank, world, 64, 5, 16, device="cuda", priority=priority)
        row = {"section": "contention", "priority": priority}
        for k in r[0]:
            row[k] = round(max(o[k] for o in r), 3)
        row["slowdown"] = round(row["comm_busy_ms"] / row["comm_alone_ms"], 2)
        emit(row)


def bench(device, world, preset, steps, batch, trace_path):
    cfg = Config.preset(preset)
    tokens = batch * cfg.seq
    emit({"section": "bench", "model": preset, "params": count_params(GPT(cfg)), "global_batch": batch, "seq": cfg.seq,
          "device": device, "ranks": world})

    def report(name, res):
        per_rank = [statistics.median(r["times"][2:]) if len(r["times"]) > 2 else r["times"][-1] for r in res]
        med = max(per_rank)
        row = {"section": "bench", "strategy": name, "step_ms": med * 1e3, "tokens_per_s": tokens / med,
               "peak_mem_MB": [None if r.get("peak_mem") is None else round(r["peak_mem"] / 2 ** 20) for r in res],
               "final_loss": statistics.mean(r["losses"][-1] for r in res if r["losses"][-1] is not None)}
        if "profile" in res[0]:
            row["profile_rank0"] = {k: (round(v, 5) if isinstance(v, float) else v) for k, v in res[0]["profile"].items()}
        emit(row)

    report("single", [run_single(device, cfg, steps, batch, 1)])
    for s in ("torch-ddp", "torch-fsdp"):
        try:
            report(s, run_torch(s, device, world, cfg, steps, batch))
        except Exception as e:
            emit({"section": "bench", "strategy": s, "error": repr(e)[:300]})
    for s in ("ddp", "ddp-nooverlap", "zero1", "zero2", "zero3", "pp-gpipe", "pp-1f1b"):
        try:
            res = run_ours(s, device, world, cfg, steps, batch, profile=s in ("ddp", "ddp-nooverlap", "zero3"))
            report(s, res)
            if trace_path and s == "ddp":
                chrome_trace([r["trace"] for r in res], trace_path)
        except Exception as e:
            emit({"section": "bench", "strategy": s, "error": repr(e)[:300]})


def main():
    global OUT
    ap = argparse.ArgumentParser()
    ap.add_argument("what", nargs="?", default="verify", choices=["verify", "allreduce", "contention", "bench", "all"])
    ap.add_argument("--device", choices=["cuda", "cpu"], default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--ranks", type=int, default=2)
    ap.add_argument("--model", default="medium")
    ap.add_argument("--steps", type=int, default=12)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--trace", default=None)
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    OUT = a.out
    if a.device == "cuda" and torch.cuda.device_count() < a.ranks:
        raise SystemExit(f"needs {a.ranks} GPUs, found {torch.cuda.device_count()}")
    if a.what in ("verify", "all"):
        verify(a.device, a.ranks)
    if a.what in ("allreduce", "all"):
        allreduce(a.device, a.ranks)
    if a.what in ("contention", "all") and a.device == "cuda":
        contention(a.ranks)
    if a.what in ("bench", "all"):
        bench(a.device, a.ranks, a.model, a.steps, a.batch, a.trace)


if __name__ == "__main__":
    main()
