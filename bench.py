"""Flagship benchmark: training throughput of the 85.8M-parameter GPT
(12 layers, d_model 768, 12 heads, MLP 3072, vocab 65, seq 512, global batch 16)
in tokens/s, on N GPUs of one node.

  python bench.py --gpus 1 --steps 20 --warmup 5
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      bench.py --gpus N --steps K --warmup W

--impl ours       tandem_b200: DDP / ZeRO-1/2 / FSDP wrappers on the sm_100a kernels, bf16 compute,
                  fp32 master weights (default strategy: ddp).
--impl reference  the unmodified reference package installed under baseline/_ref, through its own
                  launch() / DDP / model and stock fp32 code path.
--impl torch      torch DistributedDataParallel / FSDP over NCCL with bf16 autocast (context only).

--strategy ddp | zero1 | zero2 | zero3 | gpipe | 1f1b and --model 85.8m | 1.3b | pp24 select the other training
configurations of the benchmark plan (1.3B under ZeRO-3; the 24-layer model as a pipeline); analysis switches:
--global-batch, --precision fp32 (with --kernels torch), --opt, --fused-step, --update-during-backward, --balance.

Data are synthetic: token ids uniform in [0, vocab) from a seed; weights are random-init.
The global batch is fixed, so per-GPU work shrinks as N grows ("strong" scaling).
Rank 0 prints one JSON line.  `value` is timed on the device with CUDA events over exactly
--steps steps (inputs already resident), max over ranks; `e2e` repeats the measurement with,
every step, the host-to-device copy of that step's tokens from pinned memory and a
device-to-host read of the loss.
"""

import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch

MODEL = dict(vocab=65, seq=512, layers=12, heads=12, dim=768)
GLOBAL_BATCH = 16
MODEL_LABEL, MODEL_DESC = "85.8M", "gpt-85.8M (L12 d768 h12 mlp3072 vocab65)"
LR, WD = 3e-4, 0.1
PUBLISHED_TOKENS_PER_S = 10265.0  # the reference's own "tandem DDP" row: 2x T4, fp32 (its README / bench/t4 results)
# The unmodified reference (its stock fp32 path, Python engine) measured through `--impl reference` on this pool's B200s:
# tokens/s of the flagship under DDP at 1, 2, 4 and 8 GPUs.  The same-hardware denominator beside the published T4 one.
REFERENCE_ON_B200_TOKENS_PER_S = {1: 81494.0, 2: 123502.0, 4: 162418.0, 8: 187001.0}
MICRO_BATCHES = 16  # pipeline strategies

# The other training configurations of the benchmark plan (--model); the flagship above is the default.
OTHER_MODELS = {
    "1.3b": (dict(vocab=50304, seq=2048, layers=24, heads=16, dim=2048), 64, "1.3B", "gpt-1.3B (L24 d2048 h16 mlp8192 vocab50304)"),
    "pp24": (dict(vocab=50304, seq=1024, layers=24, heads=16, dim=1024), 64, "pp24L", "gpt-24L (L24 d1024 h16 mlp4096 vocab50304), 16 micro-batches of 4"),
}


def select_model(name):
    global MODEL, GLOBAL_BATCH, MODEL_LABEL, MODEL_DESC, PUBLISHED_TOKENS_PER_S
    if name in OTHER_MODELS:
        MODEL, GLOBAL_BATCH, MODEL_LABEL, MODEL_DESC = OTHER_MODELS[name]
        PUBLISHED_TOKENS_PER_S = None  # the reference publishes nothing for this configuration


# ---------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="clocks-", suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            with open(self.path) as f:
                for line in f:
                    parts = [p.strip() for p in line.split(",")]
                    if len(parts) < 8:
                        continue
                    try:
                        sm.append(float(parts[0]))
                        mx.append(float(parts[1]))
                    except ValueError:
                        continue
                    for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[4:8]):
                        if v.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# ---------------------------------------------------------------------------------------------- data
def token_batches(count, per_rank, rank, world, vocab, seq, seed=1234):
    """`count` pinned host batches (x, y) of this rank's rows of the global batch: token ids uniform in
    [0, vocab) drawn from a per-step seed (every rank draws the whole batch and keeps its rows)."""
    out = []
    for step in range(count):
        gen = torch.Generator().manual_seed(seed * 1_000_003 + step)
        rows = torch.randint(0, vocab, (per_rank * world, seq + 1), generator=gen)[rank * per_rank:(rank + 1) * per_rank]
        out.append((rows[:, :-1].contiguous().pin_memory(), rows[:, 1:].contiguous().pin_memory()))
    return out


def timed_loops(step_fn, batches, steps, warmup, device, barrier, reduce_max, launches=None):
    """Returns (device-timed ms/step with resident inputs, e2e ms/step incl. H2D + loss read, h2d bytes, d2h bytes, launches)."""
    resident = [(x.to(device), y.to(device)) for x, y in batches]
    for i in range(warmup):
        loss = step_fn(*resident[i % len(resident)])
    loss.item()
    barrier()
    torch.cuda.synchronize(device)
    if launches is not None:
        launches(True)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(steps):
        loss = step_fn(*resident[i % len(resident)])
    t1.record()
    torch.cuda.synchronize(device)
    barrier()
    n_launch = launches(False) if launches is not None else 0
    dev_ms = reduce_max(t0.elapsed_time(t1) / steps)

    # end to end: pinned host tokens -> device every step, loss back to the host every step
    for i in range(min(warmup, 3)):
        x, y = batches[i % len(batches)]
        step_fn(x.to(device, non_blocking=True), y.to(device, non_blocking=True)).item()
    barrier()
    torch.cuda.synchronize(device)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(steps):
        x, y = batches[i % len(batches)]
        loss = step_fn(x.to(device, non_blocking=True), y.to(device, non_blocking=True))
        last = loss.item()
    t1.record()
    torch.cuda.synchronize(device)
    barrier()
    e2e_ms = reduce_max(t0.elapsed_time(t1) / steps)
    x, y = batches[0]
    h2d = x.numel() * x.element_size() + y.numel() * y.element_size()
    return dev_ms, e2e_ms, h2d, 4, n_launch, last


def result_line(args, impl, strategy, dev_ms, e2e_ms, h2d, d2h, launches, clocks, dtype, extra=None):
    tokens = GLOBAL_BATCH * MODEL["seq"]
    value = tokens / (dev_ms / 1e3)
    row = {
        "metric": f"gpt_{MODEL_LABEL}_{strategy}_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": value / PUBLISHED_TOKENS_PER_S if PUBLISHED_TOKENS_PER_S else None,
        "vs_baseline_is": "value / the reference's published tandem-DDP row (2x T4, fp32)" if PUBLISHED_TOKENS_PER_S else None,
        "vs_reference_on_b200": (value / REFERENCE_ON_B200_TOKENS_PER_S[args.gpus]
                                 if PUBLISHED_TOKENS_PER_S and strategy == "ddp" and args.gpus in REFERENCE_ON_B200_TOKENS_PER_S else None),
        "dtype": dtype, "data": "synthetic uniform-random token ids, random-init weights",
        "impl": impl,
        "config": {"model": MODEL_DESC, "global_batch": GLOBAL_BATCH, "seq_len": MODEL["seq"],
                   "parallelism": f"{strategy}{args.gpus}", "optimizer": "AdamW lr 3e-4 wd 0.1",
                   "l2": "no explicit flush: each step streams parameters, gradients, optimizer state and activations "
                         "(>1.3 GB) through the 126 MB L2", "timing": "CUDA events on the training stream, max over ranks"},
        "clocks": clocks,
        "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
    }
    if extra:
        row.update(extra)
    return row


# ---------------------------------------------------------------------------------------------- ours
def run_ours(args):
    import tandem_b200
    from tandem_b200.ddp import DDP, BucketAdamW, ShardedBucketAdamW
    from tandem_b200.model import GPT, Config
    from tandem_b200.optim import ShardedAdamW
    from tandem_b200.parallel.symm import cuda_lib
    from tandem_b200.zero import FSDP, ZeRO

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    if world > 1:
        # torch.distributed is plumbing only: it lets the symmetric heap be bound to an NVSwitch multicast object
        # (NVLS all-reduce kernels) and carries pipeline point-to-point traffic.  The collectives are this library's.
        import torch.distributed as dist

        local = int(os.environ.get("LOCAL_RANK", str(rank)))
        torch.cuda.set_device(local)
        # a stalled NCCL transfer ends the run with the name of the operation instead of sitting until the job is killed
        dist.init_process_group("nccl", device_id=torch.device("cuda", local),
                                timeout=datetime.timedelta(seconds=int(os.environ.get("TANDEM_PG_TIMEOUT_S", "300"))))
    g = tandem_b200.Group.from_env(device="cuda")
    dev = g.device
    lib = cuda_lib()
    torch.manual_seed(0)
    kernels = args.kernels
    model = GPT(Config(kernels=kernels, **MODEL)).to(dev)
    pure_bf16 = kernels == "b200"
    fp32 = args.precision == "fp32"  # the reference's precision: this runtime's engine and strategies on torch's fp32 kernels
    if fp32 and pure_bf16:
        raise SystemExit("--precision fp32 needs --kernels torch (the hand-written kernels compute in bf16)")
    if pure_bf16:
        model = model.bfloat16()  # fp32 master weights live in the optimizer
    graphed = bool(args.graph) and args.strategy in ("ddp", "zero1", "zero2", "zero3")
    # measured: the replicated update is the faster one at this model size (2 GPUs: 7.4 vs 8.1 ms, 4 GPUs: 5.4 vs 6.5 ms).
    # Sharding saves (N-1)/N of 0.37 ms of optimizer traffic but puts a reduce-scatter -> all-gather chain per bucket on
    # the path to the next forward, where the all-reduce overlaps backward completely.  It is what to use when the
    # optimizer state does not fit (1/N of the memory), so it stays selectable.
    sharded_opt = args.opt == "sharded"
    if args.strategy == "ddp":
        wrapped = DDP(model, g, rebuild=False)
        # replicated: all-reduce + one AdamW kernel per bucket on every rank; sharded: reduce-scatter with the AdamW
        # update in its epilogue + all-gather of the parameters (same values, 1/N of the optimizer traffic per rank)
        if sharded_opt:
            opt = ShardedBucketAdamW(wrapped, lr=LR, weight_decay=WD)
        else:  # each span is updated as soon as its all-reduce has finished, beside the rest of backward
            opt = BucketAdamW(wrapped, lr=LR, weight_decay=WD, during_backward=bool(args.update_during_backward))
        closer = opt
    elif args.strategy in ("zero1", "zero2"):
        wrapped = ZeRO(model, g, int(args.strategy[-1]), ShardedAdamW(lr=LR, weight_decay=WD), fused_step=bool(args.fused_step),
                       capturable=graphed)
        closer = wrapped
    elif args.strategy == "zero3":
        # the GEMM that gathers its own weight keeps a host-side epoch per call, so it is not recorded into graphs
        wrapped = FSDP(model, g, ShardedAdamW(lr=LR, weight_decay=WD), fuse_gather_gemm=bool(args.fuse) and not graphed,
                       capturable=graphed)
        closer = wrapped
    elif args.strategy in ("gpipe", "1f1b"):
        from tandem_b200.pipeline import Pipeline

        # one stage per GPU, stage traffic on NCCL p2p; --balance cost deals units out by estimated compute
        wrapped = Pipeline(model, g, MICRO_BATCHES, args.strategy, balance=args.balance)
        opt = torch.optim.AdamW(wrapped.parameters(), lr=LR, weight_decay=WD, fused=True)
        closer = None
    else:
        raise SystemExit(f"unknown strategy {args.strategy}")
    finish = (lambda: (closer.step(), closer.zero_grad())) if closer is not None else None
    pipelined = args.strategy in ("gpipe", "1f1b")

    def step_fn(x, y):
        if pipelined:
            loss = wrapped.train_step(x, y)
            opt.step()
            opt.zero_grad()
            return loss if loss is not None else torch.zeros((), device=dev)
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=not pure_bf16 and not fp32):
            loss = wrapped(x, y)
        loss.backward()
        finish()
        return loss

    per_rank = GLOBAL_BATCH if pipelined else GLOBAL_BATCH // world
    if graphed:
        from tandem_b200.parallel.graph import GraphedStep

        ex = torch.zeros(per_rank, MODEL["seq"], dtype=torch.long, device=dev)
        step_fn = GraphedStep(wrapped, closer, ex, ex.clone(), autocast=None if pure_bf16 or fp32 else torch.bfloat16)

    def reduce_max(v):
        if world == 1:
            return v
        gathered = torch.zeros(world, dtype=torch.float64)
        gathered[rank] = v
        g.all_reduce(gathered)  # CPU tensor: host control plane
        return float(gathered.max())

    # a pipeline feeds the whole batch to every stage (the first uses the tokens, the last the targets)
    batches = token_batches(8, per_rank, 0 if pipelined else rank, 1 if pipelined else world, MODEL["vocab"], MODEL["seq"])
    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    lib.tb_launch_count(1)
    step_fn(batches[0][0].to(dev), batches[0][1].to(dev))  # one eager-or-replayed step to count our kernels per step
    per_step = lib.tb_launch_count(1)
    if graphed:
        per_step = step_fn.launches_per_step
    dev_ms, e2e_ms, h2d, d2h, launches, last = timed_loops(step_fn, batches, args.steps, args.warmup, dev, g.barrier, reduce_max)
    launches = per_step * args.steps
    if pipelined:
        last = reduce_max(float(last))  # only the last stage computes the loss
    clocks = sampler.stop() if rank == 0 else None
    nvls = bool(g._sym is not None and g._sym.nvls)
    g.close()
    if rank == 0:
        print(json.dumps(result_line(args, "ours", args.strategy, dev_ms, e2e_ms, h2d, d2h, int(launches), clocks, "fp32" if fp32 else "bf16",
                                     {"kernels": kernels, "final_loss": last, "cuda_graph": bool(graphed), "nvls": nvls,
                                      "optimizer": ("sharded over ranks, fused into the reduce-scatter" if sharded_opt else "replicated")
                                      if args.strategy == "ddp" else ("per stage (torch fused AdamW)" if pipelined else "sharded")})), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------- torch DDP (context)
def run_torch(args):
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel

    from tandem_b200.model import GPT, Config

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    model = GPT(Config(**MODEL)).to(dev)
    if args.strategy == "zero3" and world > 1:
        from torch.distributed.fsdp import FullyShardedDataParallel, MixedPrecision
        from torch.distributed.fsdp.wrap import ModuleWrapPolicy

        from tandem_b200.models.gpt import Block

        bf16 = torch.bfloat16
        wrapped = FullyShardedDataParallel(model, auto_wrap_policy=ModuleWrapPolicy({Block}), device_id=dev, use_orig_params=True,
                                           mixed_precision=MixedPrecision(param_dtype=bf16, reduce_dtype=bf16, buffer_dtype=bf16))
    else:
        wrapped = DistributedDataParallel(model, device_ids=[local]) if world > 1 else model
    opt = torch.optim.AdamW(wrapped.parameters(), lr=LR, weight_decay=WD, fused=True)

    def step_fn(x, y):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = wrapped(x, y)
        loss.backward()
        opt.step()
        opt.zero_grad()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()

    def reduce_max(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    batches = token_batches(8, GLOBAL_BATCH // world, rank, world, MODEL["vocab"], MODEL["seq"])
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    dev_ms, e2e_ms, h2d, d2h, _, last = timed_loops(step_fn, batches, args.steps, args.warmup, dev, barrier, reduce_max)
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        print(json.dumps(result_line(args, "torch", "fsdp" if args.strategy == "zero3" else "ddp", dev_ms, e2e_ms, h2d, d2h, 0, clocks,
                                     "bf16", {"final_loss": last})),
              flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------- reference
def reference_rank(g, steps, warmup, strategy, model_name):
    """Runs inside the reference's launch(): its GPT, its DDP / ZeRO / FSDP, torch AdamW as its bench does."""
    import torch
    from tandem.ddp import DDP
    from tandem.model import GPT, Config
    from tandem.optim import ShardedAdamW
    from tandem.zero import FSDP, ZeRO

    sys.path.insert(0, ROOT)
    select_model(model_name)  # launch() starts fresh processes: this module's configuration is set again in each
    dev = g.device
    torch.manual_seed(0)
    model = GPT(Config(**MODEL)).to(dev)
    pipelined = strategy in ("gpipe", "1f1b")
    if strategy == "ddp":
        wrapped = DDP(model, g)
        opt = torch.optim.AdamW(model.parameters(), lr=LR, weight_decay=WD, foreach=False)
        finish = lambda: (opt.step(), opt.zero_grad())
    elif strategy in ("zero1", "zero2"):
        wrapped = ZeRO(model, g, int(strategy[-1]), ShardedAdamW(lr=LR, weight_decay=WD))
        finish = lambda: (wrapped.step(), wrapped.zero_grad())
    elif strategy == "zero3":
        wrapped = FSDP(model, g, ShardedAdamW(lr=LR, weight_decay=WD))
        finish = lambda: (wrapped.step(), wrapped.zero_grad())
    elif pipelined:
        from tandem.pipeline import Pipeline

        wrapped = Pipeline(model, g, MICRO_BATCHES, strategy)  # its own schedules over its own send / recv
        opt = torch.optim.AdamW(wrapped.parameters(), lr=LR, weight_decay=WD, foreach=False)
    else:
        raise ValueError(f"the reference has no strategy {strategy!r}")

    def step_fn(x, y):
        if pipelined:
            loss = wrapped.train_step(x, y)
            opt.step()
            opt.zero_grad()
            return loss if loss is not None else torch.zeros((), device=dev)
        loss = wrapped(x, y)
        loss.backward()
        finish()
        return loss

    per_rank = GLOBAL_BATCH if pipelined else GLOBAL_BATCH // g.size
    batches = token_batches(8, per_rank, 0 if pipelined else g.rank, 1 if pipelined else g.size, MODEL["vocab"], MODEL["seq"])
    sampler = ClockSampler(dev.index)
    if g.rank == 0:
        sampler.start()
    dev_ms, e2e_ms, h2d, d2h, _, last = timed_loops(step_fn, batches, steps, warmup, dev, g.barrier, lambda v: v)
    clocks = sampler.stop() if g.rank == 0 else None
    return {"dev_ms": dev_ms, "e2e_ms": e2e_ms, "h2d": h2d, "d2h": d2h, "clocks": clocks, "loss": last}


def run_reference(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    ref = os.path.join(ROOT, "baseline", "_ref")
    done_flag = os.path.join(tempfile.gettempdir(), f"tb2-ref-done-{os.environ.get('MASTER_PORT', '0')}-{os.getppid()}")
    if rank != 0:
        # The reference starts its own ranks with launch(); the other torchrun ranks only wait for it.
        deadline = time.time() + 3600
        while not os.path.exists(done_flag) and time.time() < deadline:
            time.sleep(0.5)
        return
    try:
        if not os.path.isdir(os.path.join(ref, "tandem")):
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/tandem is missing (reference not installed)"}), flush=True)
            return
        sys.path.insert(0, ref)
        os.environ["PYTHONPATH"] = ref + os.pathsep + ROOT + os.pathsep + os.environ.get("PYTHONPATH", "")
        os.environ.setdefault("TANDEM_TIMEOUT", "120")  # the reference's own limit on its waits: a stuck engine ends in its CommError
        import tandem

        # "auto": the reference's C++ engine (its faster one, selected with backend="cpp" and built by the reference
        # itself on first use) where it has been seen to run clean on this hardware -- 2 GPUs, the group size its own
        # benchmarks use -- with its Python engine as the fall-back; its Python engine at the other sizes (measured at
        # 1, 2, 4 and 8 GPUs).  Its C++ engine waits on interprocess CUDA events without a limit, so a stall at a
        # size it was never run at would not end in an error that a fall-back could catch.
        engines = {"auto": ["cpp", "python"] if args.gpus == 2 else ["python"], "cpp": ["cpp"], "python": ["python"]}[args.ref_backend]
        out, engine, notes = None, None, []
        for engine in engines:
            try:
                out = tandem.launch(reference_rank, args.gpus, args.steps, args.warmup, args.strategy, args.model, device="cuda", backend=engine)
                break
            except Exception as e:
                notes.append(f"{engine}: {repr(e)[:200]}")
        if out is None:
            print(json.dumps({"impl": "reference", "unavailable": "the reference failed to run: " + " | ".join(notes)}), flush=True)
            return
        args.ref_backend = engine
        ref_notes = notes
        dev_ms = max(o["dev_ms"] for o in out)
        e2e_ms = max(o["e2e_ms"] for o in out)
        print(json.dumps(result_line(args, "reference", args.strategy, dev_ms, e2e_ms, out[0]["h2d"], out[0]["d2h"], 0,
                                     out[0]["clocks"], "fp32", {"engine": args.ref_backend, "engine_fallbacks": ref_notes, "final_loss": out[-1]["loss"]})),
              flush=True)
    finally:
        if world > 1:
            open(done_flag, "w").close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--strategy", default="ddp", choices=["ddp", "zero1", "zero2", "zero3", "gpipe", "1f1b"])
    ap.add_argument("--model", default="85.8m", choices=["85.8m", "1.3b", "pp24"],
                    help="85.8m: the flagship; 1.3b: the ZeRO-3 configuration; pp24: the 24-layer pipeline configuration")
    ap.add_argument("--kernels", default=os.environ.get("TANDEM_BENCH_KERNELS", "b200"), choices=["torch", "b200"])
    ap.add_argument("--ref-backend", default=os.environ.get("TANDEM_REF_BACKEND", "auto"), choices=["auto", "python", "cpp"],
                    help="the reference's engine: its Python engine, its C++ engine, or auto (C++ at 2 GPUs with a fall-back to Python; Python elsewhere)")
    ap.add_argument("--opt", default="auto", choices=["auto", "replicated", "sharded"],
                    help="ddp: AdamW replicated on every rank, or sharded and fused into the gradient reduce-scatter (auto: replicated)")
    ap.add_argument("--update-during-backward", type=int, default=1, help="ddp, replicated optimizer: update each span right after its all-reduce (1) or all spans after backward (0)")
    ap.add_argument("--fused-step", type=int, default=0,
                    help="zero2: AdamW inside the reduce-scatter kernels (1) or as its own kernel in step() (0; measured faster at "
                         "this size: 7.24 vs 7.74 ms at 2 GPUs -- with the reference's flat sharding one rank owns a whole bucket, "
                         "so the fused update runs on that rank alone inside a few-block communication kernel)")
    ap.add_argument("--global-batch", type=int, default=0, help="analysis: another global batch than the configuration's (ours and torch arms)")
    ap.add_argument("--precision", default="bf16", choices=["bf16", "fp32"],
                    help="fp32 (with --kernels torch): no autocast, the reference's precision, for a same-precision comparison")
    ap.add_argument("--balance", default="cost", choices=["cost", "units"], help="gpipe / 1f1b (ours): how units are dealt out to stages")
    ap.add_argument("--fuse", type=int, default=1, help="zero3: gather each block's qkv weight inside its GEMM kernel")
    ap.add_argument("--graph", type=int, default=1, help="record the step once as a CUDA graph and replay it (ours: ddp, zero1, zero2, zero3)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    select_model(args.model)
    if args.global_batch:
        # analysis only: e.g. --gpus 1 --global-batch 2 is one rank's share of the flagship at 8 GPUs, without communication
        global GLOBAL_BATCH, PUBLISHED_TOKENS_PER_S
        GLOBAL_BATCH, PUBLISHED_TOKENS_PER_S = args.global_batch, None
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "torch":
        run_torch(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
