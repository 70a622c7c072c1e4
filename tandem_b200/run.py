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

One JSON line per measurement, also appended to --out; the rows carry the reference driver's keys
(bench/run.py:268-271, 347-348, 422-439, 451-459) plus bus bandwidth.  On GPUs every time is device time
from CUDA events, reduced as the maximum over ranks; bus bandwidth = algorithm bandwidth x 2(n-1)/n.
"""

import argparse
import dataclasses
import json
import os
import statistics
import tempfile
import time

import torch
import torch.multiprocessing as mp

from . import launch
from .data import synthetic
from .ddp import DDP
from .model import GPT, Config, count_params, loss_fn
from .optim import ShardedAdamW
from .pipeline import Pipeline
from .profile import Timeline, chrome_trace, summarize
from .zero import FSDP, ZeRO

LEARNING_RATE, WEIGHT_DECAY = 3e-4, 0.1
CORPUS_BYTES = 200_000


# ---------------------------------------------------------------------------------------------- plumbing
class Rows:
    """JSON lines to stdout and, when a path is set, to a file."""

    path = None

    @classmethod
    def write(cls, **fields):
        text = json.dumps(fields)
        print(text, flush=True)
        if cls.path:
            with open(cls.path, "a") as f:
                f.write(text + "\n")


@dataclasses.dataclass
class Job:
    """What one training run does; travels to the ranks as one picklable value."""

    strategy: str
    config: Config
    steps: int
    rows: int                      # rows of the global batch
    micro: int = 4                 # micro-batches (pipeline strategies, single-process accumulation)
    deterministic: bool = False
    keep_weights: bool = False
    profile: bool = False


def claim_device(kind, index, deterministic):
    """Makes `index` this process's device and, when asked, pins torch to reproducible kernels."""
    if kind != "cuda":
        torch.set_num_threads(1)
        return torch.device("cpu")
    torch.cuda.set_device(index)
    if deterministic:
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
        torch.use_deterministic_algorithms(True)
        for switch in (torch.backends.cuda.enable_flash_sdp, torch.backends.cuda.enable_mem_efficient_sdp):
            switch(False)  # leaves the math kernel, the only deterministic attention backward
    return torch.device("cuda", index)


def to_host(parameters):
    return torch.cat([p.detach().float().reshape(-1).cpu() for p in parameters])


def adamw(parameters):
    return torch.optim.AdamW(parameters, lr=LEARNING_RATE, weight_decay=WEIGHT_DECAY, foreach=False)


def peak_memory(device):
    return torch.cuda.max_memory_allocated(device) if device.type == "cuda" else None


class Stopwatch:
    """`with watch: ...` appends the block's duration in seconds to `laps`: device time between two CUDA events
    on a GPU, wall time on the host."""

    def __init__(self, device):
        self.cuda = device.type == "cuda"
        self.laps = []

    def __enter__(self):
        if self.cuda:
            self._events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self._events[0].record()
        else:
            self._began = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.cuda:
            first, last = self._events
            last.record()
            last.synchronize()
            self.laps.append(first.elapsed_time(last) / 1e3)
        else:
            self.laps.append(time.perf_counter() - self._began)
        return False

    @staticmethod
    def time(device, fn):
        watch = Stopwatch(device)
        with watch:
            fn()
        return watch.laps[0]


# ---------------------------------------------------------------------------------------------- our strategies
class Replicated:
    """DDP (with or without overlapping the all-reduces with backward) and torch's per-parameter AdamW."""

    def __init__(self, model, group, job, spans):
        self.model, self.spans = model, spans
        self.wrapper = DDP(model, group, overlap=job.strategy != "ddp-nooverlap")
        self.opt = adamw(model.parameters())
        self.shard = (group.rank, group.size)

    def train_step(self, x, y):
        with self.spans.span("forward"):
            loss = self.wrapper(x, y)
        with self.spans.span("backward"):
            loss.backward()
        with self.spans.span("optimizer"):
            self.opt.step()
            self.opt.zero_grad()
        return loss

    def weights(self):
        return to_host(self.model.parameters())


class Sharded:
    """ZeRO-1/2 and FSDP: the wrapper owns the sharded AdamW."""

    def __init__(self, model, group, job, spans):
        self.model, self.spans = model, spans
        opt = ShardedAdamW(lr=LEARNING_RATE, weight_decay=WEIGHT_DECAY, fused=False if job.deterministic else None)
        stage = int(job.strategy[-1])
        self.wrapper = FSDP(model, group, opt) if stage == 3 else ZeRO(model, group, stage, opt)
        self.stage = stage
        self.shard = (group.rank, group.size)

    def train_step(self, x, y):
        with self.spans.span("forward"):
            loss = self.wrapper(x, y)
        with self.spans.span("backward"):
            loss.backward()
        with self.spans.span("optimizer"):
            self.wrapper.step()
            self.wrapper.zero_grad()
        return loss

    def weights(self):
        if self.stage == 3:
            return self.wrapper.full_parameters().float().cpu()
        return to_host(self.model.parameters())


class Staged:
    """GPipe / 1F1B: every stage is handed the whole batch; the pipeline records its own F/B spans."""

    def __init__(self, model, group, job, spans):
        self.pipe = Pipeline(model, group, job.micro, job.strategy.split("-", 1)[1], timeline=spans)
        self.opt = adamw(self.pipe.parameters())
        self.shard = (0, 1)

    def train_step(self, x, y):
        loss = self.pipe.train_step(x, y)
        self.opt.step()
        self.opt.zero_grad()
        return loss

    def weights(self):
        return to_host(self.pipe.parameters())


def strategy_class(name):
    if name.startswith("ddp"):
        return Replicated
    if name.startswith("zero"):
        return Sharded
    if name.startswith("pp-"):
        return Staged
    raise ValueError(f"unknown strategy {name}")


def train_rank(group, job):
    """One rank of one of our strategies: losses, per-step times, peak memory, optionally weights and a profile
    of the last step."""
    device = claim_device(group.device.type, group.device.index or 0, job.deterministic)
    torch.manual_seed(0)
    corpus = synthetic(CORPUS_BYTES)
    model = GPT(job.config).to(device)
    spans = Timeline(enabled=job.profile, device=device)
    runner = strategy_class(job.strategy)(model, group, job, spans)
    rank, world = runner.shard
    if device.type == "cuda":
        torch.cuda.reset_peak_memory_stats(device)
    watch, losses = Stopwatch(device), []
    for step in range(job.steps):
        x, y = corpus.batch(step, job.rows, job.config.seq, rank=rank, world=world, device=device)
        if job.profile and step + 1 == job.steps:  # trace the last step only
            for log in (group.trace, group.waits, spans.spans):
                log.clear()
            group.tracing = True
        with watch:
            loss = runner.train_step(x, y)
        losses.append(loss.item() if loss is not None else None)
    group.tracing = False
    group._drain_spans()
    result = {"losses": losses, "times": watch.laps, "peak_mem": peak_memory(device)}
    if job.profile:
        collectives = [span for span in group.trace if span[0] != "barrier"]
        result["profile"] = summarize(spans.spans, collectives, list(group.waits), watch.laps[-1])
        result["trace"] = (spans.spans, collectives)
    if job.keep_weights:
        result["weights"] = runner.weights()
    return result


def run_ours(job, device, world):
    return launch(train_rank, world, job, device=device)


# ---------------------------------------------------------------------------------------------- baselines
def _torch_rank(rank, world, rendezvous, prefix, device_kind, job):
    import torch.distributed as dist

    device = claim_device(device_kind, rank, job.deterministic)
    backend = "nccl" if device_kind == "cuda" else "gloo"
    dist.init_process_group(backend, init_method=f"file://{rendezvous}", rank=rank, world_size=world)
    torch.manual_seed(0)
    corpus = synthetic(CORPUS_BYTES)
    model = GPT(job.config).to(device)
    sharded = job.strategy == "torch-fsdp"
    if sharded:
        from torch.distributed.fsdp import FullyShardedDataParallel as TorchFSDP
        from torch.distributed.fsdp import ShardingStrategy
        from torch.distributed.fsdp.wrap import ModuleWrapPolicy

        from .model import Block, Embed, Head

        wrapper = TorchFSDP(model, auto_wrap_policy=ModuleWrapPolicy({Embed, Block, Head}), use_orig_params=True,
                            sharding_strategy=ShardingStrategy.FULL_SHARD, device_id=device if device_kind == "cuda" else None)
    else:
        from torch.nn.parallel import DistributedDataParallel

        wrapper = DistributedDataParallel(model, device_ids=[rank] if device_kind == "cuda" else None)
    opt = adamw(wrapper.parameters())
    if device.type == "cuda":
        torch.cuda.reset_peak_memory_stats(device)
    watch, losses = Stopwatch(device), []
    for step in range(job.steps):
        x, y = corpus.batch(step, job.rows, job.config.seq, rank=rank, world=world, device=device)
        with watch:
            loss = wrapper(x, y)
            loss.backward()
            opt.step()
            opt.zero_grad()
        losses.append(loss.item())
    result = {"losses": losses, "times": watch.laps, "peak_mem": peak_memory(device)}
    if job.keep_weights:
        if sharded:
            with TorchFSDP.summon_full_params(wrapper):
                result["weights"] = to_host(model.parameters())
        else:
            result["weights"] = to_host(model.parameters())
    torch.save(result, f"{prefix}.{rank}")
    dist.destroy_process_group()


def run_torch(job, device, world):
    """torch DDP ("torch-ddp") or torch FSDP ("torch-fsdp") on `world` ranks: one result per rank."""
    with tempfile.TemporaryDirectory() as scratch:
        prefix = os.path.join(scratch, "rank")
        mp.spawn(_torch_rank, args=(world, os.path.join(scratch, "rendezvous"), prefix, device, job), nprocs=world)
        return [torch.load(f"{prefix}.{rank}", weights_only=False) for rank in range(world)]


def _alone_rank(_index, device_kind, job, path):
    device = claim_device(device_kind, 0, job.deterministic)
    torch.manual_seed(0)
    corpus = synthetic(CORPUS_BYTES)
    model = GPT(job.config).to(device)
    opt = adamw(model.parameters())
    watch, losses = Stopwatch(device), []
    for step in range(job.steps):
        x, y = corpus.batch(step, job.rows, job.config.seq, device=device)
        with watch:
            step_loss = 0
            for xs, ys in zip(x.chunk(job.micro), y.chunk(job.micro)):
                piece = loss_fn(model(xs), ys) / job.micro
                piece.backward()
                step_loss = step_loss + piece.detach()
            opt.step()
            opt.zero_grad()
        losses.append(step_loss.item())
    torch.save({"losses": losses, "times": watch.laps, "weights": to_host(model.parameters()), "peak_mem": peak_memory(device),
                "unit_sizes": [sum(p.numel() for p in unit.parameters()) for unit in model.units()]}, path)


def run_alone(job, device):
    """One process accumulating gradients over `job.micro` micro-batches per step (run in a child so that its
    device settings do not leak into this process)."""
    with tempfile.TemporaryDirectory() as scratch:
        path = os.path.join(scratch, "alone.pt")
        mp.spawn(_alone_rank, args=(device, job, path), nprocs=1)
        return torch.load(path, weights_only=False)


# ---------------------------------------------------------------------------------------------- verify
def verify(device, world):
    config = Config(seq=128, layers=4, heads=4, dim=256)
    base = Job("torch-ddp", config, steps=20, rows=16, deterministic=True, keep_weights=True)
    Rows.write(section="verify", model_params=count_params(GPT(config)), device=device, ranks=world, torch=torch.__version__)
    reference = run_torch(base, device, world)[0]

    def against_torch_ddp(name, result):
        diff = (result["weights"] - reference["weights"]).abs().max()
        Rows.write(section="verify", strategy=name, against="torch-ddp", losses_equal=result["losses"] == reference["losses"],
                   weights_equal=bool(torch.equal(result["weights"], reference["weights"])), max_weight_diff=float(diff),
                   steps=len(reference["losses"]), final_loss=result["losses"][-1])

    try:
        against_torch_ddp("torch-fsdp", run_torch(dataclasses.replace(base, strategy="torch-fsdp"), device, world)[0])
    except Exception as error:
        text = repr(error)
        last = [line for line in text.replace("\\n", "\n").splitlines() if line.strip()]
        Rows.write(section="verify", strategy="torch-fsdp", error=(last[-1] if last else text)[:300],
                   note="torch's FSDP needs an accelerator in some torch builds; the row is a cross-check of torch against itself")
    for name in ("ddp", "zero1", "zero2", "zero3"):
        against_torch_ddp(name, run_ours(dataclasses.replace(base, strategy=name), device, world)[0])

    alone = run_alone(dataclasses.replace(base, strategy="alone"), device)
    for name in ("pp-gpipe", "pp-1f1b"):
        stages = run_ours(dataclasses.replace(base, strategy=name), device, world)
        weights = torch.cat([stage["weights"] for stage in stages])
        Rows.write(section="verify", strategy=name, against="single-process accumulation", stages=world,
                   losses_equal=stages[-1]["losses"] == alone["losses"], weights_equal=bool(torch.equal(weights, alone["weights"])),
                   max_weight_diff=float((weights - alone["weights"]).abs().max()))


# ---------------------------------------------------------------------------------------------- all-reduce by size
MEGABYTES = (1, 4, 16, 64, 256)
REPEATS = 10


def _median_all_reduce(device, tensor, all_reduce, barrier):
    all_reduce(tensor)  # warm-up, and the first touch of the buffers
    laps = []
    for _ in range(REPEATS):
        barrier()
        laps.append(Stopwatch.time(device, lambda: all_reduce(tensor)))
    return statistics.median(laps)


def _ours_all_reduce_rank(group):
    device = claim_device(group.device.type, group.device.index or 0, False)
    medians = {}
    for mb in MEGABYTES:
        tensor = group.empty((mb << 20) // 4, torch.float32, device)
        tensor.fill_(1.0)
        medians[mb] = _median_all_reduce(device, tensor, group.all_reduce, group.barrier)
        group.release(tensor)
    return medians


def _torch_all_reduce_rank(rank, world, rendezvous, prefix, device_kind):
    import torch.distributed as dist

    device = claim_device(device_kind, rank, False)
    dist.init_process_group("nccl" if device_kind == "cuda" else "gloo", init_method=f"file://{rendezvous}", rank=rank, world_size=world)
    medians = {mb: _median_all_reduce(device, torch.ones((mb << 20) // 4, device=device), dist.all_reduce, dist.barrier)
               for mb in MEGABYTES}
    torch.save(medians, f"{prefix}.{rank}")
    dist.destroy_process_group()


def allreduce(device, world):
    ours = launch(_ours_all_reduce_rank, world, device=device)
    with tempfile.TemporaryDirectory() as scratch:
        prefix = os.path.join(scratch, "rank")
        mp.spawn(_torch_all_reduce_rank, args=(world, os.path.join(scratch, "rendezvous"), prefix, device), nprocs=world)
        theirs = [torch.load(f"{prefix}.{rank}") for rank in range(world)]
    library = "nccl" if device == "cuda" else "gloo"
    bus_factor = 2 * (world - 1) / world
    for mb in MEGABYTES:
        slowest_ours = max(rank[mb] for rank in ours)
        slowest_theirs = max(rank[mb] for rank in theirs)
        gigabytes = mb / 1024
        Rows.write(**{"section": "allreduce", "MB": mb, "ranks": world,
                      "ours_ms": slowest_ours * 1e3, f"{library}_ms": slowest_theirs * 1e3,
                      "ours_GBps": gigabytes / slowest_ours, f"{library}_GBps": gigabytes / slowest_theirs,
                      "ours_bus_GBps": gigabytes / slowest_ours * bus_factor, f"{library}_bus_GBps": gigabytes / slowest_theirs * bus_factor})


# ---------------------------------------------------------------------------------------------- contention
def _contention_rank(group, megabytes, repeats, gemms):
    """Device time of one all-reduce alone, then while the training stream runs GEMMs that do not depend on it."""
    device = claim_device("cuda", group.device.index or 0, False)
    message = group.empty((megabytes << 20) // 4, torch.float32, device)
    matrix = torch.randn(4096, 4096, device=device).bfloat16()

    def gemm_burst(count):
        for _ in range(count):
            matrix @ matrix

    group.all_reduce(message)
    gemm_burst(1)
    torch.cuda.synchronize()

    def all_reduce_with(gemm_count):
        """(seconds the collective ran, seconds from its launch to the end of the GEMMs and the wait)"""
        group.barrier()
        message.fill_(1.0)
        group.trace.clear()
        group.tracing = True
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        handle = group.all_reduce(message, async_op=True)
        gemm_burst(gemm_count)
        handle.wait()
        end.record()
        torch.cuda.synchronize()
        group.tracing = False
        group._drain_spans()
        _name, started, finished, _bytes = group.trace[-1]
        assert torch.equal(message, torch.full_like(message, float(group.size))), "wrong all-reduce result"
        return finished - started, begin.elapsed_time(end) / 1e3

    quiet = statistics.median(all_reduce_with(0)[0] for _ in range(repeats))
    loaded = [all_reduce_with(gemms) for _ in range(repeats)]
    gemms_only = statistics.median(Stopwatch.time(device, lambda: gemm_burst(gemms)) for _ in range(repeats))
    return {"comm_alone_ms": quiet * 1e3, "comm_busy_ms": statistics.median(ran for ran, _ in loaded) * 1e3,
            "gemms_ms": gemms_only * 1e3, "gemms_plus_comm_ms": statistics.median(total for _, total in loaded) * 1e3}


def contention(world):
    Rows.write(section="contention", gpu=torch.cuda.get_device_name(0), ranks=world)
    for priority in (0, -1):  # communication stream at normal and at high priority
        per_rank = launch(_contention_rank, world, 64, 5, 16, device="cuda", priority=priority)
        worst = {key: round(max(rank[key] for rank in per_rank), 3) for key in per_rank[0]}
        Rows.write(section="contention", priority=priority, **worst, slowdown=round(worst["comm_busy_ms"] / worst["comm_alone_ms"], 2))


# ---------------------------------------------------------------------------------------------- training matrix
def bench(device, world, preset, steps, rows, trace_path):
    config = Config.preset(preset)
    Rows.write(section="bench", model=preset, params=count_params(GPT(config)), global_batch=rows, seq=config.seq,
               device=device, ranks=world)
    tokens = rows * config.seq

    def report(name, per_rank):
        def typical(times):  # the first two steps warm up allocators and bucket order
            return statistics.median(times[2:]) if len(times) > 2 else times[-1]

        step_s = max(typical(rank["times"]) for rank in per_rank)
        final = [rank["losses"][-1] for rank in per_rank if rank["losses"][-1] is not None]
        fields = {"section": "bench", "strategy": name, "step_ms": step_s * 1e3, "tokens_per_s": tokens / step_s,
                  "peak_mem_MB": [None if rank.get("peak_mem") is None else round(rank["peak_mem"] / 2 ** 20) for rank in per_rank],
                  "final_loss": statistics.mean(final)}
        if "profile" in per_rank[0]:
            fields["profile_rank0"] = {k: (round(v, 5) if isinstance(v, float) else v) for k, v in per_rank[0]["profile"].items()}
        Rows.write(**fields)

    def attempt(name, run):
        try:
            return run()
        except Exception as error:
            Rows.write(section="bench", strategy=name, error=repr(error)[:300])
            return None

    job = Job("alone", config, steps, rows, micro=1)
    report("single", [run_alone(job, device)])
    for name in ("torch-ddp", "torch-fsdp"):
        result = attempt(name, lambda: run_torch(dataclasses.replace(job, strategy=name), device, world))
        if result is not None:
            report(name, result)
    for name in ("ddp", "ddp-nooverlap", "zero1", "zero2", "zero3", "pp-gpipe", "pp-1f1b"):
        traced = name in ("ddp", "ddp-nooverlap", "zero3")
        result = attempt(name, lambda: run_ours(dataclasses.replace(job, strategy=name, micro=4, profile=traced), device, world))
        if result is None:
            continue
        report(name, result)
        if trace_path and name == "ddp":
            chrome_trace([rank["trace"] for rank in result], trace_path)


def main():
    parser = argparse.ArgumentParser(description="verification and benchmark driver")
    parser.add_argument("what", nargs="?", default="verify", choices=["verify", "allreduce", "contention", "bench", "all"])
    parser.add_argument("--device", choices=["cuda", "cpu"], default="cuda" if torch.cuda.is_available() else "cpu")
    parser.add_argument("--ranks", type=int, default=2)
    parser.add_argument("--model", default="medium")
    parser.add_argument("--steps", type=int, default=12)
    parser.add_argument("--batch", type=int, default=16)
    parser.add_argument("--trace", default=None)
    parser.add_argument("--out", default=None)
    args = parser.parse_args()
    Rows.path = args.out
    if args.device == "cuda" and torch.cuda.device_count() < args.ranks:
        raise SystemExit(f"needs {args.ranks} GPUs, found {torch.cuda.device_count()}")
    sections = ("verify", "allreduce", "contention", "bench") if args.what == "all" else (args.what,)
    for section in sections:
        if section == "verify":
            verify(args.device, args.ranks)
        elif section == "allreduce":
            allreduce(args.device, args.ranks)
        elif section == "contention":
            if args.device == "cuda":
                contention(args.ranks)
        else:
            bench(args.device, args.ranks, args.model, args.steps, args.batch, args.trace)


if __name__ == "__main__":
    main()
