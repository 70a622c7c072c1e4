"""All-reduce latency with the whole group on ONE device, 64 KB - 64 MB, median of 20: the counterpart of the
reference's bench/engine_one_gpu.py:1-57 (two ranks sharing GPU 0).

Two ranks that share a GPU cannot use the collective kernels as separate processes (kernels of different
ranks wait on one another, and nothing makes two processes' launches run at the same time), so this prints:

  host_ms      two processes on the device, staged through pinned host memory and the native CPU runtime
               (what Group does by itself when ranks share a GPU);
  kernel_ms    the same two ranks' buffers on the device reduced by ONE cooperative launch of the all-reduce
               kernel (parallel.symm.EmulatedRanks), i.e. the kernel path without the second process.

    python -m tandem_b200.bench_one_gpu [--device cuda|cpu]
"""

import argparse
import json
import statistics
import time

import torch

SIZES_KB = [64, 256, 1024, 4096, 16384, 65536]


def staged_rank(g, reps):
    dev = g.device
    out = {}
    for kb in SIZES_KB:
        x = torch.ones(kb * 1024 // 4, device=dev)
        g.all_reduce(x)
        ts = []
        for _ in range(reps):
            g.barrier()
            if dev.type == "cuda":
                torch.cuda.synchronize(dev)
            t = time.perf_counter()
            g.all_reduce(x)
            if dev.type == "cuda":
                torch.cuda.synchronize(dev)
            ts.append(time.perf_counter() - t)
        out[kb] = statistics.median(ts)
    return out, g.transport


def kernel_times(reps):
    from .parallel.symm import EmulatedRanks

    e = EmulatedRanks(2)
    out = {}
    for kb in SIZES_KB:
        bufs = [torch.ones(kb * 1024 // 4, device="cuda") for _ in range(2)]
        e.all_reduce(bufs)
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            e.all_reduce(bufs)
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) / 1e3)
        out[kb] = statistics.median(ts)
    return out


def main():
    from . import launch

    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu", choices=["cuda", "cpu"])
    ap.add_argument("--reps", type=int, default=20)
    args = ap.parse_args()
    if args.device == "cuda":
        res = launch(staged_rank, 2, args.reps, device="cuda", gpus=[0, 0])
        kernel = kernel_times(args.reps)
        print(json.dumps({"gpu": torch.cuda.get_device_name(0), "torch": torch.__version__, "transport": res[0][1]}))
    else:
        res = launch(staged_rank, 2, args.reps, device="cpu")
        kernel = {}
        print(json.dumps({"device": "cpu", "torch": torch.__version__, "transport": res[0][1]}))
    for kb in SIZES_KB:
        host = max(r[0][kb] for r in res)
        row = {"size_KB": kb, "host_ms": round(host * 1e3, 3)}
        if kb in kernel:
            row.update(kernel_ms=round(kernel[kb] * 1e3, 3), speedup=round(host / kernel[kb], 2))
        print(json.dumps(row))


if __name__ == "__main__":
    main()
