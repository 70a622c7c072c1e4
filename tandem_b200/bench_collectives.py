"""Collective sweep: this library's GPU kernels against NCCL (torch.distributed),
all_reduce / reduce_scatter / all_gather / broadcast, fp32 and bf16, 1 KB - 1 GB.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P -m tandem_b200.bench_collectives [--max-bytes 1073741824] [--out rows.jsonl]

    python -m tandem_b200.bench_collectives --reference cpp|python --ranks N [--max-bytes ...]
        the same sweep through the UNMODIFIED reference installed under baseline/_ref (its launch(), its Group, its
        C++ or Python engine), one process per GPU started by the reference itself; rows carry "impl": "reference"

Buffers are allocated once per size (ours: Group.empty(), i.e. symmetric memory, the
way DDP buckets and ZeRO buffers are; NCCL: ordinary tensors).  Every number is
device time from CUDA events around `iters` back-to-back calls, after warm-up, max
over ranks.  For messages smaller than the L2 an L2-sized buffer is overwritten
between timed batches.  Bus bandwidth: algorithm bandwidth x 2(n-1)/n for
all-reduce, x (n-1)/n for reduce-scatter / all-gather, x 1 for broadcast (the
reference reports algorithm bandwidth: bench/run.py:347-348).
"""

import argparse
import json
import os

import torch
import torch.distributed as dist


def timed(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if flush is not None:
        flush.zero_()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def reference_rank(g, min_bytes, max_bytes, ops, dtypes):
    """Runs inside the reference's launch(): its collectives on its own transport, timed with CUDA events."""
    import torch

    n = g.size
    rows = []
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=g.device)
    sizes, b = [], min_bytes
    while b <= max_bytes:
        sizes.append(b)
        b *= 4
    for dname in dtypes:
        dtype = getattr(torch, dname)
        esz = torch.empty(0, dtype=dtype).element_size()
        for nbytes in sizes:
            numel = nbytes // esz
            if numel % n:
                continue
            iters = 50 if nbytes <= (1 << 20) else (10 if nbytes <= (64 << 20) else 3)
            x = torch.randn(numel, device=g.device).to(dtype)
            for op in ops:
                fn = {"all_reduce": lambda: g.all_reduce(x, op="avg"), "reduce_scatter": lambda: g.reduce_scatter(x),
                      "all_gather": lambda: g.all_gather(x), "broadcast": lambda: g.broadcast(x, root=0)}[op]
                factor = {"all_reduce": 2 * (n - 1) / n, "reduce_scatter": (n - 1) / n, "all_gather": (n - 1) / n, "broadcast": 1.0}[op]
                for _ in range(3):
                    fn()
                torch.cuda.synchronize(g.device)
                if nbytes < (128 << 20):
                    flush.zero_()
                g.barrier()
                a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(iters):
                    fn()
                e.record()
                torch.cuda.synchronize(g.device)
                ms = a.elapsed_time(e) / iters
                rows.append({"op": op, "dtype": dname, "bytes": nbytes, "ranks": n, "impl": "reference", "engine": g.backend,
                             "us": round(ms * 1e3, 2), "bus_GBps": round(nbytes / ms / 1e6 * factor, 1)})
            del x
    return rows


def run_reference(args):
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref = os.path.join(root, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "tandem")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/tandem is missing (reference not installed)"}))
        return
    sys.path.insert(0, ref)
    os.environ["PYTHONPATH"] = ref + os.pathsep + root + os.pathsep + os.environ.get("PYTHONPATH", "")
    import tandem

    try:
        per_rank = tandem.launch(reference_rank, args.ranks, args.min_bytes, args.max_bytes, args.ops.split(","), args.dtypes.split(","),
                                 device="cuda", backend=args.reference)
    except Exception as e:
        print(json.dumps({"impl": "reference", "engine": args.reference, "unavailable": f"the reference failed to run: {repr(e)[:300]}"}))
        return
    rows = []
    for k, row in enumerate(per_rank[0]):  # device time, max over ranks
        row = dict(row)
        row["us"] = max(r[k]["us"] for r in per_rank)
        row["bus_GBps"] = min(r[k]["bus_GBps"] for r in per_rank)
        rows.append(row)
        print(json.dumps(row), flush=True)
    if args.out:
        with open(args.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None, choices=["cpp", "python"], help="sweep the reference's engine instead (no torchrun)")
    ap.add_argument("--ranks", type=int, default=2, help="with --reference: how many GPUs")
    ap.add_argument("--min-bytes", type=int, default=1 << 10)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--ops", default="all_reduce,reduce_scatter,all_gather,broadcast")
    ap.add_argument("--dtypes", default="float32,bfloat16")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    if args.reference:
        run_reference(args)
        return
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    os.environ.setdefault("TANDEM_SYMM_BYTES", str(max(args.max_bytes + (128 << 20), 1 << 30)))
    from tandem_b200 import Group

    g = Group.from_env(device="cuda")
    flush = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")
    n = world
    rows = []
    sizes = []
    b = args.min_bytes
    while b <= args.max_bytes:
        sizes.append(b)
        b *= 4
    for dname in args.dtypes.split(","):
        dtype = getattr(torch, dname)
        esz = torch.empty(0, dtype=dtype).element_size()
        for nbytes in sizes:
            numel = nbytes // esz
            iters = 200 if nbytes <= (1 << 20) else (50 if nbytes <= (64 << 20) else 10)
            mine = g.empty(numel, dtype)
            mine.normal_()
            theirs = torch.randn(numel, device="cuda").to(dtype)
            chunk = torch.empty(numel // n, device="cuda", dtype=dtype)
            fl = flush if nbytes < (128 << 20) else None
            for op in args.ops.split(","):
                if op == "all_reduce":
                    ours = lambda: g.all_reduce(mine, op="avg")
                    nccl = lambda: dist.all_reduce(theirs, op=dist.ReduceOp.AVG)
                    factor = 2 * (n - 1) / n
                elif op == "reduce_scatter":
                    if numel % n:
                        continue
                    ours = lambda: g.reduce_scatter(mine)
                    nccl = lambda: dist.reduce_scatter_tensor(chunk, theirs)
                    factor = (n - 1) / n
                elif op == "all_gather":
                    if numel % n:
                        continue
                    ours = lambda: g.all_gather(mine)
                    nccl = lambda: dist.all_gather_into_tensor(theirs, chunk)
                    factor = (n - 1) / n
                elif op == "reduce_scatter_adamw":
                    # the fused form DDP's sharded optimizer and ZeRO use: bf16 gradients averaged over the ranks, AdamW on
                    # this rank's chunk (fp32 master weights and moments, bf16 shadow) inside the same kernel.  The NCCL
                    # column is the unfused sequence: reduce-scatter, then torch's fused AdamW on an fp32 copy of the chunk.
                    if numel % n or dtype != torch.bfloat16:
                        continue
                    from tandem_b200.parallel.symm import AdamArgs

                    per = numel // n
                    p32, m32, v32 = (torch.zeros(per, device="cuda") for _ in range(3))
                    shadow = torch.zeros(per, device="cuda", dtype=torch.bfloat16)
                    args_ = AdamArgs.make(p32, m32, v32, (1 - 3e-5, 0.1, 0.999, 0.001, 0.0316, 1e-8, -3e-4), True, shadow)
                    ours = lambda: g.reduce_scatter(mine, op="avg", adam=args_)
                    q32 = torch.zeros(per, device="cuda", requires_grad=True)
                    opt = torch.optim.AdamW([q32], lr=3e-4, weight_decay=0.1, fused=True)

                    def nccl():
                        dist.reduce_scatter_tensor(chunk, theirs, op=dist.ReduceOp.AVG)
                        q32.grad = chunk.float()
                        opt.step()
                        shadow.copy_(q32.detach())

                    factor = (n - 1) / n
                else:
                    ours = lambda: g.broadcast(mine, root=0)
                    nccl = lambda: dist.broadcast(theirs, 0)
                    factor = 1.0
                t_ours = timed(ours, iters, 5, fl)
                t_nccl = timed(nccl, iters, 5, fl)
                row = {"op": op, "dtype": dname, "bytes": nbytes, "ranks": n, "ours_us": round(t_ours * 1e3, 2),
                       "nccl_us": round(t_nccl * 1e3, 2), "ours_bus_GBps": round(nbytes / t_ours / 1e6 * factor, 1),
                       "nccl_bus_GBps": round(nbytes / t_nccl / 1e6 * factor, 1), "ratio": round(t_nccl / t_ours, 3)}
                if op == "reduce_scatter_adamw":
                    # what the fused kernel cannot beat: this GPU's links carry (n-1)/n of the buffer (measured peer
                    # bandwidth 770 GB/s per direction), its HBM the chunk's optimizer state twice and the operands once
                    link_us = nbytes * (n - 1) / n / 770e3
                    hbm_us = (nbytes + (numel // n) * (4 * 3 * 2 + 2)) / 6552e3
                    row["roofline_us"] = round(max(link_us, hbm_us), 2)
                    row["fraction_of_roofline"] = round(max(link_us, hbm_us) / (t_ours * 1e3), 3)
                rows.append(row)
                if rank == 0:
                    print(json.dumps(row), flush=True)
            g.release(mine)
            del theirs, chunk
    g.check()
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    g.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
