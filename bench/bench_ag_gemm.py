"""All-gather -> GEMM, fused in one kernel versus done in sequence, on a ZeRO-3 style sharded weight.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench/bench_ag_gemm.py [--tokens 16384] [--dim 2048] [--out-features 6144]

Each rank owns 1/N of a flat bf16 buffer that contains the weight W[out, dim] (symmetric memory).
  fused     GatheredLinear: the GEMM kernel's fetch warps pull W from the owners while its tensor-core
            pipeline consumes the panels that have arrived (one cooperative launch)
  pull+gemm this library's pull all-gather kernel, then the plain GEMM kernel
  nccl      torch.distributed.all_gather_into_tensor + torch.matmul (cuBLAS)
Device time from CUDA events, max over ranks, L2 flushed between repetitions.  The roofline is the slower
of flops / measured bf16 peak and bytes that must cross NVLink / 770 GB/s.
"""

import os as _os
import sys as _sys

_sys.path.insert(0, _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))

import argparse
import json
import os

import torch  # noqa: E402
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--dim", type=int, default=2048)
    ap.add_argument("--out-features", type=int, default=6144)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--peak-tflops", type=float, default=1605.5)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from tandem_b200 import Group
    from tandem_b200.ops.gemm import GatheredLinear, gemm, gemm_error
    from tandem_b200.parallel.symm import split_offsets

    g = Group.from_env(device="cuda")
    M, K, N = args.tokens, args.dim, args.out_features
    numel = N * K
    offs = split_offsets(numel, world)
    torch.manual_seed(0)
    w_all = (torch.randn(numel, device="cuda") * 0.05).bfloat16()  # same on every rank (same seed)
    shard = g.empty(max(offs[q + 1] - offs[q] for q in range(world)), torch.bfloat16)
    mine = offs[rank + 1] - offs[rank]
    shard[:mine].copy_(w_all[offs[rank]:offs[rank + 1]])
    full = torch.zeros(numel, dtype=torch.bfloat16, device="cuda")
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    peers = g._sym._peers_of(shard)
    fused = GatheredLinear(peers, offs, rank, full, 0, N, K)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    g._sym.device_barrier()

    def run_fused():
        return fused(x)

    def run_seq():
        g._sym.gather_shards(full, shard[:mine], [offs[q + 1] - offs[q] for q in range(world)]).wait()
        return gemm(x, full, M, N, K, K, K, False, False)

    chunk = torch.empty(numel // world, dtype=torch.bfloat16, device="cuda") if numel % world == 0 else None
    gathered = torch.empty(numel, dtype=torch.bfloat16, device="cuda")

    def run_nccl():
        dist.all_gather_into_tensor(gathered, chunk)
        return x @ gathered.view(N, K).t()

    if chunk is not None:
        chunk.copy_(w_all[offs[rank]:offs[rank + 1]])

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(args.reps):
            flush.zero_()
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        t = torch.tensor([total / args.reps], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    want = x.float() @ w_all.view(N, K).float().t()
    err = (run_fused().float() - want).abs().max().item() / want.abs().max().item()
    t_fused, t_seq = timed(run_fused), timed(run_seq)
    t_nccl = timed(run_nccl) if chunk is not None else None
    flops = 2.0 * M * N * K
    link_bytes = numel * 2 * (world - 1) / world
    roof_ms = max(flops / (args.peak_tflops * 1e12), link_bytes / 770e9) * 1e3
    if rank == 0:
        print(json.dumps({"op": "all_gather->gemm", "ranks": world, "M": M, "N": N, "K": K, "fused_ms": round(t_fused, 4),
                          "pull_then_gemm_ms": round(t_seq, 4), "nccl_cublas_ms": None if t_nccl is None else round(t_nccl, 4),
                          "roofline_ms": round(roof_ms, 4), "fused_fraction_of_roofline": round(roof_ms / t_fused, 3),
                          "fused_tflops": round(flops / t_fused / 1e9, 1), "rel_err": err, "wait_timeouts": gemm_error()}), flush=True)
    g.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
