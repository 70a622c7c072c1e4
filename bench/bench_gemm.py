"""Times the tcgen05 GEMM against torch.matmul (cuBLAS) on the twelve linear-layer shapes of a GPT block
(forward, input gradient, weight gradient of qkv / proj / fc / out).

Each measurement replays a CUDA graph of `reps` x [write a buffer larger than L2, GEMM] and subtracts the
same graph without the GEMM, so neither Python dispatch nor warm caches flatter the number.

    python bench/bench_gemm.py [--tokens 8192] [--dim 768]            planned tile and split count vs cuBLAS
    python bench/bench_gemm.py --sweep [--tokens 1024]                 every tile shape x split count, best and planned
"""

import argparse
import ctypes
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from tandem_b200.ops._lib import lib
from tandem_b200.ops.gemm import gemm, gemm_error

TILES = {0: "256x256", 1: "128x256", 2: "128x128", 5: "128x192", 3: "pair 256x256", 4: "pair 256x128"}


def graph_us(fn, flush, reps=8):
    """Device time of one fn() in microseconds, L2 flushed before each call."""
    def build(with_fn):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                flush.zero_()
                if with_fn:
                    fn()
        return g

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    both, base = build(True), build(False)

    def run(g):
        g.replay()
        torch.cuda.synchronize()
        best = 1e30
        for _ in range(3):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            best = min(best, a.elapsed_time(b))
        return best

    return (run(both) - run(base)) / reps * 1e3


def block_shapes(M, d):
    out = []
    for name, n, k in (("qkv", 3 * d, d), ("proj", d, d), ("fc", 4 * d, d), ("out", d, 4 * d)):
        out.append((f"{name} fwd", M, n, k, False, False))
        out.append((f"{name} dX", M, k, n, False, True))
        out.append((f"{name} dW", n, k, M, True, True))
    return out


def planned(m, n, k):
    three = (ctypes.c_int * 4)()
    lib().tb_gemm_plan(m, n, k, three)
    return {"tile": f"{'pair ' if three[0] == 512 else ''}{256 if three[0] == 512 else three[0]}x{three[1]}", "splits": three[2]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--dim", type=int, default=768)
    ap.add_argument("--only", default=None, help="run just the named shape (e.g. 'fc fwd')")
    ap.add_argument("--reps", type=int, default=8)
    ap.add_argument("--tile", type=int, default=-1, help="pin a tile shape: " + ", ".join(f"{k} {v}" for k, v in TILES.items()))
    ap.add_argument("--splits", type=int, default=0, help="pin the number of k-parts")
    ap.add_argument("--sweep", action="store_true", help="try every tile shape and split count")
    args = ap.parse_args()
    flush = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")
    L = lib()
    total_ours = total_ref = 0.0
    for name, m, n, k, a_mn, b_mn in block_shapes(args.tokens, args.dim):
        if args.only and name != args.only:
            continue
        a = torch.randn((k, m) if a_mn else (m, k), device="cuda").bfloat16()
        b = torch.randn((k, n) if b_mn else (n, k), device="cuda").bfloat16()
        run = lambda: gemm(a, b, m, n, k, a.stride(0), b.stride(0), a_mn, b_mn)
        ta, tb = (a.t() if a_mn else a), (b if b_mn else b.t())
        ref = graph_us(lambda: torch.matmul(ta, tb), flush, args.reps)
        row = {"gemm": name, "M": m, "N": n, "K": k, "cublas_us": round(ref, 1)}
        if args.sweep:
            table = {}
            for tile in (1, 2, 5, 0, 3):
                for splits in ((1,) if tile == 3 else (1, 2, 3, 4, 6, 8)):
                    L.tb_gemm_force_tile(tile)
                    L.tb_gemm_force_splits(splits)
                    got = planned(m, n, k)
                    if got["splits"] != splits:
                        continue  # no partial last round, or the reduction is too short for that many parts
                    table[f"{TILES[tile]}/{splits}"] = round(graph_us(run, flush, args.reps), 1)
            L.tb_gemm_force_tile(-1)
            L.tb_gemm_force_splits(0)
            best = min(table, key=table.get)
            row.update(best=best, best_us=table[best], table=table)
        else:
            L.tb_gemm_force_tile(args.tile)
            L.tb_gemm_force_splits(args.splits)
        plan = planned(m, n, k)
        ours = graph_us(run, flush, args.reps)
        flops = 2.0 * m * n * k
        row.update(planned=f"{plan['tile']}/{plan['splits']}", ours_us=round(ours, 1), ours_tflops=round(flops / ours / 1e6, 1),
                   cublas_tflops=round(flops / ref / 1e6, 1), vs_cublas=round(ref / ours, 3))
        total_ours += ours
        total_ref += ref
        print(json.dumps(row), flush=True)
    L.tb_gemm_force_tile(-1)
    L.tb_gemm_force_splits(0)
    print(json.dumps({"tokens": args.tokens, "dim": args.dim, "sum_ours_us": round(total_ours, 1), "sum_cublas_us": round(total_ref, 1),
                      "gemm_wait_timeouts": gemm_error()}))


if __name__ == "__main__":
    main()
