"""Times the tcgen05 GEMM against torch.matmul (cuBLAS) on the linear-layer
shapes of the GPT configs.  CUDA events, warm-up, L2 flushed between timed calls.

    python -m tandem_b200.ops.bench_gemm [--tokens 8192] [--dim 768]
"""

import argparse
import json

import torch

from .gemm import gemm, gemm_error


def time_ms(fn, flush, reps=10):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(reps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / reps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--dim", type=int, default=768)
    ap.add_argument("--only", default=None, help="run just the named shape (e.g. 'fc fwd'), for profiling")
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--tile", type=int, default=-1, help="force a tile shape: 0 256x256, 1 128x256, 2 128x128")
    ap.add_argument("--discard", action="store_true", help="skip the epilogue's math and stores (how much does it cost?)")
    ap.add_argument("--flags", type=int, default=0, help="extra epilogue flags (128: skip only the global stores)")
    args = ap.parse_args()
    M, d = args.tokens, args.dim
    from ._lib import lib

    lib().tb_gemm_force_tile(args.tile)
    flags = (64 if args.discard else 0) | args.flags
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    shapes = [("qkv fwd", M, 3 * d, d, False, False), ("fc fwd", M, 4 * d, d, False, False), ("out fwd", M, d, 4 * d, False, False),
              ("fc dX", M, d, 4 * d, False, True), ("fc dW", 4 * d, d, M, True, True), ("out dW", d, 4 * d, M, True, True)]
    for name, m, n, k, a_mn, b_mn in shapes:
        if args.only and name != args.only:
            continue
        a = torch.randn((k, m) if a_mn else (m, k), device="cuda").bfloat16()
        b = torch.randn((k, n) if b_mn else (n, k), device="cuda").bfloat16()
        ours = time_ms(lambda: gemm(a, b, m, n, k, a.stride(0), b.stride(0), a_mn, b_mn, flags), flush, args.reps)
        ta = a.t() if a_mn else a
        tb = b if b_mn else b.t()
        ref = time_ms(lambda: torch.matmul(ta, tb), flush, args.reps)
        flops = 2.0 * m * n * k
        print(json.dumps({"tile": args.tile, "discard": args.discard, "flags": args.flags, "gemm": name, "M": m, "N": n, "K": k, "ours_ms": round(ours, 4), "cublas_ms": round(ref, 4),
                          "ours_tflops": round(flops / ours / 1e9, 1), "cublas_tflops": round(flops / ref / 1e9, 1)}), flush=True)
    print(json.dumps({"gemm_wait_timeouts": gemm_error()}))


if __name__ == "__main__":
    main()
