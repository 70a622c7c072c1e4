"""Runs ONE kernel of this library a few times on a small, fixed case, so that a profiler can capture it:

    python bench/profile_kernels.py gemm_fwd | gemm_dx | gemm_dw | attn | attn_long | adamw | layernorm |
                                               allreduce | reduce_scatter_adam | gather_gemm

Inputs are larger than the 126 MB L2 where the kernel is memory-bound, and at most a few hundred MB in
total.  The multi-rank kernels run with all ranks' buffers on this one GPU under one cooperative launch
(parallel.symm.EmulatedRanks), so the capture involves no other process.  Prints one JSON line with the
CUDA-event time of the last repetition and the algorithmic bytes / flops of the case.
"""

import os as _os
import sys as _sys

_sys.path.insert(0, _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))

import json
import sys

import torch  # noqa: E402


def run(which, reps=3):
    dev = "cuda"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def rnd(*shape, scale=0.5):
        return (torch.randn(*shape, device=dev) * scale).bfloat16()

    info = {}
    if which in ("gemm_fwd", "gemm_dx", "gemm_dw"):
        from tandem_b200.ops.gemm import BIAS, gemm

        M, N, K = 8192, 3072, 768
        if which == "gemm_fwd":
            a, b, bias = rnd(M, K), rnd(N, K), rnd(N)
            fn = lambda: gemm(a, b, M, N, K, K, K, False, False, BIAS, bias)
        elif which == "gemm_dx":
            M, N, K = 8192, 768, 3072
            a, b = rnd(M, K), rnd(K, N)
            fn = lambda: gemm(a, b, M, N, K, K, N, False, True)
        else:
            M, N, K = 3072, 768, 8192
            a, b = rnd(K, M), rnd(K, N)
            fn = lambda: gemm(a, b, M, N, K, M, N, True, True)
        info = {"flops": 2.0 * M * N * K, "bytes": 2.0 * (M * K + N * K + M * N)}
    elif which in ("attn", "attn_long"):
        from tandem_b200.ops import causal_attention

        B, T, H, hd = (16, 512, 12, 64) if which == "attn" else (8, 2048, 16, 128)  # the flagship's and the 1.3B model's shapes
        qkv = rnd(B, T, 3 * H * hd).requires_grad_()
        dy = rnd(B, T, H * hd)

        def fn():
            qkv.grad = None
            causal_attention(qkv, H).backward(dy)

        info = {"flops": 3.5 * 4.0 * B * H * T * T * hd / 2, "bytes": 2.0 * B * T * H * hd * (3 + 1 + 1 + 3)}
    elif which == "adamw":
        from tandem_b200.ops import fused_adamw

        n = 64 << 20
        p, m, v = torch.randn(n, device=dev), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        gr, sh = rnd(n, scale=0.1), torch.empty(n, dtype=torch.bfloat16, device=dev)
        sc = (1 - 3e-5, 0.1, 0.999, 0.001, 0.0316, 1e-8, -3e-3)
        fn = lambda: fused_adamw(p, gr, m, v, sc, True, sh)
        info = {"bytes": n * (4 * 3 * 2 + 2 + 2)}
    elif which == "layernorm":
        from tandem_b200.ops import layer_norm

        M, D = 65536, 768
        x, w, b = rnd(M, D).requires_grad_(), rnd(D).requires_grad_(), rnd(D).requires_grad_()
        dy = rnd(M, D)

        def fn():
            x.grad = w.grad = b.grad = None
            layer_norm(x, w, b).backward(dy)

        info = {"bytes": 2.0 * M * D * (2 + 3)}
    elif which in ("allreduce", "reduce_scatter_adam"):
        from tandem_b200.parallel.symm import AdamArgs, EmulatedRanks

        n, numel = 4, 16 << 20
        e = EmulatedRanks(n, timeout_s=5.0, max_blocks=32)
        bufs = [torch.randn(numel, device=dev) for _ in range(n)]
        if which == "allreduce":
            fn = lambda: e.all_reduce(bufs, average=True, algo="twoshot")
            info = {"bytes": 4.0 * numel * (n + n), "note": "4 ranks emulated on one GPU: reads n operands and writes n copies of each chunk"}
        else:
            per = numel // n
            ps = [torch.randn(per, device=dev) for _ in range(n)]
            ms = [torch.zeros(per, device=dev) for _ in range(n)]
            vs = [torch.zeros(per, device=dev) for _ in range(n)]
            sc = (1 - 3e-5, 0.1, 0.999, 0.001, 0.0316, 1e-8, -3e-3)
            args = [AdamArgs.make(ps[r], ms[r], vs[r], sc, True) for r in range(n)]
            fn = lambda: e.reduce_scatter(bufs, [per] * n, average=True, adam=args)
            info = {"bytes": 4.0 * numel * (n + 1) + 4.0 * numel * 6}
    elif which == "gather_gemm":
        from tandem_b200.parallel.symm import split_offsets
        from tandem_b200.ops.gemm import GatheredLinear

        n, M, N, K = 4, 8192, 6144, 2048
        flat = rnd(N * K, scale=0.1)
        offs = split_offsets(flat.numel(), n)
        shards = [flat[offs[q]:offs[q + 1]].clone() for q in range(n)]
        full = torch.zeros_like(flat)
        x = rnd(M, K)
        op = GatheredLinear([s.data_ptr() for s in shards], offs, 1, full, 0, N, K)
        fn = lambda: op(x)
        info = {"flops": 2.0 * M * N * K, "bytes": 2.0 * (M * K + 2 * N * K + M * N)}
    else:
        raise SystemExit(f"unknown kernel {which}")
    ms = 0.0
    for _ in range(reps):
        flush.zero_()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        fn()
        t1.record()
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1)
    row = {"kernel": which, "ms": round(ms, 4), **info}
    if "flops" in info:
        row["tflops"] = round(info["flops"] / ms / 1e9, 1)
    if "bytes" in info:
        row["GBps"] = round(info["bytes"] / ms / 1e6, 1)
    print(json.dumps(row), flush=True)


if __name__ == "__main__":
    run(sys.argv[1] if len(sys.argv) > 1 else "gemm_fwd")
