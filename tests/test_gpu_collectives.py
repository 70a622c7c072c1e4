"""The collective kernels on one GPU: all ranks' buffers live on the device and
each collective is ONE cooperative launch whose blockIdx.y is the rank, so the
flag barriers, chunk ownership, fold order, fused divide, staging path and the
fused epilogues are exercised exactly as on several GPUs (minus NVLink).
Expected values are plain PyTorch fp32 folds in the documented order."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def expected_fold(xs, average, sizes=None, exact_dtype=None):
    """Left fold over ranks c+1, ..., c for each chunk c, operands divided first."""
    n, numel = len(xs), xs[0].numel()
    from tandem_b200.parallel.symm import split_offsets

    offs = split_offsets(numel, n, sizes)

    def prep(t):
        t = t.float()
        if average:
            t = t * (1.0 / n)  # ATen's CUDA div_ by a host scalar multiplies by the reciprocal
        return t.to(exact_dtype).float() if exact_dtype else t

    out = torch.empty(numel, dtype=torch.float32, device=xs[0].device)
    for c in range(n):
        lo, hi = offs[c], offs[c + 1]
        acc = prep(xs[(c + 1) % n][lo:hi])
        for j in range(2, n + 1):
            acc = acc + prep(xs[(c + j) % n][lo:hi])
            if exact_dtype:
                acc = acc.to(exact_dtype).float()
        out[lo:hi] = acc
    return out, offs


@pytest.fixture(scope="module")
def emu():
    from tandem_b200.parallel.symm import EmulatedRanks

    made = {}

    def get(n):
        if n not in made:
            made[n] = EmulatedRanks(n, timeout_s=5.0)
        return made[n]

    yield get
    for e in made.values():
        e.close()


@pytest.mark.parametrize("n", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("numel,algo", [(1, "auto"), (37, "oneshot"), (4099, "oneshot"), (4099, "twoshot"),
                                        (65536, "auto"), (1_000_003, "twoshot")])
def test_all_reduce_matches_ordered_fold(emu, n, dtype, numel, algo):
    e = emu(n)
    g = torch.Generator(device="cuda").manual_seed(numel + n)
    xs = [(torch.randn(numel, generator=g, device="cuda") * 3).to(dtype) for _ in range(n)]
    for average in (False, True):
        bufs = [x.clone() for x in xs]
        e.all_reduce(bufs, average=average, algo=algo)
        torch.cuda.synchronize()
        assert e.status[0] == 0
        want, _ = expected_fold(xs, average)
        want = want.to(dtype)
        for r in range(n):
            assert torch.equal(bufs[r], want), (r, average, (bufs[r].float() - want.float()).abs().max())


@pytest.mark.parametrize("n", [2, 4])
def test_all_reduce_exact16_rounds_every_partial_sum(emu, n):
    e = emu(n)
    xs = [torch.randn(10_007, device="cuda").bfloat16() for _ in range(n)]
    bufs = [x.clone() for x in xs]
    e.all_reduce(bufs, average=True, exact=True, algo="twoshot")
    want, _ = expected_fold(xs, True, exact_dtype=torch.bfloat16)
    assert torch.equal(bufs[0], want.bfloat16()) and torch.equal(bufs[0], bufs[-1])


@pytest.mark.parametrize("n", [2, 4])
@pytest.mark.parametrize("dtype", [torch.float64, torch.int64, torch.int32])
def test_all_reduce_generic_dtypes(emu, n, dtype):
    e = emu(n)
    xs = [torch.randint(-100, 100, (5003,), device="cuda").to(dtype) for _ in range(n)]
    bufs = [x.clone() for x in xs]
    e.all_reduce(bufs)
    want = sum(x.double() for x in xs).to(dtype)
    assert all(torch.equal(b, want) for b in bufs)


@pytest.mark.parametrize("n", [2, 3, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_reduce_scatter_uneven_with_accumulate(emu, n, dtype):
    e = emu(n)
    numel = 50_021
    sizes = [numel // n] * n
    sizes[-1] += numel - sum(sizes)
    sizes = sizes[1:] + sizes[:1]
    sizes[0], sizes[1] = 0, sizes[0] + sizes[1]  # one rank owns nothing
    xs = [torch.randn(numel, device="cuda").to(dtype) for _ in range(n)]
    bufs = [x.clone() for x in xs]
    shards = [torch.randn(s, device="cuda").to(dtype) for s in sizes]
    before = [s.clone() for s in shards]
    offs = e.reduce_scatter(bufs, sizes, average=True, accumulate_into=shards)
    want, _ = expected_fold(xs, True, sizes)
    for r in range(n):
        lo, hi = offs[r], offs[r + 1]
        got = bufs[r][lo:hi]
        assert torch.equal(got, want[lo:hi].to(dtype)), r
        assert torch.equal(shards[r], (before[r].float() + got.float()).to(dtype)), r


def adam_scalars(lr, betas, eps, wd, step):
    b1, b2 = betas
    return (1 - lr * wd, 1 - b1, b2, 1 - b2, (1 - b2 ** step) ** 0.5, eps, -(lr / (1 - b1 ** step)))


@pytest.mark.parametrize("n", [2, 4])
def test_reduce_scatter_with_fused_adamw_matches_torch(emu, n):
    from tandem_b200.parallel.symm import AdamArgs

    e = emu(n)
    numel = 40_000
    xs = [torch.randn(numel, device="cuda") for _ in range(n)]
    full = torch.randn(numel, device="cuda")
    ref = full.clone().requires_grad_()
    opt = torch.optim.AdamW([ref], lr=3e-3, weight_decay=0.1, foreach=False, fused=False)
    offs = [numel * r // n for r in range(n + 1)]
    sizes = [offs[r + 1] - offs[r] for r in range(n)]
    params = [full[offs[r]:offs[r + 1]].clone() for r in range(n)]
    m = [torch.zeros_like(p) for p in params]
    v = [torch.zeros_like(p) for p in params]
    shadow = [torch.zeros_like(p, dtype=torch.bfloat16) for p in params]
    worst = 0.0
    for step in range(1, 4):
        grads = [x * step for x in xs]
        bufs = [g_.clone() for g_ in grads]
        sc = adam_scalars(3e-3, (0.9, 0.999), 1e-8, 0.1, step)
        args = [AdamArgs.make(params[r], m[r], v[r], sc, True, shadow[r]) for r in range(n)]
        e.reduce_scatter(bufs, sizes, average=True, adam=args)
        want, _ = expected_fold(grads, True, sizes)
        ref.grad = want.clone()
        opt.step()
        got = torch.cat(params)
        worst = max(worst, (got - ref.detach()).abs().max().item())
        assert torch.allclose(got, ref.detach(), rtol=1e-6, atol=1e-7), worst
        assert torch.equal(torch.cat(shadow), got.bfloat16())
    print("fused reduce-scatter+AdamW vs torch AdamW: max abs diff", worst)


@pytest.mark.parametrize("n", [2, 4, 8])
def test_gather_pull_and_broadcast(emu, n):
    e = emu(n)
    sizes = [1000 + 17 * r for r in range(n)]
    offs = [0]
    for s in sizes:
        offs.append(offs[-1] + s)
    shards = [torch.randn(max(sizes), device="cuda")[:sizes[r]] * 0 + r + torch.arange(sizes[r], device="cuda") / 4096
              for r in range(n)]
    shard_bufs = [torch.zeros(max(sizes), device="cuda") for _ in range(n)]
    for r in range(n):
        shard_bufs[r][:sizes[r]] = shards[r]
    fulls = [torch.full((offs[-1],), -1.0, device="cuda") for _ in range(n)]
    e.gather(shard_bufs, fulls, [0] * n, [o * 4 for o in offs[:-1]], [s * 4 for s in sizes], sync=False)
    want = torch.cat(shards)
    assert all(torch.equal(f, want) for f in fulls)
    # in-place all-gather of a symmetric buffer, then a broadcast from the last rank
    bufs = [torch.full((offs[-1],), float(r), device="cuda") for r in range(n)]
    e.gather(bufs, bufs, [o * 4 for o in offs[:-1]], [o * 4 for o in offs[:-1]], [s * 4 for s in sizes])
    want = torch.cat([torch.full((s,), float(r), device="cuda") for r, s in enumerate(sizes)])
    assert all(torch.equal(b, want) for b in bufs)
    root = n - 1
    bufs = [torch.full((777,), float(r), device="cuda") for r in range(n)]
    e.gather(bufs, bufs, [0] * n, [0] * n, [777 * 4 if q == root else 0 for q in range(n)])
    assert all(torch.equal(b, torch.full((777,), float(root), device="cuda")) for b in bufs)


def test_wait_gives_up_and_reports_instead_of_hanging():
    """A peer that never signals: the kernel returns after its limit with a
    status the host can read, and the device stays usable."""
    from tandem_b200.parallel.symm import FLAG_BYTES, MAX_BLOCKS, _ptr_array, check_rc, cuda_lib

    lib = cuda_lib()
    mine = torch.zeros(FLAG_BYTES // 4, dtype=torch.int32, device="cuda")
    nobody = torch.zeros(FLAG_BYTES // 4, dtype=torch.int32, device="cuda")  # stands in for an absent peer's pad
    epoch = torch.zeros(MAX_BLOCKS, dtype=torch.int32, device="cuda")
    host, dev = ctypes.c_void_p(), ctypes.c_void_p()
    check_rc(lib.tb_status_alloc(ctypes.byref(host), ctypes.byref(dev), 64), "status")
    status = (ctypes.c_uint32 * 16).from_address(host.value)
    comm = lib.tb_comm_create(2, 0, 0, _ptr_array([mine.data_ptr(), nobody.data_ptr()]),
                              _ptr_array([epoch.data_ptr(), None]), dev, 0.2, 4)
    check_rc(lib.tb_barrier(comm, torch.cuda.current_stream().cuda_stream), "barrier")
    torch.cuda.synchronize()
    assert [status[k] for k in range(3)] == [1, 0, 1]  # timeout, seen by rank 0, waiting for rank 1
    assert torch.ones(4, device="cuda").sum().item() == 4.0  # the context survived
    lib.tb_comm_destroy(comm)
    lib.tb_status_free(host)


def test_multi_copy_and_fused_adamw_match_torch():
    from tandem_b200.ops import fused_adamw, pack_into

    shapes = [(7,), (128, 33), (1,), (1000, 129)] * 15  # more than one launch table
    srcs = [torch.randn(s, device="cuda") for s in shapes]
    flat = torch.zeros(sum(s.numel() for s in srcs), device="cuda")
    views, at = [], 0
    for s in srcs:
        views.append(flat[at:at + s.numel()].view_as(s))
        at += s.numel()
    pack_into(flat, list(zip(views, srcs)))
    assert torch.equal(flat, torch.cat([s.reshape(-1) for s in srcs]))

    p = torch.randn(100_003, device="cuda")
    ref = p.clone().requires_grad_()
    opt = torch.optim.AdamW([ref], lr=3e-4, weight_decay=0.1, foreach=False, fused=False)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    shadow = torch.zeros_like(p, dtype=torch.bfloat16)
    exact = True
    for step in range(1, 6):
        g = torch.randn_like(p) * 0.1
        fused_adamw(p, g, m, v, adam_scalars(3e-4, (0.9, 0.999), 1e-8, 0.1, step), True, shadow)
        ref.grad = g.clone()
        opt.step()
        assert torch.allclose(p, ref.detach(), rtol=1e-6, atol=1e-7)
        exact = exact and torch.equal(p, ref.detach())
    assert torch.equal(shadow, p.bfloat16())
    print("fused AdamW bit-identical to torch.optim.AdamW(foreach=False):", exact)
