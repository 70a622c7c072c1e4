"""Multi-GPU checks (need at least 2 GPUs): the collectives over real NVLink peer
memory against locally computed values, NCCL point-to-point, and GPU training with
DDP / ZeRO-1/2 / FSDP / pipeline against torch DDP (NCCL) and single-process runs.
Integer-valued data make sums exact; training runs use deterministic torch kernels."""

import os
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu

needs2 = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
needs3 = pytest.mark.skipif(torch.cuda.device_count() < 3, reason="needs 3 GPUs")
needs4 = pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
needs8 = pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs 8 GPUs")


def data(rank, n, dtype, seed=0):
    """Rank `rank`'s integer-valued operand (the generator of the CPU collective tests)."""
    from test_comm import operand

    return operand(rank, n, dtype, salt=seed)


def gpu_collectives(g):
    r, w, dev = g.rank, g.size, g.device
    for dtype in (torch.float32, torch.bfloat16, torch.float64, torch.int64):
        for n in (0, 1, 5, 1000, 4099, 300_001):
            want = sum(data(q, n, dtype).double() for q in range(w))
            for registered in (False, True):
                x = g.empty(n, dtype) if registered else torch.empty(n, dtype=dtype, device=dev)
                x.copy_(data(r, n, dtype))
                g.all_reduce(x)
                assert torch.equal(x.double().cpu(), want), ("all_reduce", dtype, n, registered)
                if registered:
                    g.release(x)
            sizes = [n // w] * w
            sizes[-1] += n - sum(sizes)
            sizes = sizes[1:] + sizes[:1]
            lo = sum(sizes[:r])
            x = data(r, n, dtype).to(dev)
            mine = g.reduce_scatter(x, sizes)
            assert torch.equal(mine.double().cpu(), want[lo:lo + sizes[r]]), ("reduce_scatter", dtype, n)
            full = want.to(dtype)
            x = torch.full((n,), -7, dtype=dtype)
            x[lo:lo + sizes[r]] = full[lo:lo + sizes[r]]
            x = x.to(dev)
            g.all_gather(x, sizes)
            assert torch.equal(x.cpu(), full), ("all_gather", dtype, n)
            x = data(r, n, dtype, seed=1).to(dev)
            g.broadcast(x, root=w - 1)
            assert torch.equal(x.cpu(), data(w - 1, n, dtype, seed=1)), ("broadcast", dtype, n)
    x = data(r, 4097, torch.float32).to(dev)
    works = [g.all_reduce(x, op="avg", async_op=True)]
    works[0].wait()
    want = sum(data(q, 4097, torch.float32).double() for q in range(w)) / w
    assert torch.allclose(x.double().cpu(), want, rtol=0, atol=1e-5)
    # point to point over NCCL
    other = (r + 1) % w
    src = (r - 1) % w
    a = torch.arange(10_000, dtype=torch.float32, device=dev) * (r + 1)
    b = torch.empty_like(a)
    g.sendrecv(a, other, b, src)
    assert torch.equal(b.cpu(), torch.arange(10_000, dtype=torch.float32) * (src + 1))
    g.check()
    return r


def wide_reduce_scatter(g):
    """Tensors outside the heap and larger than the scratch area: staged through a block that grows on demand."""
    r, w, dev = g.rank, g.size, g.device
    for n in (600_001, 1_500_000, 700_000):
        want = sum(data(q, n, torch.float32).double() for q in range(w))
        sizes = [n // w] * w
        sizes[0] += n - sum(sizes)
        lo = sum(sizes[:r])
        for async_op in (False, True):
            x = data(r, n, torch.float32).to(dev)
            mine = g.reduce_scatter(x, sizes, async_op=async_op)
            if async_op:
                mine = mine.wait()
            assert torch.equal(mine.double().cpu(), want[lo:lo + sizes[r]]), (n, async_op)
    g.check()
    return r


@needs2
def test_reduce_scatter_of_a_tensor_larger_than_the_scratch_area(monkeypatch):
    from tandem_b200 import launch

    monkeypatch.setenv("TANDEM_SCRATCH_BYTES", str(1 << 20))
    assert launch(wide_reduce_scatter, 2, device="cuda") == [0, 1]


@needs2
def test_collectives_on_two_gpus():
    from tandem_b200 import launch

    assert launch(gpu_collectives, 2, device="cuda") == [0, 1]


@needs4
def test_collectives_on_four_gpus():
    from tandem_b200 import launch

    assert launch(gpu_collectives, 4, device="cuda") == [0, 1, 2, 3]


@needs8
def test_collectives_on_eight_gpus():
    from tandem_b200 import launch

    assert launch(gpu_collectives, 8, device="cuda") == list(range(8))


def odd_group_collectives(g):
    """A group size that is not a power of two: the kernels' predicated (runtime rank count) paths, 16-bit types
    included, and the mean as a multiply by float(1/3) per operand (what ATen's div_ by a host scalar does on CUDA).
    Behaviours of tests/test_engine_cuda.py:84-96 of the reference (world 3, n = 10,007, f32 / f16 / bf16 / int64)."""
    r, w, dev = g.rank, g.size, g.device
    n = 10_007
    for dtype in (torch.float32, torch.float16, torch.bfloat16, torch.int64):
        want = sum(data(q, n, dtype).double() for q in range(w))
        for registered in (False, True):
            x = g.empty(n, dtype) if registered else torch.empty(n, dtype=dtype, device=dev)
            x.copy_(data(r, n, dtype))
            g.all_reduce(x)
            assert torch.equal(x.double().cpu(), want), ("all_reduce", dtype, registered)
            if registered:
                g.release(x)
        sizes = [n // w] * w
        sizes[0] += n - sum(sizes)
        lo = sum(sizes[:r])
        x = data(r, n, dtype).to(dev)
        mine = g.reduce_scatter(x, sizes)
        assert torch.equal(mine.double().cpu(), want[lo:lo + sizes[r]]), ("reduce_scatter", dtype)
        x = torch.zeros(n, dtype=dtype, device=dev)
        x[lo:lo + sizes[r]] = want.to(dtype)[lo:lo + sizes[r]].to(dev)
        g.all_gather(x, sizes)
        assert torch.equal(x.cpu(), want.to(dtype)), ("all_gather", dtype)
        x = data(r, n, dtype, seed=3).to(dev)
        g.broadcast(x, root=1)
        assert torch.equal(x.cpu(), data(1, n, dtype, seed=3)), ("broadcast", dtype)
        if dtype.is_floating_point:
            x = (torch.randn(n, generator=torch.Generator().manual_seed(r)) * 3).to(dtype).to(dev)
            every = [(torch.randn(n, generator=torch.Generator().manual_seed(q)) * 3).to(dtype) for q in range(w)]
            g.all_reduce(x, op="avg")
            exact = sum(t.double() for t in every) / w
            tol = 1e-5 if dtype == torch.float32 else 2e-2
            assert torch.allclose(x.double().cpu(), exact, rtol=tol, atol=tol), ("avg", dtype)
            if dtype == torch.float32:  # bit for bit: each operand times float(1/3), folded in ring order for its chunk
                third = torch.tensor(1.0 / 3.0, dtype=torch.float32)
                chunks = [t.float() * third for t in every]
                bounds = [0]
                for q in range(w):
                    bounds.append(bounds[-1] + n // w + (1 if q < n % w else 0))
                model = torch.empty(n)
                for c in range(w):
                    a, b = bounds[c], bounds[c + 1]
                    acc = chunks[(c + 1) % w][a:b].clone()
                    for j in range(2, w + 1):
                        acc = acc + chunks[(c + j) % w][a:b]
                    model[a:b] = acc
                assert torch.equal(x.cpu(), model), "avg is not the ring-ordered sum of operands scaled by float(1/n)"
    g.check()
    return r


@needs3
def test_collectives_on_three_gpus():
    from tandem_b200 import launch

    assert launch(odd_group_collectives, 3, device="cuda") == [0, 1, 2]


# ------------------------------------------------------------------ training equality
def _setup_deterministic():
    os.environ["CUBLAS_WORKSPACE_CONFIG"] = ":4096:8"
    torch.use_deterministic_algorithms(True)
    torch.backends.cuda.enable_flash_sdp(False)
    torch.backends.cuda.enable_mem_efficient_sdp(False)
    torch.backends.cuda.matmul.allow_tf32 = False


def _cfg():
    from tandem_b200.model import Config

    return Config(seq=64, layers=2, heads=2, dim=64)


STEPS, BATCH = 5, 8


def ours_rank(g, strategy):
    from tandem_b200.data import synthetic
    from tandem_b200.ddp import DDP
    from tandem_b200.model import GPT
    from tandem_b200.optim import ShardedAdamW
    from tandem_b200.pipeline import Pipeline
    from tandem_b200.zero import FSDP, ZeRO

    _setup_deterministic()
    torch.manual_seed(0)
    cfg = _cfg()
    text = synthetic(20_000)
    model = GPT(cfg).to(g.device)
    pipe = None
    if strategy == "ddp":
        wrapped = DDP(model, g, bucket_bytes=64 << 10)
        opt = torch.optim.AdamW(model.parameters(), lr=3e-3, weight_decay=0.1, foreach=False)
    elif strategy in ("zero1", "zero2"):
        wrapped = ZeRO(model, g, int(strategy[-1]), ShardedAdamW(lr=3e-3, weight_decay=0.1, fused=False), 64 << 10)
    elif strategy == "zero3":
        wrapped = FSDP(model, g, ShardedAdamW(lr=3e-3, weight_decay=0.1, fused=False))
    else:
        pipe = Pipeline(model, g, 4, strategy)
        opt = torch.optim.AdamW(pipe.parameters(), lr=3e-3, weight_decay=0.1, foreach=False)
    losses = []
    for step in range(STEPS):
        if pipe is not None:
            x, y = text.batch(step, BATCH, cfg.seq, device=g.device)
            loss = pipe.train_step(x, y)
            opt.step()
            opt.zero_grad()
        else:
            x, y = text.batch(step, BATCH, cfg.seq, rank=g.rank, world=g.size, device=g.device)
            loss = wrapped(x, y)
            loss.backward()
            if strategy == "ddp":
                opt.step()
                opt.zero_grad()
            else:
                wrapped.step()
                wrapped.zero_grad()
        losses.append(None if loss is None else loss.item())
    if strategy == "zero3":
        w = wrapped.full_parameters().float().cpu()
    elif pipe is not None:
        w = torch.cat([p.detach().reshape(-1) for p in pipe.parameters()]).cpu()
    else:
        w = torch.cat([p.detach().reshape(-1) for p in model.parameters()]).cpu()
    g.check()
    return losses, w


def torch_ddp_rank(rank, world, init, out):
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel

    from tandem_b200.data import synthetic
    from tandem_b200.model import GPT

    torch.cuda.set_device(rank)
    _setup_deterministic()
    dist.init_process_group("nccl", init_method=f"file://{init}", rank=rank, world_size=world)
    torch.manual_seed(0)
    cfg = _cfg()
    text = synthetic(20_000)
    model = GPT(cfg).cuda()
    ddp = DistributedDataParallel(model, device_ids=[rank])
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3, weight_decay=0.1, foreach=False)
    losses = []
    for step in range(STEPS):
        x, y = text.batch(step, BATCH, cfg.seq, rank=rank, world=world, device="cuda")
        loss = ddp(x, y)
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(loss.item())
    torch.save((losses, torch.cat([p.detach().reshape(-1) for p in model.parameters()]).cpu()), f"{out}.{rank}")
    dist.destroy_process_group()


@pytest.fixture(scope="module")
def torch_ddp_2gpu():
    import torch.multiprocessing as mp

    with tempfile.TemporaryDirectory() as d:
        mp.spawn(torch_ddp_rank, args=(2, os.path.join(d, "init"), os.path.join(d, "out")), nprocs=2)
        return [torch.load(os.path.join(d, f"out.{r}")) for r in range(2)]


@needs2
@pytest.mark.parametrize("strategy", ["ddp", "zero1", "zero2", "zero3"])
def test_gpu_training_bit_identical_to_torch_ddp_nccl(strategy, torch_ddp_2gpu):
    from tandem_b200 import launch

    ours = launch(ours_rank, 2, strategy, device="cuda")
    for r in range(2):
        assert ours[r][0] == torch_ddp_2gpu[r][0], (strategy, r, ours[r][0], torch_ddp_2gpu[r][0])
        assert torch.equal(ours[r][1], torch_ddp_2gpu[r][1]), (strategy, r, (ours[r][1] - torch_ddp_2gpu[r][1]).abs().max())


def single_accumulate():
    from tandem_b200.data import synthetic
    from tandem_b200.model import GPT, loss_fn

    _setup_deterministic()
    torch.manual_seed(0)
    cfg = _cfg()
    text = synthetic(20_000)
    model = GPT(cfg).cuda()
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3, weight_decay=0.1, foreach=False)
    losses = []
    for step in range(STEPS):
        x, y = text.batch(step, BATCH, cfg.seq, device="cuda")
        total = 0
        for xb, yb in zip(x.chunk(4), y.chunk(4)):
            loss = loss_fn(model(xb), yb) / 4
            loss.backward()
            total = total + loss.detach()
        losses.append(total.item())
        opt.step()
        opt.zero_grad()
    return losses, [torch.cat([p.detach().reshape(-1) for p in u.parameters()]).cpu() for u in model.units()]


@needs2
@pytest.mark.parametrize("schedule", ["gpipe", "1f1b"])
def test_gpu_pipeline_matches_single_process_accumulation(schedule):
    from tandem_b200 import launch
    from tandem_b200.pipeline import split_units

    ours = launch(ours_rank, 2, schedule, device="cuda")
    ref_losses, ref_units = single_accumulate()
    for r, (lo, hi) in enumerate(split_units(len(ref_units), 2)):
        assert torch.equal(ours[r][1], torch.cat(ref_units[lo:hi])), f"stage {r} weights differ"
    assert ours[-1][0] == ref_losses


def fused_gather_gemm_rank(g):
    """A weight sharded over the ranks' symmetric memory, gathered by the GEMM kernel itself over NVLink."""
    from tandem_b200.ops.gemm import GatheredLinear, gemm_error
    from tandem_b200.parallel.symm import split_offsets

    torch.manual_seed(0)
    M, N, K, before = 512, 1024, 512, 1536
    flat = (torch.randn(before + N * K + 77, device=g.device) * 0.2).bfloat16()  # identical on every rank
    offs = split_offsets(flat.numel(), g.size)
    shard = g.empty(max(offs[q + 1] - offs[q] for q in range(g.size)), torch.bfloat16)
    mine = offs[g.rank + 1] - offs[g.rank]
    shard[:mine].copy_(flat[offs[g.rank]:offs[g.rank + 1]])
    g._sym.device_barrier()
    full = torch.zeros_like(flat)
    x = (torch.randn(M, K, device=g.device) * 0.5).bfloat16()
    op = GatheredLinear(g._sym._peers_of(shard), offs, g.rank, full, before, N, K)
    y = op(x)
    torch.cuda.synchronize()
    want = x.float() @ flat[before:before + N * K].view(N, K).float().t()
    ok = bool(((y.float() - want).abs() <= 2e-2 * want.abs() + 1e-2 * want.abs().max()).all())
    same = torch.equal(full[before:before + N * K], flat[before:before + N * K])
    g._sym.device_barrier()
    return ok and same and not gemm_error()


@needs2
def test_fused_gather_gemm_over_peer_memory():
    from tandem_b200 import launch

    assert launch(fused_gather_gemm_rank, 2, device="cuda") == [True, True]


def fsdp_kernel_rank(g, fuse):
    """FSDP over the hand-written kernels in bf16; with `fuse` each block's qkv GEMM gathers its own weight."""
    from tandem_b200.data import synthetic
    from tandem_b200.model import Config, GPT
    from tandem_b200.ops.gemm import GATHERED, gemm_error
    from tandem_b200.optim import ShardedAdamW
    from tandem_b200.zero import FSDP

    torch.manual_seed(0)
    cfg = Config(seq=128, layers=3, heads=4, dim=256, kernels="b200")
    text = synthetic(50_000)
    model = GPT(cfg).to(g.device).bfloat16()
    wrapped = FSDP(model, g, ShardedAdamW(lr=1e-3, weight_decay=0.1), fuse_gather_gemm=fuse)
    fused_units = sum(u.fused is not None for u in wrapped.units)
    losses = []
    for step in range(4):
        x, y = text.batch(step, 16, cfg.seq, rank=g.rank, world=g.size, device=g.device)
        loss = wrapped(x, y)
        loss.backward()
        wrapped.step()
        wrapped.zero_grad()
        losses.append(loss.item())
    w = wrapped.full_parameters().float().cpu()
    g.check()
    return losses, w, fused_units, len(GATHERED), gemm_error()


@needs2
def test_fsdp_with_qkv_weight_gathered_inside_the_gemm():
    from tandem_b200 import launch

    plain = launch(fsdp_kernel_rank, 2, False, device="cuda")
    fused = launch(fsdp_kernel_rank, 2, True, device="cuda")
    for r in range(2):
        assert plain[r][2] == 0 and fused[r][2] == 3  # one fused GEMM per block
        assert fused[r][3] == 0 and not fused[r][4]  # every registered gather was consumed; no kernel error
        assert all(l == l and l < 7 for l in fused[r][0])
        assert fused[r][0] == plain[r][0], (fused[r][0], plain[r][0])
        assert torch.equal(fused[r][1], plain[r][1]), (fused[r][1] - plain[r][1]).abs().max()


def shared_gpu_rank(g):
    x = torch.full((1000,), float(g.rank + 1), device=g.device)
    g.all_reduce(x)
    y = torch.arange(8, device=g.device, dtype=torch.float32) * (g.rank + 1)
    g.broadcast(y, root=1)
    return g.transport, g.fused, float(x[0]), float(y[7])


def test_ranks_sharing_one_gpu_stage_through_the_host():
    """Two ranks on GPU 0 (the reference's one-GPU engine benchmark layout): their collective kernels would wait on
    one another as separate launches on one GPU, so the group must fall back to host staging by itself."""
    from tandem_b200 import launch

    assert launch(shared_gpu_rank, 2, device="cuda", gpus=[0, 0]) == [("host", False, 3.0, 14.0)] * 2


def nvls_checks(g):
    """The four collectives through the NVSwitch multicast mapping (multimem.ld_reduce / multimem.st), forced on."""
    from tandem_b200.parallel.symm import ALGO

    rank, world = g.rank, g.size
    ok = True
    for dtype in (torch.float32, torch.bfloat16):
        for n in (1 << 20, 300_000 * 8):
            x = g.empty(n, dtype)
            x.copy_(data(rank, n, dtype))
            g._sym.all_reduce(x, False, x, 0, False, algo="nvls")
            want = sum(data(q, n, dtype).double() for q in range(world))
            ok = ok and torch.equal(x.double().cpu(), want)
            x.copy_(data(rank, n, dtype))
            g.all_reduce(x, op="avg")  # large enough to pick the NVLS kernel by itself where the group is large enough
            ok = ok and torch.allclose(x.double().cpu(), want / world, rtol=1e-2, atol=1e-2)
            g.release(x)
    auto, g._sym.algo = g._sym.algo, ALGO["nvls"]
    for dtype in (torch.float32, torch.bfloat16):
        n = 1 << 20
        # all-gather: each rank multicasts its own chunk (multimem.st)
        full = data(7, n, dtype)
        x = g.empty(n, dtype)
        x.fill_(-7)
        lo, hi = n * rank // world, n * (rank + 1) // world
        x[lo:hi].copy_(full[lo:hi])
        g.all_gather(x)
        ok = ok and torch.equal(x.cpu(), full)
        # reduce-scatter: the switch sums this rank's chunk (multimem.ld_reduce), with and without the accumulate epilogue
        want = sum(data(q, n, dtype).double() for q in range(world))
        x.copy_(data(rank, n, dtype))
        mine = g.reduce_scatter(x)
        ok = ok and torch.equal(mine.double().cpu(), want[lo:hi])
        x.copy_(data(rank, n, dtype))
        acc = torch.ones(hi - lo, dtype=dtype, device=g.device)
        g.reduce_scatter(x, accumulate_into=acc)
        ok = ok and torch.equal(acc.double().cpu(), want[lo:hi] + 1)
        # broadcast: the root writes once to the multicast address
        x.copy_(data(rank, n, dtype, seed=5))
        g.broadcast(x, root=world - 1)
        ok = ok and torch.equal(x.cpu(), data(world - 1, n, dtype, seed=5))
        g.release(x)
    g._sym.algo = auto
    g.check()
    return ok


def nvls_rank(rank, world, init, out):
    """A heap bound to a multicast object by torch's symmetric memory (needs a NCCL process group)."""
    import torch.distributed as dist

    from tandem_b200 import Group

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"file://{init}", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    g = Group(rank, world, f"cuda:{rank}", job=os.path.basename(init)[-12:])
    result = {"nvls": g._sym.nvls, "why": g._sym._nvls_error}
    if g._sym.nvls:
        result["ok"] = nvls_checks(g)
    g.close()
    dist.destroy_process_group()
    torch.save(result, f"{out}.{rank}")


def own_multicast_rank(g):
    """The same through this library's own set-up: launch() only, no torch.distributed anywhere."""
    sym = g._sym
    facts = {"vmm": bool(sym._vmm_segments), "nvls": sym.nvls, "why": sym._nvls_error, "peer_ok": False, "ok": False}
    try:  # a rank never leaves early: its memory stays bound to the multicast object until every rank closes
        # ordinary peer loads over the VMM mappings
        x = g.empty(100_003, torch.float32)
        x.copy_(data(g.rank, 100_003, torch.float32))
        g.all_reduce(x)
        facts["peer_ok"] = torch.equal(x.double().cpu(), sum(data(q, 100_003, torch.float32).double() for q in range(g.size)))
        g.release(x)
        if sym.nvls:
            facts["ok"] = nvls_checks(g)
    except Exception as e:
        facts["why"] = repr(e)
    return facts


@needs2
def test_own_multicast_binding_through_launch(monkeypatch):
    """cuMemCreate segments exchanged as file descriptors and bound to a multicast object by this library itself:
    the product's own launcher gets the in-switch kernels without any process group."""
    from tandem_b200 import launch

    monkeypatch.setenv("TANDEM_VMM", "1")
    res = launch(own_multicast_rank, 2, device="cuda")
    assert all(r["vmm"] for r in res), res[0]["why"]
    assert all(r["peer_ok"] for r in res)
    if not res[0]["nvls"]:
        pytest.skip(f"no NVSwitch multicast on this machine: {res[0]['why']}")
    assert all(r["ok"] for r in res)


@needs2
def test_nvls_multimem_all_reduce_and_all_gather():
    import torch.multiprocessing as mp
    import uuid

    with tempfile.TemporaryDirectory() as d:
        init = os.path.join(d, "init" + uuid.uuid4().hex[:12])
        mp.spawn(nvls_rank, args=(2, init, os.path.join(d, "out")), nprocs=2)
        res = [torch.load(os.path.join(d, f"out.{r}")) for r in range(2)]
    if not res[0]["nvls"]:
        pytest.skip(f"no NVSwitch multicast on this machine: {res[0]['why']}")
    assert all(r["ok"] for r in res)


def zero2_fused_rank(g, fused):
    from tandem_b200.data import synthetic
    from tandem_b200.model import GPT
    from tandem_b200.optim import ShardedAdamW
    from tandem_b200.zero import ZeRO

    torch.manual_seed(0)
    cfg = _cfg()
    text = synthetic(20_000)
    model = GPT(cfg).to(g.device)
    z = ZeRO(model, g, 2, ShardedAdamW(lr=3e-3, weight_decay=0.1), 64 << 10, fused_step=fused)
    losses = []
    for step in range(STEPS):
        x, y = text.batch(step, BATCH, cfg.seq, rank=g.rank, world=g.size, device=g.device)
        loss = z(x, y)
        loss.backward()
        z.step()
        z.zero_grad()
        losses.append(loss.item())
    g.check()
    return losses, torch.cat([p.detach().reshape(-1) for p in model.parameters()]).cpu()


@needs2
def test_zero2_adamw_fused_into_reduce_scatter_matches_unfused():
    from tandem_b200 import launch

    fused = launch(zero2_fused_rank, 2, True, device="cuda")
    plain = launch(zero2_fused_rank, 2, False, device="cuda")
    assert torch.equal(fused[0][1], fused[1][1])  # ranks stay in step
    for a, b in zip(fused[0][0], plain[0][0]):
        assert abs(a - b) < 1e-4, (fused[0][0], plain[0][0])
    assert torch.allclose(fused[0][1], plain[0][1], rtol=1e-5, atol=1e-6), (fused[0][1] - plain[0][1]).abs().max()


def ddp_optimizer_rank(g, sharded):
    """DDP on the torch kernels in fp32 with this library's bucket optimizers: replicated (one AdamW kernel per bucket)
    or sharded (reduce-scatter with the AdamW update in its epilogue, then all-gather of the parameters)."""
    from tandem_b200.data import synthetic
    from tandem_b200.ddp import DDP, BucketAdamW, ShardedBucketAdamW
    from tandem_b200.model import GPT

    _setup_deterministic()
    torch.manual_seed(0)
    cfg = _cfg()
    text = synthetic(20_000)
    model = GPT(cfg).to(g.device)
    wrapped = DDP(model, g, bucket_bytes=64 << 10, rebuild=False)
    opt = (ShardedBucketAdamW if sharded else BucketAdamW)(wrapped, lr=3e-3, weight_decay=0.1)
    losses = []
    for step in range(STEPS):
        x, y = text.batch(step, BATCH, cfg.seq, rank=g.rank, world=g.size, device=g.device)
        loss = wrapped(x, y)
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(loss.item())
    g.check()
    return losses, torch.cat([p.detach().reshape(-1) for p in model.parameters()]).cpu(), opt.state_bytes()


@needs2
def test_ddp_with_the_optimizer_sharded_into_the_reduce_scatter():
    from tandem_b200 import launch

    sharded = launch(ddp_optimizer_rank, 2, True, device="cuda")
    replicated = launch(ddp_optimizer_rank, 2, False, device="cuda")
    assert torch.equal(sharded[0][1], sharded[1][1])  # every rank ends with the same parameters
    assert sharded[0][0] == replicated[0][0], (sharded[0][0], replicated[0][0])
    assert torch.equal(sharded[0][1], replicated[0][1]), (sharded[0][1] - replicated[0][1]).abs().max()
    assert sharded[0][2] * 2 <= replicated[0][2] + 64  # half the optimizer state per rank


@needs2
def test_optimizer_during_backward_on_two_gpus():
    """The replicated optimizer applied span by span behind each all-reduce gives what applying it after backward gives."""
    from tandem_b200 import launch
    from test_gpu_ops import optimizer_timing_rank

    after = launch(optimizer_timing_rank, 2, False, False, device="cuda")
    during = launch(optimizer_timing_rank, 2, True, True, device="cuda")
    for r in range(2):
        assert after[r][0] == during[r][0]
        assert torch.equal(after[r][1], during[r][1])
    assert torch.equal(during[0][1], during[1][1])


def graphed_rank(g, strategy, graphed):
    """A sharded strategy on the hand-written kernels in bf16, stepped eagerly or replayed from one CUDA graph."""
    from tandem_b200.data import synthetic
    from tandem_b200.ddp import DDP, ShardedBucketAdamW
    from tandem_b200.model import Config, GPT
    from tandem_b200.optim import ShardedAdamW
    from tandem_b200.parallel.graph import GraphedStep
    from tandem_b200.zero import FSDP, ZeRO

    torch.manual_seed(0)
    cfg = Config(seq=128, layers=2, heads=2, dim=128, kernels="b200")
    text = synthetic(50_000)
    model = GPT(cfg).to(g.device).bfloat16()
    if strategy == "ddp":
        wrapped = DDP(model, g, bucket_bytes=256 << 10, rebuild=False)
        closer = ShardedBucketAdamW(wrapped, lr=1e-3, weight_decay=0.1)
    elif strategy == "zero2":
        wrapped = closer = ZeRO(model, g, 2, ShardedAdamW(lr=1e-3, weight_decay=0.1), 256 << 10, fused_step=True, capturable=graphed)
    else:
        wrapped = closer = FSDP(model, g, ShardedAdamW(lr=1e-3, weight_decay=0.1), capturable=graphed)
    batches = [text.batch(step, 8, cfg.seq, rank=g.rank, world=g.size, device=g.device) for step in range(8)]
    losses = []
    if graphed:
        step_fn = GraphedStep(wrapped, closer, *batches[0], warmup=3)  # three eager steps on batch 0, then the capture
        for x, y in batches[3:]:
            losses.append(step_fn(x, y).item())
    else:
        for k, (x, y) in enumerate([batches[0]] * 3 + batches[3:]):  # the same sequence of batches (a capture runs nothing)
            loss = wrapped(x, y)
            loss.backward()
            closer.step()
            closer.zero_grad()
            if k >= 3:
                losses.append(loss.item())
    g.check()
    return losses


@needs2
@pytest.mark.parametrize("strategy", ["ddp", "zero2", "zero3"])
def test_steps_replayed_from_a_cuda_graph_track_eager_steps(strategy):
    from tandem_b200 import launch

    eager = launch(graphed_rank, 2, strategy, False, device="cuda")
    replay = launch(graphed_rank, 2, strategy, True, device="cuda")
    for r in range(2):
        assert len(eager[r]) == len(replay[r]) == 5
        for a, b in zip(eager[r], replay[r]):
            assert a == a and abs(a - b) < 5e-3, (strategy, eager[r], replay[r])


def ddp_eight_rank(g):
    """DDP with many small spans in flight on eight GPUs; every rank must end with the same weights, and they must
    track one process that sees the whole batch (the mean over eight ranks is associated differently)."""
    from tandem_b200.data import synthetic
    from tandem_b200.ddp import DDP
    from tandem_b200.model import GPT

    _setup_deterministic()
    torch.manual_seed(0)
    cfg = _cfg()
    text = synthetic(20_000)
    model = GPT(cfg).to(g.device)
    wrapped = DDP(model, g, bucket_bytes=64 << 10)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3, weight_decay=0.1, foreach=False)
    for step in range(STEPS):
        x, y = text.batch(step, 16, cfg.seq, rank=g.rank, world=g.size, device=g.device)
        wrapped(x, y).backward()
        opt.step()
        opt.zero_grad()
    g.check()
    return torch.cat([p.detach().reshape(-1) for p in model.parameters()]).cpu()


@needs8
def test_ddp_on_eight_gpus_stays_in_step_and_tracks_one_process():
    from tandem_b200 import launch
    from tandem_b200.data import synthetic
    from tandem_b200.model import GPT

    ours = launch(ddp_eight_rank, 8, device="cuda")
    assert all(torch.equal(ours[0], ours[r]) for r in range(1, 8))
    _setup_deterministic()
    torch.manual_seed(0)
    cfg = _cfg()
    text = synthetic(20_000)
    model = GPT(cfg).cuda()
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3, weight_decay=0.1, foreach=False)
    for step in range(STEPS):
        x, y = text.batch(step, 16, cfg.seq, device="cuda")
        model(x, y).backward()
        opt.step()
        opt.zero_grad()
    alone = torch.cat([p.detach().reshape(-1) for p in model.parameters()]).cpu()
    assert torch.allclose(ours[0], alone, rtol=0, atol=5e-4), (ours[0] - alone).abs().max()
