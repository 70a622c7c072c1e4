"""Numerics of the sm_100a compute kernels against plain PyTorch fp32 references
computed from the same bf16 inputs.  Tolerances are those of one bf16 rounding of
the output (2^-8 relative) plus fp32 accumulation-order noise."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def close(got, want, rtol=1.6e-2, atol=1e-2, frobenius=1.5e-2):
    """Element-wise bound (absolute part scaled by the largest entry) AND a bound on the relative Frobenius error: the
    first alone would let small entries be entirely wrong."""
    got, want = got.float(), want.float()
    err = (got - want).abs()
    tol = atol * want.abs().max().clamp_min(1e-6) + rtol * want.abs()
    assert bool((err <= tol).all()), f"max err {err.max().item():.4g} (|want| max {want.abs().max().item():.4g})"
    if want.norm().item() > 0:
        rel = (err.norm() / want.norm()).item()
        assert rel <= frobenius, f"relative Frobenius error {rel:.4g} > {frobenius}"


def gelu_slope(x):
    """d/dx of the exact GELU: Phi(x) + x * phi(x)."""
    x = x.float()
    return 0.5 * (1 + torch.erf(x * 0.7071067811865476)) + x * torch.exp(-0.5 * x * x) * 0.3989422804014327


def rnd(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


@pytest.fixture(autouse=True)
def no_gemm_timeouts():
    yield
    from tandem_b200.ops.gemm import gemm_error

    torch.cuda.synchronize()
    assert not gemm_error(), "a GEMM wait ran out"


@pytest.fixture(autouse=True)
def planner_left_alone():
    """Whatever a test pins (tile shape, number of k-parts) is unpinned again when it ends, also when it fails."""
    yield
    from tandem_b200.ops._lib import lib

    lib().tb_gemm_force_tile(-1)
    lib().tb_gemm_force_splits(0)


@pytest.fixture
def force_tile():
    """Pins the GEMM's tile shape (0: 256x256, 1: 128x256, 2: 128x128, 3/4: CTA-pair 256x256 / 256x128, 5: 128x192) for one test."""
    from tandem_b200.ops._lib import lib

    yield lib().tb_gemm_force_tile
    lib().tb_gemm_force_tile(-1)


@pytest.mark.parametrize("tile", [-1, 0, 1, 2, 3, 4, 5])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 128), (256, 384, 768), (1024, 2304, 768), (512, 65, 768),
                                   (384, 768, 3072), (130, 72, 200)])
def test_gemm_three_layouts(M, N, K, tile, force_tile):
    from tandem_b200.ops._lib import empty_padded
    from tandem_b200.ops.gemm import gemm

    force_tile(tile)

    def padded(rows, cols):
        t = empty_padded(rows, cols, torch.bfloat16, "cuda")
        t.copy_(rnd(rows, cols, scale=0.5))
        return t

    a, b = padded(M, K), padded(N, K)  # forward: A K-major, B K-major
    out = gemm(a, b, M, N, K, a.stride(0), b.stride(0), False, False)
    close(out, a.float() @ b.float().t())
    bt = padded(K, N)  # dX-style: B is [K, N] with N contiguous
    out = gemm(a, bt, M, N, K, a.stride(0), bt.stride(0), False, True)
    close(out, a.float() @ bt.float())
    at = padded(K, M)  # dW-style: both MN-major
    out = gemm(at, bt, M, N, K, at.stride(0), bt.stride(0), True, True)
    close(out, at.float().t() @ bt.float())
    out32 = gemm(at, bt, M, N, K, at.stride(0), bt.stride(0), True, True, out_dtype=torch.float32)
    close(out32, at.float().t() @ bt.float(), rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("splits", [2, 3, 8])
@pytest.mark.parametrize("tile", [-1, 0, 1, 2, 5])
@pytest.mark.parametrize("M,N,K", [(768, 768, 8192), (384, 200, 2048), (130, 72, 4096), (1024, 2304, 768)])
def test_gemm_split_k(M, N, K, splits, tile, force_tile):
    """The reduction cut into parts inside one kernel: producers park fp32 partial tiles, the consumer folds them in and runs
    the epilogue.  Weight-gradient shapes (both operands MN-major) and a forward shape with bias, GELU and residual."""
    from tandem_b200.ops import gemm as G
    from tandem_b200.ops._lib import empty_padded, lib

    force_tile(tile)
    lib().tb_gemm_force_splits(splits)
    try:
        a2, b2 = empty_padded(K, M, torch.bfloat16, "cuda"), empty_padded(K, N, torch.bfloat16, "cuda")
        a2.copy_(rnd(K, M, scale=0.5)), b2.copy_(rnd(K, N, scale=0.5))
        want = a2.float().t() @ b2.float()
        out = G.gemm(a2, b2, M, N, K, a2.stride(0), b2.stride(0), True, True)
        close(out, want)
        again = G.gemm(a2, b2, M, N, K, a2.stride(0), b2.stride(0), True, True)
        assert torch.equal(out, again)  # the parts are folded in a fixed order
        acc = torch.ones_like(out)
        G.gemm(a2, b2, M, N, K, a2.stride(0), b2.stride(0), True, True, G.ACCUMULATE, out=acc)
        close(acc, want + 1)
        if N % 8 == 0:
            x, w, bias, res = rnd(M, K, scale=0.5), rnd(N, K, scale=0.5), rnd(N), rnd(M, N)
            ref = x.float() @ w.float().t() + bias.float()
            close(G.gemm(x, w, M, N, K, K, K, False, False, G.BIAS | G.RESIDUAL, bias, res), ref + res.float())
            slope = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
            act = G.gemm(x, w, M, N, K, K, K, False, False, G.BIAS | G.GELU, bias, None, slope)
            close(slope, gelu_slope(ref))
            close(act, torch.nn.functional.gelu(ref))
    finally:
        lib().tb_gemm_force_splits(0)


def test_gemm_planner_splits_where_tiles_are_few():
    import ctypes

    from tandem_b200.ops._lib import lib

    def plan(m, n, k):
        three = (ctypes.c_int * 4)()
        lib().tb_gemm_plan(m, n, k, three)
        return tuple(three)

    assert plan(768, 768, 8192)[2] > 1      # a few dozen output tiles, 128 k-blocks: the square weight gradient
    assert plan(1024, 768, 768)[2] == 1     # twelve k-blocks: folding would cost more than it saves
    bm, bn, splits, whole = plan(8192, 768, 3072)
    tiles = -(-8192 // bm) * -(-768 // bn)
    assert splits == 1 or (0 < tiles - whole and (tiles - whole) * splits <= 148)  # only the last, partial round is ever split


@pytest.mark.parametrize("tile", [-1, 1, 3, 5])
def test_gemm_epilogues(tile, force_tile):
    from tandem_b200.ops import gemm as G

    force_tile(tile)

    M, N, K = 256, 512, 384
    a, w, bias, res = rnd(M, K, scale=0.5), rnd(N, K, scale=0.5), rnd(N), rnd(M, N)
    ref = a.float() @ w.float().t() + bias.float()
    close(G.gemm(a, w, M, N, K, K, K, False, False, G.BIAS, bias), ref)
    close(G.gemm(a, w, M, N, K, K, K, False, False, G.BIAS | G.RESIDUAL, bias, res), ref + res.float())
    slope = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    act = G.gemm(a, w, M, N, K, K, K, False, False, G.BIAS | G.GELU, bias, None, slope)
    close(slope, gelu_slope(ref))  # the forward epilogue saves gelu'(pre-activation) ...
    close(act, torch.nn.functional.gelu(ref))
    x = ref.clone().requires_grad_()
    torch.nn.functional.gelu(x).sum().backward()
    close(slope, x.grad)           # ... which is autograd's derivative of the exact (erf) GELU
    close(G.gemm(a, w, M, N, K, K, K, False, False, G.DGELU, None, slope), (a.float() @ w.float().t()) * slope.float())
    acc = torch.ones(M, N, dtype=torch.float32, device="cuda")
    G.gemm(a, w, M, N, K, K, K, False, False, G.ACCUMULATE, out=acc)
    close(acc, a.float() @ w.float().t() + 1, rtol=2e-3, atol=2e-3)
    acc16 = torch.ones(M, N, dtype=torch.bfloat16, device="cuda")
    G.gemm(a, w, M, N, K, K, K, False, False, G.ACCUMULATE, out=acc16)
    close(acc16, a.float() @ w.float().t() + 1)


@pytest.mark.parametrize("N", [768, 65])
def test_linear_autograd_matches_fp32(N):
    from tandem_b200 import ops

    B, T, K = 4, 96, 256
    x, w, b = rnd(B, T, K).requires_grad_(), rnd(N, K, scale=0.1).requires_grad_(), rnd(N).requires_grad_()
    res = rnd(B, T, N).requires_grad_() if N % 8 == 0 else None
    y = ops.linear(x, w, b, residual=res)
    dy = rnd(B, T, N)
    y.backward(dy)
    xf, wf, bf = (t.detach().float().requires_grad_() for t in (x, w, b))
    yf = torch.nn.functional.linear(xf, wf, bf)
    if res is not None:
        rf = res.detach().float().requires_grad_()
        yf = yf + rf
    yf.backward(dy.float())
    close(y, yf)
    close(x.grad, xf.grad)
    close(w.grad, wf.grad)
    close(b.grad, bf.grad)
    if res is not None:
        close(res.grad, rf.grad)


def test_mlp_autograd_matches_fp32():
    from tandem_b200 import ops

    B, T, D = 2, 128, 256
    x = rnd(B, T, D).requires_grad_()
    w1, b1 = rnd(4 * D, D, scale=0.05).requires_grad_(), rnd(4 * D, scale=0.1).requires_grad_()
    w2, b2 = rnd(D, 4 * D, scale=0.05).requires_grad_(), rnd(D, scale=0.1).requires_grad_()
    res = rnd(B, T, D).requires_grad_()
    y = ops.mlp(x, w1, b1, w2, b2, res)
    dy = rnd(B, T, D)
    y.backward(dy)
    f = [t.detach().float().requires_grad_() for t in (x, w1, b1, w2, b2, res)]
    F = torch.nn.functional
    yf = f[5] + F.linear(F.gelu(F.linear(f[0], f[1], f[2])), f[3], f[4])
    yf.backward(dy.float())
    close(y, yf)
    for got, want in zip((x, w1, b1, w2, b2, res), f):
        close(got.grad, want.grad, rtol=3e-2, atol=2e-2)


@pytest.mark.parametrize("D", [256, 768, 2048])
def test_layer_norm_matches_fp32(D):
    from tandem_b200 import ops

    x, w, b = rnd(3, 100, D, scale=2).requires_grad_(), rnd(D).requires_grad_(), rnd(D).requires_grad_()
    y = ops.layer_norm(x, w, b, 1e-5)
    dy = rnd(3, 100, D)
    y.backward(dy)
    xf, wf, bf = (t.detach().float().requires_grad_() for t in (x, w, b))
    yf = torch.nn.functional.layer_norm(xf, (D,), wf, bf, 1e-5)
    yf.backward(dy.float())
    close(y, yf)
    close(x.grad, xf.grad)
    close(w.grad, wf.grad)
    close(b.grad, bf.grad)


def test_residual_layer_norm_sums_both_gradients():
    from tandem_b200 import ops

    M, D = 300, 768
    x = rnd(M, D).requires_grad_()
    w, b = (1 + rnd(D, scale=0.1)).requires_grad_(), rnd(D, scale=0.1).requires_grad_()
    xr, n = ops.residual_layer_norm(x, w, b)
    up, un = rnd(M, D), rnd(M, D)
    (xr.float() * up.float()).sum().backward(retain_graph=True)  # only the residual branch: the gradient passes through
    close(x.grad, up)
    x.grad = None
    ((xr.float() * up.float()).sum() + (n.float() * un.float()).sum()).backward()
    xf, wf, bf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_(), b.detach().float().requires_grad_()
    nf = torch.nn.functional.layer_norm(xf, (D,), wf, bf)
    ((xf * up.float()).sum() + (nf * un.float()).sum()).backward()
    close(n, nf)
    close(x.grad, xf.grad)
    close(w.grad, wf.grad, rtol=3e-2, atol=3e-2)
    close(b.grad, bf.grad, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("V", [65, 50304])
def test_cross_entropy_matches_fp32(V):
    from tandem_b200 import ops
    from tandem_b200.ops._lib import empty_padded

    rows = 300
    logits = empty_padded(rows, V, torch.bfloat16, "cuda")
    logits.copy_(rnd(rows, V, scale=3))
    ref_in = logits.detach().float().clone().requires_grad_()
    targets = torch.randint(0, V, (rows,), device="cuda")
    leaf = logits.detach().requires_grad_()
    loss = ops.cross_entropy(leaf, targets)
    want = torch.nn.functional.cross_entropy(ref_in, targets)
    (loss * 0.5).backward()
    (want * 0.5).backward()
    assert abs(loss.item() - want.item()) < 1e-4 * max(1.0, abs(want.item()))
    close(leaf.grad, ref_in.grad, rtol=2e-2, atol=1e-3)


def test_embedding_matches_fp32():
    from tandem_b200 import ops

    V, S, D, B, T = 65, 128, 256, 4, 128
    tok, pos = rnd(V, D).requires_grad_(), rnd(S, D).requires_grad_()
    idx = torch.randint(0, V, (B, T), device="cuda")
    y = ops.embedding(idx, tok, pos)
    dy = rnd(B, T, D)
    y.backward(dy)
    tf, pf = tok.detach().float().requires_grad_(), pos.detach().float().requires_grad_()
    yf = tf[idx] + pf[torch.arange(T, device="cuda")]
    yf.backward(dy.float())
    close(y, yf)
    close(tok.grad, tf.grad)
    close(pos.grad, pf.grad)


def test_gpt_on_b200_kernels_tracks_torch_path():
    """Same weights, same batch: loss and gradients of the kernel path stay within bf16 noise of the torch path."""
    from tandem_b200.model import GPT, Config

    torch.manual_seed(0)
    cfg_t = Config(vocab=65, seq=128, layers=2, heads=4, dim=256, kernels="torch")
    cfg_k = Config(vocab=65, seq=128, layers=2, heads=4, dim=256, kernels="b200")
    ref = GPT(cfg_t).cuda()
    ker = GPT(cfg_k).cuda().bfloat16()
    ker.load_state_dict({k: v.bfloat16() for k, v in ref.state_dict().items()})
    ref.load_state_dict({k: v.float() for k, v in ker.state_dict().items()})  # identical (bf16-representable) weights
    x = torch.randint(0, 65, (4, 128), device="cuda")
    y = torch.randint(0, 65, (4, 128), device="cuda")
    lk = ker(x, y)
    lk.backward()
    lr = ref(x, y)
    lr.backward()
    assert abs(lk.item() - lr.item()) < 2e-2, (lk.item(), lr.item())
    for (name, pk), (_, pr) in zip(ker.named_parameters(), ref.named_parameters()):
        g, w = pk.grad.float(), pr.grad
        denom = w.norm().clamp_min(1e-6)
        assert ((g - w).norm() / denom).item() < 6e-2, (name, ((g - w).norm() / denom).item())


def test_twenty_training_steps_track_torch_autocast():
    """Mixed precision end to end: the bf16 kernel path (bf16 parameters, fp32 master weights and moments in BucketAdamW)
    against the same model trained by torch with fp32 parameters under bf16 autocast and torch's AdamW.  Twenty steps on
    the same batches from the same initial weights: the loss curves must stay together and both must fall."""
    import tandem_b200
    from tandem_b200.data import synthetic
    from tandem_b200.ddp import DDP, BucketAdamW
    from tandem_b200.model import GPT, Config

    text = synthetic(60_000)
    shape = dict(vocab=256, seq=128, layers=3, heads=4, dim=256)
    torch.manual_seed(0)
    ref = GPT(Config(kernels="torch", **shape)).cuda()
    torch.manual_seed(0)
    ker = GPT(Config(kernels="b200", **shape)).cuda().bfloat16()
    group = tandem_b200.Group(0, 1, "cuda:0", job=f"curve{torch.randint(0, 1 << 30, (1,)).item()}")
    wrapped = DDP(ker, group, rebuild=False)
    opt_k = BucketAdamW(wrapped, lr=1e-3, weight_decay=0.1)
    opt_r = torch.optim.AdamW(ref.parameters(), lr=1e-3, weight_decay=0.1)
    ours, theirs = [], []
    for step in range(20):
        x, y = text.batch(step, 16, shape["seq"], device="cuda")
        loss = wrapped(x, y)
        loss.backward()
        opt_k.step()
        opt_k.zero_grad()
        ours.append(loss.item())
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = ref(x, y)
        loss.backward()
        opt_r.step()
        opt_r.zero_grad()
        theirs.append(loss.item())
    group.close()
    assert all(a == a for a in ours)
    assert max(abs(a - b) for a, b in zip(ours, theirs)) < 0.05, (ours, theirs)
    assert ours[-1] < ours[0] - 0.5 and theirs[-1] < theirs[0] - 0.5, (ours, theirs)


@pytest.mark.parametrize("B,T,H,hd", [(2, 128, 2, 64), (2, 512, 3, 64), (1, 256, 2, 128), (3, 1024, 2, 64), (1, 384, 2, 128), (2, 640, 1, 64),
                                      (1, 2048, 2, 128)])
@pytest.mark.parametrize("spread", [1.0, 3.0])
def test_causal_attention_matches_fp32(B, T, H, hd, spread):
    """Odd and even numbers of 128-row tiles (the forward pairs them up), both head sizes, and scores spread widely
    enough that the running maximum keeps moving (the lazy accumulator rescale in the forward kernel)."""
    from tandem_b200 import ops
    from tandem_b200.ops.attention import attention_error

    d = H * hd
    qkv = rnd(B, T, 3 * d, scale=spread).requires_grad_()
    y = ops.causal_attention(qkv, H)
    dy = rnd(B, T, d)
    y.backward(dy)
    ref = qkv.detach().float().requires_grad_()
    q, k, v = (z.view(B, T, H, hd).transpose(1, 2) for z in ref.split(d, dim=2))
    yf = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, d)
    yf.backward(dy.float())
    torch.cuda.synchronize()
    assert not attention_error(), "an attention wait ran out"
    close(y, yf, rtol=2e-2, atol=1e-2)
    close(qkv.grad, ref.grad, rtol=4e-2, atol=2e-2)
    for part in range(3):  # dq, dk and dv each on their own scale
        close(qkv.grad[..., part * d:(part + 1) * d], ref.grad[..., part * d:(part + 1) * d], rtol=4e-2, atol=2e-2, frobenius=1e-2)


def test_causal_attention_is_deterministic():
    """No atomics anywhere: two runs give the same bits."""
    from tandem_b200 import ops

    qkv = rnd(2, 512, 3 * 256).requires_grad_()
    dy = rnd(2, 512, 256)
    outs = []
    for _ in range(2):
        qkv.grad = None
        y = ops.causal_attention(qkv, 4)
        y.backward(dy)
        outs.append((y.detach().clone(), qkv.grad.clone()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


@pytest.mark.parametrize("n,rank", [(1, 0), (4, 2), (8, 7)])
def test_gemm_with_fused_weight_gather(n, rank):
    """The weight lives in `n` shards of a flat buffer (here all on this GPU, standing in for the peers'
    symmetric memory); the kernel assembles it in `full` while it multiplies."""
    from tandem_b200.ops.gemm import GatheredLinear
    from tandem_b200.parallel.symm import split_offsets

    M, N, K = 1024, 2304, 768
    before, after = 1536, 2304 + 1003
    flat = rnd(before + N * K + after, scale=0.3)
    offs = split_offsets(flat.numel(), n)
    shards = [flat[offs[q]:offs[q + 1]].clone() for q in range(n)]
    full = torch.zeros_like(flat)
    x, bias = rnd(M, K, scale=0.5), rnd(N)
    op = GatheredLinear([s.data_ptr() for s in shards], offs, rank, full, before, N, K)
    w = flat[before:before + N * K].view(N, K)
    for _ in range(2):  # the second call reuses the flags with a new epoch
        full.zero_()
        y = op(x, bias)
        close(y, x.float() @ w.float().t() + bias.float())
        assert torch.equal(full[before:before + N * K], flat[before:before + N * K])
    # the bias sits right behind the weight in the flat buffer and is fetched with it
    op2 = GatheredLinear([s.data_ptr() for s in shards], offs, rank, full, before, N, K, bias_follows=True)
    b2 = flat[before + N * K:before + N * K + N]
    for _ in range(2):
        full.zero_()
        y = op2(x, None)
        close(y, x.float() @ w.float().t() + b2.float())
        assert torch.equal(full[before:before + N * K + N], flat[before:before + N * K + N])


def optimizer_timing_rank(g, during_backward, graphed):
    """DDP on the hand-written kernels in bf16 with the replicated optimizer applied after backward or span by span
    during it; eager or replayed from a CUDA graph."""
    from tandem_b200.data import synthetic
    from tandem_b200.ddp import DDP, BucketAdamW
    from tandem_b200.model import Config, GPT
    from tandem_b200.parallel.graph import GraphedStep

    torch.manual_seed(0)
    cfg = Config(seq=128, layers=2, heads=2, dim=128, kernels="b200")
    text = synthetic(50_000)
    model = GPT(cfg).to(g.device).bfloat16()
    wrapped = DDP(model, g, bucket_bytes=128 << 10, rebuild=False)
    opt = BucketAdamW(wrapped, lr=1e-3, weight_decay=0.1, during_backward=during_backward)
    batches = [text.batch(step, 8, cfg.seq, rank=g.rank, world=g.size, device=g.device) for step in range(8)]
    losses = []
    if graphed:
        step_fn = GraphedStep(wrapped, opt, *batches[0], warmup=3)
        for x, y in batches[3:]:
            losses.append(step_fn(x, y).item())
    else:
        for k, (x, y) in enumerate([batches[0]] * 3 + batches[3:]):
            loss = wrapped(x, y)
            loss.backward()
            opt.step()
            opt.zero_grad()
            if k >= 3:
                losses.append(loss.item())
    g.check()
    return losses, torch.cat([p.detach().float().reshape(-1) for p in model.parameters()]).cpu()


def test_optimizer_during_backward_equals_optimizer_after_backward():
    from tandem_b200 import launch

    after = launch(optimizer_timing_rank, 1, False, False, device="cuda")[0]
    during = launch(optimizer_timing_rank, 1, True, False, device="cuda")[0]
    replayed = launch(optimizer_timing_rank, 1, True, True, device="cuda")[0]
    assert after[0] == during[0], (after[0], during[0])
    assert torch.equal(after[1], during[1])  # the same arithmetic on the same gradients: bit for bit
    assert after[0] == replayed[0] and torch.equal(after[1], replayed[1])
