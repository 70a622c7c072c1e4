"""Out-of-bounds writes, caught on the host: every output (and scratch) buffer a kernel is handed sits between two
guard bands filled with a pattern, and the bands must come back untouched.  compute-sanitizer is not available
on the machines these tests run on, so this is the mechanical check that the kernels' tile-edge, tail and padding
logic never stores outside what it was given.  Shapes are deliberately ragged: rows and columns that are not multiples
of any tile, reductions with a tail, a vocabulary of 65, uneven shards."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

GUARD = 4096  # bytes on either side
PATTERN = 0xA5


class Guarded:
    """A tensor of `shape` carved from the middle of a larger byte buffer whose margins hold a known pattern."""

    def __init__(self, shape, dtype, row_stride=None, fill=None):
        esz = torch.empty(0, dtype=dtype).element_size()
        rows = shape[0] if len(shape) == 2 else 1
        cols = shape[-1]
        stride = row_stride or cols
        body = (rows - 1) * stride * esz + cols * esz if len(shape) == 2 else cols * esz
        body = (body + 15) // 16 * 16
        self.raw = torch.full((GUARD + body + GUARD,), PATTERN, dtype=torch.uint8, device="cuda")
        flat = self.raw[GUARD:GUARD + body].view(dtype)
        self.t = torch.as_strided(flat, shape, (stride, 1)) if len(shape) == 2 else flat[:cols]
        if fill is not None:
            self.t.copy_(fill)
        self.body = body

    def intact(self):
        torch.cuda.synchronize()
        lo, hi = self.raw[:GUARD], self.raw[GUARD + self.body:]
        return bool((lo == PATTERN).all()) and bool((hi == PATTERN).all())


def rnd(*shape, scale=0.5):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


def pad8(n):
    return (n + 7) // 8 * 8


@pytest.mark.parametrize("tile", [-1, 0, 1, 2, 5])
@pytest.mark.parametrize("M,N,K", [(130, 72, 200), (257, 264, 72), (1, 8, 64), (129, 1000, 136)])
def test_gemm_never_writes_outside_its_output(M, N, K, tile):
    from tandem_b200.ops import gemm as G
    from tandem_b200.ops._lib import lib

    lib().tb_gemm_force_tile(tile)
    try:
        a = Guarded((M, K), torch.bfloat16, pad8(K), rnd(M, K))
        w = Guarded((N, K), torch.bfloat16, pad8(K), rnd(N, K))
        bias = Guarded((N,), torch.bfloat16, fill=rnd(N))
        res = Guarded((M, N), torch.bfloat16, pad8(N), rnd(M, N))
        for flags, aux_in, want_slope in ((G.BIAS, None, False), (G.BIAS | G.RESIDUAL, res.t, False), (G.BIAS | G.GELU, None, True)):
            out = Guarded((M, N), torch.bfloat16, pad8(N))
            slope = Guarded((M, N), torch.bfloat16, pad8(N)) if want_slope else None
            G.gemm(a.t, w.t, M, N, K, pad8(K), pad8(K), False, False, flags, bias.t, aux_in, slope.t if slope else None, out=out.t)
            assert out.intact() and (slope is None or slope.intact()), (flags, "output guard bands were written")
            ref = a.t.float() @ w.t.float().t() + bias.t.float()
            if flags & G.RESIDUAL:
                ref = ref + res.t.float()
            if flags & G.GELU:
                ref = torch.nn.functional.gelu(ref)
            assert (out.t.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2
        out32 = Guarded((M, N), torch.float32, (N + 3) // 4 * 4 if N % 8 else N)
        if out32.t.stride(0) % 8 == 0:
            G.gemm(a.t, w.t, M, N, K, pad8(K), pad8(K), False, False, out=out32.t)
            assert out32.intact()
        assert a.intact() and w.intact() and bias.intact() and res.intact()
    finally:
        lib().tb_gemm_force_tile(-1)


@pytest.mark.parametrize("M,N,K,splits", [(136, 200, 1024, 2), (384, 72, 2048, 3)])
def test_split_k_stays_inside_output_and_workspace(M, N, K, splits):
    """Both operands MN-major (the weight-gradient layout), reduction cut into parts: partial tiles are parked in a
    workspace that is guarded too."""
    from tandem_b200.ops._lib import lib, stream

    L = lib()
    L.tb_gemm_force_splits(splits)
    try:
        at = Guarded((K, M), torch.bfloat16, pad8(M), rnd(K, M))
        bt = Guarded((K, N), torch.bfloat16, pad8(N), rnd(K, N))
        out = Guarded((M, N), torch.bfloat16, pad8(N))
        need = L.tb_gemm_workspace_bytes(M, N, K)
        assert need > 0
        ws = Guarded((need,), torch.uint8)
        rc = L.tb_gemm_bf16(at.t.data_ptr(), bt.t.data_ptr(), out.t.data_ptr(), M, N, K, pad8(M), pad8(N), pad8(N), 1, 1, 0, None, None, None, 0,
                            ws.t.data_ptr(), need, stream(out.t))
        assert rc == 0
        assert out.intact() and ws.intact() and at.intact() and bt.intact()
        ref = at.t.float().t() @ bt.t.float()
        assert (out.t.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2
    finally:
        L.tb_gemm_force_splits(0)


@pytest.mark.parametrize("M,D", [(37, 72), (1000, 768), (5, 2048)])
def test_layer_norm_and_column_sums_stay_inside(M, D):
    from tandem_b200.ops._lib import lib, stream

    L = lib()
    x, w, b, dy = rnd(M, D), rnd(D) + 1, rnd(D), rnd(M, D)
    y, dx = Guarded((M, D), torch.bfloat16), Guarded((M, D), torch.bfloat16)
    mean, rstd = Guarded((M,), torch.float32), Guarded((M,), torch.float32)
    dw, db = Guarded((D,), torch.bfloat16), Guarded((D,), torch.bfloat16)
    s = stream(x)
    assert L.tb_layernorm_fwd(x.data_ptr(), w.data_ptr(), b.data_ptr(), y.t.data_ptr(), mean.t.data_ptr(), rstd.t.data_ptr(), M, D, 1e-5, s) == 0
    blocks = L.tb_layernorm_bwd_blocks(M)
    scratch = Guarded((blocks * 2 * D,), torch.float32)
    assert L.tb_layernorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), mean.t.data_ptr(), rstd.t.data_ptr(), dx.t.data_ptr(), dw.t.data_ptr(),
                              db.t.data_ptr(), scratch.t.data_ptr(), M, D, s) == 0
    for g in (y, dx, mean, rstd, dw, db, scratch):
        assert g.intact()
    ref = torch.nn.functional.layer_norm(x.float(), (D,), w.float(), b.float())
    assert (y.t.float() - ref).abs().max().item() < 5e-2
    # column sums: vector path (aligned rows) and the 2-byte path (65 columns in rows of 72)
    for cols, ld in ((D, D), (65, 72)):
        src = rnd(M, ld)
        out = Guarded((cols,), torch.bfloat16)
        part = Guarded((32 * cols,), torch.float32)
        assert L.tb_col_sum(src.data_ptr(), M, cols, ld, out.t.data_ptr(), part.t.data_ptr(), s) == 0
        assert out.intact() and part.intact()
        want = src[:, :cols].float().sum(0)
        assert (out.t.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item() + 5e-2


@pytest.mark.parametrize("V", [65, 1000])
def test_cross_entropy_stays_inside_padded_rows(V):
    from tandem_b200.ops._lib import lib, stream

    L = lib()
    rows, ld = 77, pad8(V)
    logits = Guarded((rows, V), torch.bfloat16, ld, rnd(rows, V, scale=2))
    targets = torch.randint(0, V, (rows,), device="cuda")
    lse, row_loss, loss = Guarded((rows,), torch.float32), Guarded((rows,), torch.float32), Guarded((1,), torch.float32)
    s = stream(targets)
    assert L.tb_xent_fwd(logits.t.data_ptr(), targets.data_ptr(), lse.t.data_ptr(), row_loss.t.data_ptr(), loss.t.data_ptr(), rows, V, ld, s) == 0
    scale = torch.ones(1, device="cuda")
    assert L.tb_xent_bwd(logits.t.data_ptr(), targets.data_ptr(), lse.t.data_ptr(), scale.data_ptr(), rows, V, ld, V, s) == 0
    for g in (logits, lse, row_loss, loss):
        assert g.intact()


@pytest.mark.parametrize("B,T,H,hd", [(1, 128, 1, 64), (2, 384, 3, 64), (1, 256, 2, 128)])
def test_attention_stays_inside(B, T, H, hd):
    from tandem_b200.ops.attention import _fns
    from tandem_b200.ops._lib import stream

    F = _fns()
    d = H * hd
    qkv, go = rnd(B, T, 3 * d, scale=1.0), rnd(B, T, d, scale=1.0)
    out = Guarded((B * T, d), torch.bfloat16)
    lse = Guarded((B * H * T,), torch.float32)
    s = stream(qkv)
    assert F.tb_attn_fwd(qkv.data_ptr(), out.t.data_ptr(), lse.t.data_ptr(), B, T, H, hd, s) == 0
    dqkv = Guarded((B * T, 3 * d), torch.bfloat16)
    delta = Guarded((B * H * T,), torch.float32)
    assert F.tb_attn_bwd(qkv.data_ptr(), out.t.data_ptr(), go.data_ptr(), lse.t.data_ptr(), dqkv.t.data_ptr(), delta.t.data_ptr(), B, T, H, hd, s) == 0
    for g in (out, lse, dqkv, delta):
        assert g.intact()
    assert not F.tb_attn_error()
    assert bool(torch.isfinite(dqkv.t.float()).all())
