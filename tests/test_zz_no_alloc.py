"""tb_col_sum_noalloc, the column-sum entry point that keeps its scratch inside the
library for callers that cannot allocate device memory (see
tandem_b200/cuda/noalloc.h).  Called here through its exported C symbol, twice in a
row on different inputs, and compared with the ordinary entry point tb_col_sum, which
takes a caller-allocated scratch.  Collected last so that a failure here cannot hide
another test's result in a run that stops at the first failure."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry_points():
    from tandem_b200.ops._lib import lib

    L = lib()
    vp, i = ctypes.c_void_p, ctypes.c_int
    L.tb_col_sum_noalloc.argtypes = [vp, i, i, i, vp, vp]
    L.tb_col_sum_noalloc.restype = i
    L.tb_noalloc_last_error.argtypes = []
    L.tb_noalloc_last_error.restype = ctypes.c_char_p
    return L


def _close(got, want, rtol=1.6e-2, atol=1e-2):
    got, want = got.float(), want.float()
    err = (got - want).abs()
    tol = atol * want.abs().max().clamp_min(1e-6) + rtol * want.abs()
    assert bool((err <= tol).all()), f"max err {err.max().item():.4g}"


def test_no_alloc_column_sum_matches_the_allocating_entry_point_twice():
    L = _entry_points()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (M, N, ld) in enumerate([(4096, 3072, 3072), (300, 65, 72), (2100, 8192, 8192)]):  # the last: exactly the widest allowed
        x = (torch.randn(M, ld, device="cuda") * (call + 1)).bfloat16()
        want = torch.empty(N, dtype=torch.bfloat16, device="cuda")
        scratch = torch.empty(32 * N, dtype=torch.float32, device="cuda")
        assert L.tb_col_sum(x.data_ptr(), M, N, ld, want.data_ptr(), scratch.data_ptr(), stream) == 0
        got = torch.full((N,), float("nan"), dtype=torch.bfloat16, device="cuda")
        before = torch.cuda.memory_allocated()
        rc = L.tb_col_sum_noalloc(x.data_ptr(), M, N, ld, got.data_ptr(), stream)
        assert rc == 0, L.tb_noalloc_last_error()
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        _close(got, want)
        _close(got, x[:, :N].float().sum(0))  # and both agree with a plain fp32 sum


def test_no_alloc_column_sum_refuses_more_columns_than_its_scratch_holds():
    L = _entry_points()
    x = torch.zeros(8, 8, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(8, dtype=torch.bfloat16, device="cuda")
    rc = L.tb_col_sum_noalloc(x.data_ptr(), 8, 8192 + 8, 8192 + 8, out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == -30
    assert b"exceeds" in L.tb_noalloc_last_error()


def test_no_alloc_column_sum_over_no_rows_is_zero():
    L = _entry_points()
    out = torch.full((24,), float("nan"), dtype=torch.bfloat16, device="cuda")
    x = torch.zeros(1, 24, dtype=torch.bfloat16, device="cuda")
    assert L.tb_col_sum_noalloc(x.data_ptr(), 0, 24, 24, out.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert bool((out == 0).all())


def test_no_alloc_calls_on_two_streams_ordered_by_an_event():
    """The documented safe pattern: calls on different streams share the one scratch array, so the second waits for
    an event recorded after the first."""
    L = _entry_points()
    a = torch.randn(3000, 512, device="cuda").bfloat16()
    b = torch.randn(2500, 768, device="cuda").bfloat16()
    out_a = torch.empty(512, dtype=torch.bfloat16, device="cuda")
    out_b = torch.empty(768, dtype=torch.bfloat16, device="cuda")
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    assert L.tb_col_sum_noalloc(a.data_ptr(), 3000, 512, 512, out_a.data_ptr(), s1.cuda_stream) == 0
    done = torch.cuda.Event()
    done.record(s1)
    s2.wait_event(done)
    assert L.tb_col_sum_noalloc(b.data_ptr(), 2500, 768, 768, out_b.data_ptr(), s2.cuda_stream) == 0
    torch.cuda.synchronize()
    _close(out_a, a.float().sum(0))
    _close(out_b, b.float().sum(0))
