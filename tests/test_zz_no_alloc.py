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
    for call, (M, N, ld) in enumerate([(4096, 3072, 3072), (300, 65, 72)]):
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
