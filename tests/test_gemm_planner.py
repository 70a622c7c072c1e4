"""The GEMM planner (tile shape, how many parts the last round's tiles are cut into) is host code in the kernel
library; without a device it plans for a B200's 148 SMs, so its choices are checked here on CPU."""

import ctypes
import os

import pytest

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tandem_b200", "libtb200_cuda.so")
pytestmark = pytest.mark.skipif(not os.path.exists(LIB), reason="the kernel library has not been built")


def plan(m, n, k):
    lib = ctypes.CDLL(LIB)
    out = (ctypes.c_int * 4)()
    lib.tb_gemm_plan(m, n, k, out)
    bm, bn, parts, whole = out
    return bm, bn, parts, whole


def test_whole_rounds_are_never_split():
    for m, n, k in [(8192, 768, 3072), (8192, 3072, 768), (8192, 2304, 768), (3072, 768, 8192), (768, 768, 8192), (1024, 768, 3072)]:
        bm, bn, parts, whole = plan(m, n, k)
        tiles = -(-m // bm) * -(-n // bn)
        assert parts >= 1 and 0 <= whole <= tiles
        if parts > 1:
            tail = tiles - whole
            assert whole % 148 == 0 and 0 < tail and tail * parts <= 148  # the parts run on the SMs the last round leaves idle
            assert -(-k // 64) // parts >= 2  # every part keeps at least two k-blocks
        else:
            assert whole == 0


def test_long_reductions_with_few_tiles_are_split():
    assert plan(768, 768, 8192)[2] >= 3      # 36 tiles, 128 k-blocks: the square weight gradient
    assert plan(3072, 768, 8192)[2] == 2     # 72 tiles of 128 x 256
    assert plan(1024, 768, 3072)[2] >= 2     # 48 tiles, 48 k-blocks: one rank's share at 8 GPUs


def test_short_reductions_are_not_split():
    assert plan(1024, 768, 768)[2] == 1      # twelve k-blocks: folding would cost more than it saves
    assert plan(8192, 3072, 768)[:3] == (128, 256, 1) or plan(8192, 3072, 768)[2] <= 2


def test_narrow_outputs_get_narrow_tiles():
    assert plan(8192, 128, 768)[1] == 128
