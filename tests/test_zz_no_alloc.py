"""tsm_block_matmul_static against tsm_block_matmul (needs a B200).

The static entry point serves hosts that must not allocate device memory during a call: its activation
scratch is a fixed array inside the library instead of a buffer grown on demand.  It has to give the very
bits of the allocating entry point, on call after call, because every call reuses the same array.  This file
is collected last, so a run that stops at the first failure has already run every other test.
"""
import numpy as np
import pytest

from helpers import bits, oracle, pkg

pytestmark = pytest.mark.gpu


def test_static_scratch_product_equals_the_allocating_one_twice_in_a_row():
    dev = pkg.B200(0)
    rng = np.random.default_rng(21)
    try:
        # two calls in a row, of different shapes and formats, the second smaller than the first so that it
        # runs over whatever the first left in the array; then the first again
        cases = [(oracle.Q4_0, 3, 640, 4096), (oracle.Q8_0, 1, 96, 576), (oracle.Q4_0, 3, 640, 4096), (oracle.Q4_1, 16, 64, 2048)]
        for kind, rows, n, k in cases:
            w = oracle.quantize(kind, rng.normal(0, 0.02, n * k).astype(np.float32))
            x = rng.normal(0, 1, (rows, k)).astype(np.float32)
            bias = rng.normal(0, 1, n).astype(np.float32)
            wb = dev.tensor(w)
            want = dev.block_matmul(x, wb, kind, n, bias=bias)
            got = dev.block_matmul_static(x, wb, kind, n, bias=bias)
            again = dev.block_matmul_static(x, wb, kind, n, bias=bias)
            wb.free()
            assert np.array_equal(bits(got), bits(want)), (kind, rows, n, k)
            assert np.array_equal(bits(again), bits(want)), (kind, rows, n, k)
        # beyond the array's size the call is refused, not truncated
        wb = dev.tensor(oracle.quantize(oracle.Q8_0, np.zeros(32 * 8192, dtype=np.float32)))
        with pytest.raises(pkg.ShapeError, match="static scratch"):
            dev.block_matmul_static(np.zeros((129, 8192), dtype=np.float32), wb, oracle.Q8_0, 32)
    finally:
        dev.close()
