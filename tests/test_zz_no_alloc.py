"""tsm_block_matmul_static against tsm_block_matmul and against the CPU oracle (needs a B200).

The static entry point serves hosts that must not allocate device memory during a call: its activation
scratch is a fixed array inside the library instead of a buffer grown on demand.  It has to give the very
bits of the allocating entry point and of the oracle, on call after call, because every call reuses the same
array; and it must not allocate: with the operands already on the device, neither the library's allocation
counters nor the device's free memory may move during a call.  This file is collected last, so a run that
stops at the first failure has already run every other test.
"""
import ctypes as C

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
            host = oracle.matmul_reference(kind, x, w, n, bias=bias)   # the third party: the CPU path's bits
            assert np.array_equal(bits(want), bits(host)), (kind, rows, n, k)
            assert np.array_equal(bits(got), bits(host)), (kind, rows, n, k)
            assert np.array_equal(bits(again), bits(host)), (kind, rows, n, k)
        # beyond the array's size the call is refused, not truncated
        wb = dev.tensor(oracle.quantize(oracle.Q8_0, np.zeros(32 * 8192, dtype=np.float32)))
        with pytest.raises(pkg.ShapeError, match="static scratch"):
            dev.block_matmul_static(np.zeros((129, 8192), dtype=np.float32), wb, oracle.Q8_0, 32)
    finally:
        dev.close()


@pytest.mark.parametrize("rows", [2, 24])   # the streamed kernel (at most 4 rows) and the tensor-map pipeline (5 and more)
def test_static_scratch_product_allocates_nothing(rows):
    """What the entry point is for: once the operands are on the device, a call neither asks the library's pool nor the
    driver for memory.  Checked on the library's own counters and on cudaMemGetInfo around two calls."""
    import torch
    dev = pkg.B200(0)
    rng = np.random.default_rng(22 + rows)
    kind, n, k = oracle.Q4_0, 512, 2048
    try:
        w = oracle.quantize(kind, rng.normal(0, 0.02, n * k).astype(np.float32))
        x = rng.normal(0, 1, (rows, k)).astype(np.float32)
        bias = rng.normal(0, 1, n).astype(np.float32)
        wb, xb, bb, out = dev.tensor(w), dev.tensor(x), dev.tensor(bias), dev.alloc(rows * n * 4)

        def call():
            dev.check(dev.lib.tsm_block_matmul_static(dev.ctx, C.c_uint64(xb.ptr), C.c_int(rows), C.c_int(k), C.c_int64(k), C.c_uint64(wb.ptr),
                                                      C.c_int(kind), C.c_int(n), C.c_uint64(bb.ptr), C.c_uint64(out.ptr)), "tsm_block_matmul_static")
            dev.sync()

        call()   # the first call on a device looks the array's address up and sets the kernels' attributes
        torch.cuda.synchronize()
        before, free_before = dev.counters(), torch.cuda.mem_get_info(0)[0]
        call()
        call()
        after, free_after = dev.counters(), torch.cuda.mem_get_info(0)[0]
        for name in ("allocs", "pool_misses", "pool_hits", "frees"):
            assert after[name] == before[name], name
        assert free_after == free_before
        assert after["launches"] > before["launches"]
        want = oracle.matmul_reference(kind, x, w, n, bias=bias)
        assert np.array_equal(bits(out.numpy(np.float32).reshape(rows, n)), bits(want))
    finally:
        dev.close()
