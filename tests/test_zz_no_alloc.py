"""vkg_col_sum_static: the column sum for callers that must not allocate.

A host that cannot call cudaMalloc while it runs (a plugin in someone else's process,
a loop with a latency budget, code inside a stream capture) uses this entry: the
partial sums live in an array built into the library.  It must give exactly what
vkg_col_sum_det gives with caller scratch, on repeated calls that reuse the array,
and refuse shapes the array cannot hold.  Collected last on purpose.
"""

import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _up(dev, arr):
    b = dev.buffer(arr.nbytes, "cached")
    b.array(arr.dtype, arr.shape)[...] = arr
    b.flush()
    return b


def _get(b, n):
    b.invalidate()
    return b.array(np.float32, (n,)).copy()


def test_static_scratch_matches_caller_scratch_twice(dev):
    from vkgrad_b200._lib import F16, F32
    from vkgrad_b200.vk import _check
    lib, h = dev.lib, dev.handle
    rng = np.random.default_rng(11)
    # two calls in a row with different shapes and dtypes: the second reuses (and must
    # fully overwrite) whatever the first left in the built-in array
    cases = [(4096, 768, F16, np.float16, 0), (1000, 200, F32, np.float32, 1),
             (4096, 768, F16, np.float16, 1)]
    bufs = []
    try:
        for nrow, ncol, code, dt, accumulate in cases:
            g = rng.standard_normal((nrow, ncol)).astype(dt)
            bg = _up(dev, g)
            start = rng.standard_normal(ncol).astype(np.float32)
            ref_out, new_out = _up(dev, start), _up(dev, start)
            scratch = dev.buffer(lib.vkg_col_sum_scratch_floats(ncol, nrow) * 4, "device")
            bufs += [bg, ref_out, new_out, scratch]
            _check(lib.vkg_col_sum_det(h, bg.dptr, code, ref_out.dptr, scratch.dptr, ncol, nrow,
                                       accumulate), "col_sum_det")
            _check(lib.vkg_col_sum_static(h, bg.dptr, code, new_out.dptr, ncol, nrow, accumulate),
                   "col_sum_static")
            dev.sync()
            want, got = _get(ref_out, ncol), _get(new_out, ncol)
            assert np.array_equal(got, want)      # same kernels, same order: bit-identical
            base = start if accumulate else 0.0
            exact = g.astype(np.float32).sum(0) + base
            assert np.abs(got - exact).max() <= 1e-5 * max(np.abs(exact).max(), 1.0)
    finally:
        for b in bufs:
            b.destroy()


def test_static_scratch_rejects_oversize(dev):
    from vkgrad_b200._lib import F32
    lib, h = dev.lib, dev.handle
    cap = lib.vkg_col_sum_static_max_floats()
    assert cap == 1 << 20
    ncol, nrow = 4 * cap, 64     # 4M columns: even one row chunk of partials overflows the array
    assert lib.vkg_col_sum_scratch_floats(ncol, nrow) > cap
    dummy = dev.buffer(64, "device")
    try:
        assert lib.vkg_col_sum_static(h, dummy.dptr, F32, dummy.dptr, ncol, nrow, 0) != 0
        assert b"built-in" in lib.vkg_last_error()
    finally:
        dummy.destroy()
