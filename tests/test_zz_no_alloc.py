"""The allocation-free RMSNorm backward entry point against the regular one.

Some hosts may not let the library allocate (ojas charges every device byte to its Budget first); for them
ojc_rms_norm_backward_noalloc keeps its partial sums in a fixed device array. This file is collected last so a run that
stops at the first failure has already run every other test. Two calls in a row check that nothing left in the shared
array by the first call leaks into the second.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def rnd(seed, shape):
    return np.random.Generator(np.random.PCG64(seed)).standard_normal(shape, dtype=np.float32)


def test_noalloc_rms_backward_matches_the_regular_entry_point_twice_in_a_row():
    from ojas_b200 import CudaBackend
    from ojas_b200._lib import lib
    from ojas_b200.backend import _check
    be = CudaBackend(0, 4 << 30)
    try:
        for call, (rows, dim) in enumerate([(4099, 768), (1000, 64), (5000, 2048)]):   # the last one has more partial rows than the array holds: fewer, longer blocks
            x, gy = rnd(10 + call, (rows, dim)), rnd(20 + call, (rows, dim))
            w = (1.0 + 0.1 * rnd(30 + call, (dim,))).astype(np.float32)
            dx, dw, dgy = be.upload(x), be.upload(w), be.upload(gy)
            want_gx, want_gw = be.rms_norm_backward(dx, dw, dgy, 1e-6)
            gx, gw = be.empty((rows, dim)), be.empty((dim,))
            live = be.budget()["live"]
            _check(lib.ojc_rms_norm_backward_noalloc(C.c_void_p(be.stream()), C.c_void_p(dx.ptr), C.c_void_p(dw.ptr), C.c_void_p(dgy.ptr), C.c_int64(rows),
                                                     C.c_int64(dim), C.c_float(1e-6), C.c_void_p(gx.ptr), C.c_void_p(gw.ptr)))
            assert be.budget()["live"] == live  # nothing was charged or allocated by the call
            a, b = gx.numpy(), want_gx.numpy()
            assert np.array_equal(a.view(np.uint32), b.view(np.uint32))  # dX is computed row by row: same bits
            ga, gb = gw.numpy().astype(np.float64), want_gw.numpy().astype(np.float64)
            assert np.linalg.norm(ga - gb) <= 1e-4 * np.linalg.norm(gb)  # the gradient tolerance of the other GPU tests
            ogx, ogw = orc.rms_norm_backward(x, w, gy, 1e-6)            # and the CPU oracle, at the same tolerance
            assert np.linalg.norm(a.astype(np.float64) - ogx) <= 1e-4 * np.linalg.norm(ogx) and np.linalg.norm(ga - ogw) <= 1e-4 * np.linalg.norm(ogw)
        with pytest.raises(Exception) as e:  # sizes beyond the fixed workspace's reach are refused, not clamped
            _check(lib.ojc_rms_norm_backward_noalloc(C.c_void_p(be.stream()), C.c_void_p(dx.ptr), C.c_void_p(dw.ptr), C.c_void_p(dgy.ptr), C.c_int64(8),
                                                     C.c_int64(4096), C.c_float(1e-6), C.c_void_p(gx.ptr), C.c_void_p(gw.ptr)))
        assert "Unsupported" in str(e.value)
        be.sync()
    finally:
        be.close()
