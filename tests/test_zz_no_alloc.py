"""GPU: ct_matmul_f32_static, the matmul for callers that may not allocate device memory
(a plugin host with a fixed memory budget, a thread that must not stall others with a
cudaMalloc, a latency-bound loop).  Its operand planes live in a fixed 16 MiB array inside
the library, so the entry point performs no allocation at all.

The file name makes pytest collect it last: a failure here cannot hide the other tests from a
run that stops at the first failure.  The test passes both on its own in a fresh process and
after the rest of the suite.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GEMM_TOL = 1e-5  # the tolerance of the 3xTF32 contraction tests


def _rel(got, ref):
    return float(np.max(np.abs(got.astype(np.float64) - ref.astype(np.float64)))) / float(np.max(np.abs(ref)))


def test_static_matmul_matches_regular_entry_point_twice():
    from camel_b200 import _lib, tensor as T
    from camel_b200._lib import check, lib

    rng = np.random.default_rng(42)
    status = T.Tensor(_lib.I64, (1,))  # 8 bytes of device memory; the first 4 are the status word
    # calls in a row with different shapes: none may see anything of the one before.  The third
    # fills the 16 MiB exactly and takes the 128 x 256 tiles; then a width that is no multiple of
    # four (scalar stores), fewer rows than a tile, and k = 0 (the product is all zeros).
    for (m, k, n) in ((384, 300, 512), (200, 1000, 136), (4096, 256, 4096), (300, 64, 130), (100, 40, 260), (33, 0, 70)):
        a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
        b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
        ta, tb = T.from_numpy(a), T.from_numpy(b)
        want = T.matmul(ta, tb).numpy()
        T.check_async()
        out = T.Tensor(_lib.F32, (m, n))
        check(lib.ct_fill(_lib.F32, 7.0, m * n, out.ptr))
        check(lib.ct_matmul_f32_static(ta.ptr, tb.ptr, m, k, n, out.ptr, status.ptr))
        got = out.numpy()
        assert int(status.numpy()[0]) & 0xFFFFFFFF == 0, "the kernel reported a timed-out wait"
        ref = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
        if k == 0:
            assert not got.any() and not want.any()
            continue
        assert _rel(got, want) <= GEMM_TOL
        assert _rel(got, ref) <= GEMM_TOL


def test_static_matmul_rejects_oversized_shapes():
    from camel_b200 import _lib
    from camel_b200._lib import lib

    # 8 * (m + n) * roundup(k, 32) = 8 * 4096 * 1024 = 32 MiB > 16 MiB: refused before any launch
    rc = lib.ct_matmul_f32_static(C.c_void_p(256), C.c_void_p(256), 2048, 1024, 2048, C.c_void_p(256), None)
    assert rc == _lib.ERR_TOO_LARGE
    msg = lib.ct_last_error().decode()
    assert "static scratch" in msg and "ct_matmul" in msg
