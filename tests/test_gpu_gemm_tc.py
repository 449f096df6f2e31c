"""The tcgen05 3xTF32 tensor-core contractions against float64 and against the exact FP32 kernels.
3xTF32 keeps fp32-level accuracy (hi*hi + hi*lo + lo*hi with fp32 accumulation in tensor memory),
so the same 1e-4 bound as everywhere else applies; in practice the error is ~1e-6."""
import ctypes as C

import numpy as np
import pytest

from helpers import assert_close, max_abs_rel, rng

pytestmark = pytest.mark.gpu


def gemm(capi, ta, tb, m, n, k, a, b, c0=None, accumulate=0, lda=None, ldb=None):
    da, db = capi.to_device(a), capi.to_device(b)
    dc = capi.to_device(c0) if c0 is not None else capi.empty((m, n))
    capi.call("gemm", C.c_int(ta), C.c_int(tb), C.c_int64(m), C.c_int64(n), C.c_int64(k), da.ptr, C.c_int64(lda or a.shape[1]),
              db.ptr, C.c_int64(ldb or b.shape[1]), dc.ptr, C.c_int64(n), C.c_int(accumulate))
    code = C.c_int(0)
    capi.call("device_status", C.byref(code))
    return dc.numpy()


SHAPES = [(128, 128, 32), (128, 128, 64), (256, 128, 3136), (256, 3136, 128), (3136, 128, 256), (64, 2048, 577), (577, 2048, 64),
          (64, 577, 2048), (130, 70, 33), (257, 129, 65), (1000, 24, 200), (128, 32, 4096), (512, 512, 512), (33, 17, 2000),
          # more 128x64 tiles than the GPU has multiprocessors: the shared-memory-operand kernel takes these
          (1024, 1536, 160), (2100, 1030, 72)]


@pytest.mark.parametrize("m,n,k", SHAPES, ids=str)
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_tensor_core_gemm_matches_float64_and_fp32_path(capi, m, n, k, ta, tb):
    r = rng(m * 7 + n * 3 + k + ta * 2 + tb)
    a = r.standard_normal((k, m) if ta else (m, k)).astype(np.float32)
    b = r.standard_normal((n, k) if tb else (k, n)).astype(np.float32)
    A = (a.T if ta else a).astype(np.float64)
    B = (b.T if tb else b).astype(np.float64)
    ref = A @ B
    capi.call("set_tensor_cores", C.c_int(1))
    l0 = capi.launches()
    tc = gemm(capi, ta, tb, m, n, k, a, b)
    capi.call("set_tensor_cores", C.c_int(0))
    fp = gemm(capi, ta, tb, m, n, k, a, b)
    capi.call("set_tensor_cores", C.c_int(1))
    assert_close(tc, ref, 1e-4, "tensor-core gemm vs float64")
    assert_close(tc, fp, 1e-4, "tensor-core gemm vs FP32 kernel")
    # fp32-level accuracy: the error against float64 is of the same order as the exact-FP32 kernel's
    scale = np.abs(A) @ np.abs(B)
    e_tc = float(np.max(np.abs(tc - ref) / scale))
    e_fp = float(np.max(np.abs(fp - ref) / scale))
    assert e_tc < 4e-6, (e_tc, e_fp)


def test_tensor_core_gemm_accumulate_and_unaligned_ld(capi):
    r = rng(5)
    m, n, k = 256, 192, 100
    a = r.standard_normal((m, k + 1)).astype(np.float32)  # lda = k+1: rows are not 16-byte aligned
    b = r.standard_normal((k, n)).astype(np.float32)
    c0 = r.standard_normal((m, n)).astype(np.float32)
    out = gemm(capi, 0, 0, m, n, k, a, b, c0=c0, accumulate=1, lda=k + 1)
    assert_close(out, c0 + a[:, :k].astype(np.float64) @ b.astype(np.float64), 1e-4, "accumulate + odd lda")


def test_tensor_core_gemm_is_deterministic(capi):
    r = rng(6)
    a = r.standard_normal((256, 3136)).astype(np.float32)
    b = r.standard_normal((3136, 128)).astype(np.float32)
    assert np.array_equal(gemm(capi, 0, 0, 256, 128, 3136, a, b), gemm(capi, 0, 0, 256, 128, 3136, a, b))
