"""Failure detection without a GPU fault: a wait that can never be satisfied runs into the library's limit, the kernel
returns with the time-out bit set, the host reads it as an error code, and the same context goes on working."""
import numpy as np
import pytest

from tscale2_b200 import capi
from tscale2_b200.device import DeviceBuffer, check

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_the_context_survives():
    lib = capi.load_library()
    assert lib.ts2_dev_sync(0) == capi.TS2_OK
    rc = lib.ts2_selftest_wait_limit(0)
    assert rc == capi.TS2_ERR_DEVICE_STATUS, lib.ts2_last_error(None)
    assert b"timed out" in lib.ts2_last_error(None)
    # the status word was cleared by the report, and the device still computes
    assert lib.ts2_dev_sync(0) == capi.TS2_OK
    M = N = K = 256
    rng = np.random.default_rng(0)
    a = rng.standard_normal((M, K)).astype(np.float16)
    b = rng.standard_normal((N, K)).astype(np.float16)
    A, B, Cb = DeviceBuffer.from_numpy(a), DeviceBuffer.from_numpy(b), DeviceBuffer(M * N * 4)
    check(lib.ts2_gemm_tn(0, None, capi.PREC_F16, capi.OUT_F32, M, N, K, A.ptr, K, B.ptr, K, Cb.ptr, N, 1.0, None, None))
    check(lib.ts2_dev_sync(0))
    got = Cb.download((M, N), np.float32)
    ref = a.astype(np.float32) @ b.astype(np.float32).T
    assert np.abs(got - ref).max() < 1e-2 * np.abs(ref).max()
