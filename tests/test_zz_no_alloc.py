"""ts2_gemm_dw_noalloc: the weight-gradient contraction for hosts that cannot allocate device
memory (all of it already sits in their own pools, or a cudaMalloc would stall their other
streams).  Its split-K scratch is a fixed array inside the library; the result must equal what
ts2_gemm_dw computes with a caller-provided workspace.  The file is named to be collected last:
the entry point shares one static array between all calls of a process, so its tests run after
every test of the ordinary entry points, and a run that stops at the first failure (-x) has
exercised those first.  It depends on no state left by other tests and passes alone in a fresh
process as well."""
import ml_dtypes
import numpy as np
import pytest

from tscale2_b200 import capi
from tscale2_b200.device import DeviceBuffer, check, sync

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


@pytest.mark.parametrize("prec", [capi.PREC_FP8, capi.PREC_F16])
def test_noalloc_matches_workspace_variant_twice_in_a_row(prec):
    lib = capi.load_library()
    rng = np.random.default_rng(17 + prec)
    T, in_dim, out_dim = 4096, 256, 384  # 3 output tiles: the scheduler splits K, so the scratch is used
    dt = ml_dtypes.float8_e4m3fn if prec == capi.PREC_FP8 else np.float16
    dy = rng.standard_normal((T, out_dim)).astype(np.float32).astype(dt)
    DW_ref, DW_new = DeviceBuffer(out_dim * in_dim * 4), DeviceBuffer(out_dim * in_dim * 4)
    DY = DeviceBuffer.from_numpy(dy)
    ws_bytes = lib.ts2_gemm_dw_workspace_bytes(T, in_dim, out_dim)
    assert ws_bytes > 0, "shape must exercise the split-K scratch"
    WS = DeviceBuffer(ws_bytes)
    for call in range(2):
        # different activations on the second call: the scratch still holds the first call's partial tiles
        x = (rng.standard_normal((T, in_dim)) * (1.0 + call)).astype(np.float32).astype(dt)
        X = DeviceBuffer.from_numpy(x)
        check(lib.ts2_gemm_dw(0, None, prec, capi.OUT_F32, T, in_dim, out_dim, DY.ptr, X.ptr, DW_ref.ptr, 0.25, WS.ptr, ws_bytes))
        check(lib.ts2_gemm_dw_noalloc(0, None, prec, capi.OUT_F32, T, in_dim, out_dim, DY.ptr, X.ptr, DW_new.ptr, 0.25))
        sync()
        ref = DW_ref.download((out_dim, in_dim), np.float32)
        got = DW_new.download((out_dim, in_dim), np.float32)
        exact = dy.astype(np.float64).T @ x.astype(np.float64) * 0.25
        assert rel_l2(ref, exact) < 2e-5
        assert rel_l2(got, ref) < 2e-5, f"call {call}"
    # accumulate form
    check(lib.ts2_gemm_dw_noalloc(0, None, prec, capi.OUT_F32_ADD, T, in_dim, out_dim, DY.ptr, X.ptr, DW_new.ptr, 0.25))
    sync()
    assert rel_l2(DW_new.download((out_dim, in_dim), np.float32), 2 * ref) < 2e-5


def test_noalloc_refuses_what_does_not_fit():
    lib = capi.load_library()
    buf = DeviceBuffer(65536 * 768)
    out = DeviceBuffer(768 * 768 * 4)
    # 18 output tiles x 8 K-splits of 128 KiB each = 18.9 MB of partial tiles > the 16 MiB array
    rc = lib.ts2_gemm_dw_noalloc(0, None, capi.PREC_FP8, capi.OUT_F32, 65536, 768, 768, buf.ptr, buf.ptr, out.ptr, 1.0)
    assert rc == capi.TS2_ERR_TOO_LARGE
    assert b"16777216" in lib.ts2_last_error(None)
    rc = lib.ts2_gemm_dw_noalloc(0, None, capi.PREC_FP8, capi.OUT_F16, 4096, 256, 384, buf.ptr, buf.ptr, out.ptr, 1.0)
    assert rc == capi.TS2_ERR_INVALID_ARG


def test_noalloc_without_split_and_on_a_stream_of_its_own():
    """A shape with enough output tiles that the scheduler does not split K (no scratch is touched, the epilogue
    stores directly), launched on an explicit non-default stream; compared with the float64 product and with
    ts2_gemm_dw.  ts2_dev_sync after a good call reports TS2_OK (it reads the entry point's own status word too)."""
    import torch
    lib = capi.load_library()
    rng = np.random.default_rng(5)
    T, in_dim, out_dim = 1024, 2048, 2048
    assert lib.ts2_gemm_dw_workspace_bytes(T, in_dim, out_dim) == 0, "shape must not split K"
    dy = rng.standard_normal((T, out_dim)).astype(np.float16)
    x = rng.standard_normal((T, in_dim)).astype(np.float16)
    DY, X = DeviceBuffer.from_numpy(dy), DeviceBuffer.from_numpy(x)
    DW_ref, DW_new = DeviceBuffer(out_dim * in_dim * 4), DeviceBuffer(out_dim * in_dim * 4)
    stream = torch.cuda.Stream(device=0)
    check(lib.ts2_gemm_dw(0, None, capi.PREC_F16, capi.OUT_F32, T, in_dim, out_dim, DY.ptr, X.ptr, DW_ref.ptr, 1.0, None, 0))
    check(lib.ts2_gemm_dw_noalloc(0, stream.cuda_stream, capi.PREC_F16, capi.OUT_F32, T, in_dim, out_dim, DY.ptr, X.ptr, DW_new.ptr, 1.0))
    assert lib.ts2_dev_sync(0) == capi.TS2_OK
    exact = dy.astype(np.float64).T @ x.astype(np.float64)
    got = DW_new.download((out_dim, in_dim), np.float32)
    assert rel_l2(got, exact) < 2e-5
    assert rel_l2(got, DW_ref.download((out_dim, in_dim), np.float32)) < 2e-5


def test_noalloc_status_word_reaches_the_host():
    """The entry point's kernels raise a status word of their own (a static device variable; the ordinary one is
    allocated on first use).  A wait that runs out there must surface through ts2_dev_sync like any other; the
    self-test lets one run out the allowed way (a barrier nothing arrives at, given up after the limit)."""
    lib = capi.load_library()
    assert lib.ts2_dev_sync(0) == capi.TS2_OK
    rc = lib.ts2_selftest_wait_limit_noalloc(0)
    assert rc == capi.TS2_ERR_DEVICE_STATUS, lib.ts2_last_error(None)
    assert b"ts2_gemm_dw_noalloc" in lib.ts2_last_error(None)
    assert lib.ts2_dev_sync(0) == capi.TS2_OK  # cleared by the report
    test_noalloc_without_split_and_on_a_stream_of_its_own()  # and the context still computes
