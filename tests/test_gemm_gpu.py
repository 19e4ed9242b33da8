"""Parity of the tcgen05 contraction kernels (through the C ABI) with the oracle's
MulForward / MulBackwardWithAccum / SumRankOne on the same quantized operands.

The operands are already e4m3 / fp16 / int8 values, so both sides see identical
inputs and the only difference left is fp32 summation order: tolerance 2e-5 relative
L2 for fp32 outputs (north-star bound for a contraction in isolation: 1e-2 fp8 /
5e-3 int8), plus output rounding (2^-11 fp16, 2^-8 bf16) for 16-bit outputs."""
import ctypes as C

import ml_dtypes
import numpy as np
import pytest

from tscale2_b200 import capi
from tscale2_b200.device import DeviceBuffer, check, sync

pytestmark = pytest.mark.gpu

OUT_DTYPES = {capi.OUT_F32: np.float32, capi.OUT_F32_ADD: np.float32, capi.OUT_F16: np.float16,
              capi.OUT_BF16: ml_dtypes.bfloat16}


def make_operand(rng, shape, prec, scale=1.0):
    """Returns (bytes as stored on the device, the same values as fp32)."""
    x = rng.standard_normal(shape).astype(np.float32) * scale
    if prec == capi.PREC_FP8:
        q = x.astype(ml_dtypes.float8_e4m3fn)
    elif prec == capi.PREC_F16:
        q = x.astype(np.float16)
    else:
        q = np.clip(np.rint(x * 20), -127, 127).astype(np.int8)
    return q, q.astype(np.float32)


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


def tol_for(out_kind):
    return {capi.OUT_F16: 6e-4, capi.OUT_BF16: 4e-3}.get(out_kind, 2e-5)


@pytest.fixture(scope="module")
def lib():
    return capi.load_library()


@pytest.mark.parametrize("prec", [capi.PREC_FP8, capi.PREC_F16, capi.PREC_INT8])
@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 256, 256), (384, 128, 512), (200, 384, 320), (512, 1280, 256)])
def test_forward_contraction_matches_mul_forward(lib, oracle_port, prec, M, N, K):
    rng = np.random.default_rng(M * 7 + N * 3 + K + prec)
    a_q, a_f = make_operand(rng, (M, K), prec)
    b_q, b_f = make_operand(rng, (N, K), prec)
    ref = oracle_port.mul_forward(a_f, b_f)  # includes sqrt(1/K)
    A, B = DeviceBuffer.from_numpy(a_q), DeviceBuffer.from_numpy(b_q)
    for out_kind in (capi.OUT_F32, capi.OUT_F16, capi.OUT_BF16):
        dt = OUT_DTYPES[out_kind]
        Cb = DeviceBuffer(M * N * np.dtype(dt).itemsize)
        Cb.zero()
        check(lib.ts2_gemm_tn(0, None, prec, out_kind, M, N, K, A.ptr, K, B.ptr, K, Cb.ptr, N,
                              float(np.float32(np.sqrt(np.float32(1.0) / K))), None, None))
        sync()
        got = Cb.download((M, N), dt).astype(np.float32)
        assert rel_l2(got, ref) < tol_for(out_kind), (prec, out_kind, M, N, K)


def test_epilogue_scales_and_accumulate(lib, oracle_port):
    rng = np.random.default_rng(11)
    M, N, K = 256, 512, 384
    a_q, a_f = make_operand(rng, (M, K), capi.PREC_FP8)
    b_q, b_f = make_operand(rng, (N, K), capi.PREC_FP8)
    rs = rng.uniform(0.01, 0.1, M).astype(np.float32)
    cs = rng.uniform(0.01, 0.1, N).astype(np.float32)
    c0 = rng.standard_normal((M, N)).astype(np.float32)
    ref = c0 + oracle_port.mul_forward(a_f, b_f) * rs[:, None] * cs[None, :]
    A, B, RS, CS, Cb = (DeviceBuffer.from_numpy(x) for x in (a_q, b_q, rs, cs, c0))
    check(lib.ts2_gemm_tn(0, None, capi.PREC_FP8, capi.OUT_F32_ADD, M, N, K, A.ptr, K, B.ptr, K, Cb.ptr, N,
                          float(np.float32(np.sqrt(np.float32(1.0) / K))), RS.ptr, CS.ptr))
    sync()
    assert rel_l2(Cb.download((M, N), np.float32), ref) < 2e-5


@pytest.mark.parametrize("prec", [capi.PREC_FP8, capi.PREC_F16, capi.PREC_INT8])
def test_dx_matches_mul_backward(lib, oracle_port, prec):
    """dX = dY · W with the transposed weight copy the requantizer keeps."""
    rng = np.random.default_rng(21 + prec)
    T, in_dim, out_dim = 384, 256, 640
    dy_q, dy_f = make_operand(rng, (T, out_dim), prec)
    w_q, w_f = make_operand(rng, (out_dim, in_dim), prec)
    ref = oracle_port.mul_backward(w_f, dy_f)  # sqrt(1/in) * dY·W
    DY, WT = DeviceBuffer.from_numpy(dy_q), DeviceBuffer.from_numpy(np.ascontiguousarray(w_q.T))
    DX = DeviceBuffer(T * in_dim * 4)
    check(lib.ts2_gemm_dx(0, None, prec, capi.OUT_F32, T, in_dim, out_dim, DY.ptr, WT.ptr, DX.ptr,
                          float(np.float32(np.sqrt(np.float32(1.0) / in_dim))), None, None))
    sync()
    assert rel_l2(DX.download((T, in_dim), np.float32), ref) < 2e-5


@pytest.mark.parametrize("prec", [capi.PREC_FP8, capi.PREC_F16, capi.PREC_INT8])
@pytest.mark.parametrize("T,in_dim,out_dim", [(128, 128, 128), (1024, 256, 384), (4096, 128, 256), (1000, 256, 128),
                                              (2048, 1280, 1536)])
def test_dw_matches_sum_rank_one(lib, oracle_port, prec, T, in_dim, out_dim):
    """dW = dY^T · X from token-major operands (no transposed copies), split over K."""
    rng = np.random.default_rng(T + in_dim + out_dim + prec)
    if prec != capi.PREC_FP8 and T % 8:
        pytest.skip("row pitch rule")
    dy_q, dy_f = make_operand(rng, (T, out_dim), prec)
    x_q, x_f = make_operand(rng, (T, in_dim), prec)
    ref = oracle_port.sum_rank_one(x_f, dy_f) if T * in_dim * out_dim <= 2 ** 28 else (
        dy_f.astype(np.float64).T @ x_f.astype(np.float64))
    DY, X = DeviceBuffer.from_numpy(dy_q), DeviceBuffer.from_numpy(x_q)
    ws_bytes = lib.ts2_gemm_dw_workspace_bytes(T, in_dim, out_dim)
    WS = DeviceBuffer(max(ws_bytes, 16))
    DW = DeviceBuffer(out_dim * in_dim * 4)
    DW.zero()
    check(lib.ts2_gemm_dw(0, None, prec, capi.OUT_F32, T, in_dim, out_dim, DY.ptr, X.ptr, DW.ptr, 1.0, WS.ptr, ws_bytes))
    sync()
    got = DW.download((out_dim, in_dim), np.float32)
    assert rel_l2(got, ref) < 2e-5, (prec, T, in_dim, out_dim, ws_bytes)
    # accumulate into an existing gradient (gradient accumulation steps)
    check(lib.ts2_gemm_dw(0, None, prec, capi.OUT_F32_ADD, T, in_dim, out_dim, DY.ptr, X.ptr, DW.ptr, 0.5, WS.ptr, ws_bytes))
    sync()
    assert rel_l2(DW.download((out_dim, in_dim), np.float32), 1.5 * np.asarray(ref, np.float64)) < 2e-5


def test_rejects_bad_arguments(lib):
    A = DeviceBuffer(1024)
    rc = lib.ts2_gemm_tn(0, None, capi.PREC_FP8, capi.OUT_F32, 128, 100, 128, A.ptr, 128, A.ptr, 128, A.ptr, 100, 1.0, None, None)
    assert rc == capi.TS2_ERR_INVALID_ARG
    rc = lib.ts2_gemm_tn(0, None, capi.PREC_FP8, capi.OUT_F32, 0, 128, 128, A.ptr, 128, A.ptr, 128, A.ptr, 128, 1.0, None, None)
    assert rc == capi.TS2_ERR_INVALID_ARG
    rc = lib.ts2_gemm_tn(0, None, 9, capi.OUT_F32, 128, 128, 128, A.ptr, 128, A.ptr, 128, A.ptr, 128, 1.0, None, None)
    assert rc == capi.TS2_ERR_INVALID_ARG


@pytest.mark.parametrize("prec", [capi.PREC_FP8, capi.PREC_F16])
def test_grouped_contractions(lib, prec):
    """Expert-sorted rows: every 128-row tile uses its expert's weights; per-expert dW over row segments."""
    rng = np.random.default_rng(31 + prec)
    E, N, K = 4, 256, 128
    seg = np.array([0, 128, 128, 512, 640], np.int32)  # expert 1 has no rows
    rows = 768  # the last 128-row tile belongs to nobody
    tile_group = np.array([0, 2, 2, 2, 3, -1], np.int32)
    a_q, a_f = make_operand(rng, (rows, K), prec)
    a_f[640:] = 0
    a_q[640:] = 0
    b_q, b_f = make_operand(rng, (E * N, K), prec)
    A, B = DeviceBuffer.from_numpy(a_q), DeviceBuffer.from_numpy(b_q)
    TG, SEG = DeviceBuffer.from_numpy(tile_group), DeviceBuffer.from_numpy(seg)
    Cb = DeviceBuffer(rows * N * 4)
    Cb.upload(np.full((rows, N), 7.0, np.float32))
    check(lib.ts2_gemm_tn_grouped(0, None, prec, capi.OUT_F32, rows, N, K, A.ptr, B.ptr, Cb.ptr, 0.5, E, TG.ptr))
    sync()
    got = Cb.download((rows, N), np.float32)
    for t, g in enumerate(tile_group):
        r = slice(128 * t, 128 * t + 128)
        ref = 0.5 * a_f[r].astype(np.float64) @ b_f[g * N:(g + 1) * N].astype(np.float64).T if g >= 0 else np.full((128, N), 7.0)
        assert rel_l2(got[r], ref) < 2e-5, (t, g)
    # per-expert weight gradients from token-major operands
    out_dim, in_dim = 128, 256
    dy_q, dy_f = make_operand(rng, (rows, out_dim), prec)
    x_q, x_f = make_operand(rng, (rows, in_dim), prec)
    DY, X = DeviceBuffer.from_numpy(dy_q), DeviceBuffer.from_numpy(x_q)
    DW = DeviceBuffer(E * out_dim * in_dim * 4)
    DW.upload(np.full((E, out_dim, in_dim), 3.0, np.float32))
    check(lib.ts2_gemm_dw_grouped(0, None, prec, capi.OUT_F32_ADD, rows, in_dim, out_dim, DY.ptr, X.ptr, DW.ptr, 2.0, E, SEG.ptr))
    sync()
    got = DW.download((E, out_dim, in_dim), np.float32)
    for g in range(E):
        r = slice(seg[g], seg[g + 1])
        ref = 3.0 + 2.0 * dy_f[r].astype(np.float64).T @ x_f[r].astype(np.float64)
        assert rel_l2(got[g], ref) < 2e-5, g
