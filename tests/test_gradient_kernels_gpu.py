"""The bandwidth-bound gradient kernels, one at a time through the C ABI, against the oracle's primitives
(NormalizeStateBackward, BackpropLoLU) on the same fp16 / fp32 inputs.  fp16 outputs: 2e-3; the e4m3 cast is compared
bit for bit with the published format's conversion."""
import ctypes as C

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


@pytest.mark.parametrize("T,D,add", [(300, 256, False), (1000, 768, True)])
def test_tilenorm_backward(oracle_port, T, D, add):
    lib = capi.load_library()
    rng = np.random.default_rng(T)
    x = rng.standard_normal((T, D)).astype(np.float32) * 3
    x[5, 128:256] = 0  # an all-zero tile has a zero gradient (cpu_util.cpp:108-111)
    dn = rng.standard_normal((T, D)).astype(np.float32)
    g0 = rng.standard_normal((T, D)).astype(np.float32) * 50
    dyn = np.array([0.37], np.float32)
    X, DN, G, DYN = (DeviceBuffer.from_numpy(a) for a in (x, dn, g0, dyn))
    AM = DeviceBuffer.from_numpy(np.zeros(1, np.uint32))
    check(lib.ts2_op_tilenorm_backward(0, None, X.ptr, DN.ptr, DYN.ptr, T, D, G.ptr, int(add), AM.ptr))
    sync()
    want = oracle_port.normalize_state_backward(x, dn * dyn[0], D // 128) + (g0 if add else 0)
    got = G.download((T, D), np.float32)
    assert rel_l2(got, want) < 1e-5
    assert np.all(got[5, 128:256] == (g0[5, 128:256] if add else 0))
    assert AM.download(1, np.uint32).view(np.float32)[0] == np.abs(got).max()


@pytest.mark.parametrize("scale", [1e-3, 7.0, 3000.0])
def test_cast_grad_is_the_published_e4m3_rounding_at_a_power_of_two(scale):
    lib = capi.load_library()
    rng = np.random.default_rng(3)
    g = (rng.standard_normal(128 * 257) * scale).astype(np.float32)
    g[::97] *= 30  # a heavy tail, as state gradients have
    G = DeviceBuffer.from_numpy(g)
    AM = DeviceBuffer.from_numpy(np.array([np.abs(g).max()], np.float32).view(np.uint32))
    OUT, GINV = DeviceBuffer(g.size), DeviceBuffer(4)
    check(lib.ts2_op_cast_grad(0, None, capi.PREC_FP8, G.ptr, g.size, AM.ptr, OUT.ptr, GINV.ptr))
    sync()
    mult = 2.0 ** np.floor(np.log2(128.0 / np.abs(g).max()))
    assert GINV.download(1, np.float32)[0] == np.float32(1.0 / mult)
    assert 64 < np.abs(g).max() * mult <= 128
    want = (g * np.float32(mult)).astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
    assert np.array_equal(OUT.download(g.size, np.uint8), want)


def _e4m3(buf, shape):
    return buf.download(shape, np.uint8).view(ml_dtypes.float8_e4m3fn).astype(np.float32)


def _e4m3_close(got, want, what):
    """got holds e4m3 values of `want`.  The kernels compute in packed fp16: where two terms cancel, its 2^-11 error is
    relative to the terms, not to the small difference, so single elements may land a few e4m3 steps off; but nearly
    all must be the nearest e4m3 value or its neighbour, and the whole tensor must be within the format's rounding
    noise (about 3 % rms for values spread over many binades)."""
    w = np.clip(want, -448, 448)
    near = w.astype(ml_dtypes.float8_e4m3fn).astype(np.float32)
    step = np.maximum(np.abs(near) * 2.0 ** -3, 2.0 ** -9)
    assert np.mean(np.abs(got - w) <= step * 1.01) > 0.995, what
    assert np.mean(got == near) > 0.95, (what, np.mean(got == near))
    assert rel_l2(got, w) < 4e-2, (what, rel_l2(got, w))


@pytest.mark.parametrize("prec", [capi.PREC_F16, capi.PREC_FP8])
def test_ffn_activation_backward(oracle_port, prec):
    lib = capi.load_library()
    rng = np.random.default_rng(11)
    T, F = 200, 512
    wide = rng.standard_normal((T, F)).astype(np.float32) * 2.5
    wide_n = oracle_port.normalize_state(wide, F // 128)
    wscale = np.sqrt(128.0 / (wide.reshape(T, F // 128, 128) ** 2).sum(-1)).astype(np.float32)
    gate = rng.standard_normal((T, F)).astype(np.float32)
    drg = rng.standard_normal((T, F)).astype(np.float32) * 4
    wg16 = np.concatenate([wide_n, gate], 1).astype(np.float16)
    drg16 = drg.astype(np.float16)
    WG, DRG, WS = DeviceBuffer.from_numpy(wg16), DeviceBuffer.from_numpy(drg16), DeviceBuffer.from_numpy(wscale)
    OUT = DeviceBuffer(T * 2 * F * 2)
    check(lib.ts2_op_ffn_act_backward(0, None, prec, DRG.ptr, WG.ptr, WS.ptr, T, F, OUT.ptr))
    sync()
    wn32, gate32, drg32 = wg16[:, :F].astype(np.float32), wg16[:, F:].astype(np.float32), drg16.astype(np.float32)
    dgate, dwn = oracle_port.backprop_lolu(gate32, wn32, drg32)
    # the oracle's tile-norm backward takes the un-normalized vector: wide = normalized / scale
    dwide = oracle_port.normalize_state_backward(wn32 / np.repeat(wscale, 128, 1), dwn, F // 128)
    if prec == capi.PREC_FP8:
        got = _e4m3(OUT, (T, 2 * F))
        _e4m3_close(got[:, F:], dgate, "d gate")
        _e4m3_close(got[:, :F], dwide, "d wide")
        return
    got = OUT.download((T, 2 * F), np.float16).astype(np.float32)
    assert rel_l2(got[:, F:], dgate) < 2e-3
    assert rel_l2(got[:, :F], dwide) < 2e-3


@pytest.mark.parametrize("prec", [capi.PREC_F16, capi.PREC_FP8])
def test_attention_gate_backward(oracle_port, prec):
    lib = capi.load_library()
    rng = np.random.default_rng(12)
    T, H = 150, 3
    Q = 128 * H
    qkvg = rng.standard_normal((T, 4 * Q)).astype(np.float16)
    o = rng.standard_normal((T, Q)).astype(np.float16)
    drg = (rng.standard_normal((T, Q)) * 3).astype(np.float16)
    QK, O, DRG = DeviceBuffer.from_numpy(qkvg), DeviceBuffer.from_numpy(o), DeviceBuffer.from_numpy(drg)
    D4 = DeviceBuffer.from_numpy(np.zeros((T, 4 * Q), np.float16))
    DOUT, DS = DeviceBuffer(T * Q * 2), DeviceBuffer(T * H * 4)
    check(lib.ts2_op_att_gate_backward(0, None, prec, DRG.ptr, QK.ptr, O.ptr, T, Q, D4.ptr, DOUT.ptr, DS.ptr))
    sync()
    dgate, dval = oracle_port.backprop_lolu(qkvg[:, 3 * Q:].astype(np.float32), o.astype(np.float32), drg.astype(np.float32))
    if prec == capi.PREC_FP8:
        d4 = _e4m3(D4, (2 * T, 4 * Q))[:T]  # the buffer was sized for fp16: the e4m3 rows fill its first half
        assert np.all(d4[:, :3 * Q] == 0), "only the gate block is written"
        _e4m3_close(d4[:, 3 * Q:], dgate, "d gate")
    else:
        d4 = D4.download((T, 4 * Q), np.float16).astype(np.float32)
        assert np.all(d4[:, :3 * Q] == 0), "only the gate block is written"
        assert rel_l2(d4[:, 3 * Q:], dgate) < 2e-3
    dout = DOUT.download((T, Q), np.float16).astype(np.float32)
    assert rel_l2(dout, dval) < 2e-3
    want_ds = (dval * o.astype(np.float32)).reshape(T, H, 128).sum(-1)
    assert rel_l2(DS.download((T, H), np.float32), want_ds) < 2e-3


@pytest.mark.parametrize("T,D", [(64, 256), (300, 768), (33, 6144)])
def test_row_quantization_is_bit_exact_with_the_reference_generator(oracle_port, T, D):
    """int8 row quantization with the reference's linear congruential generator: same bytes and scales as the oracle's
    restatement of NormalizeVecsRowMaxKernel on the same fp32 rows (rows of very different magnitude, a zero row)."""
    lib = capi.load_library()
    rng = np.random.default_rng(T + D)
    x = (rng.standard_normal((T, D)) * np.exp(rng.uniform(-8, 8, (T, 1)))).astype(np.float32)
    x[3] = 0
    X, Q, S = DeviceBuffer.from_numpy(x), DeviceBuffer(T * D), DeviceBuffer(T * 4)
    check(lib.ts2_op_rowquant_i8(0, None, X.ptr, T, D, Q.ptr, S.ptr))
    sync()
    q_ref, s_ref = oracle_port.rowquant_i8(x)
    assert np.array_equal(S.download(T, np.float32), s_ref)
    q = Q.download((T, D), np.int8)
    assert np.array_equal(q, q_ref), f"{np.count_nonzero(q != q_ref)} of {q.size} bytes differ"
    # unbiased: the mean of the dequantized rows is the mean of the rows to well within a rounding step
    nz = s_ref > 0
    assert np.abs((q[nz] * s_ref[nz, None] - x[nz]).mean(1)).max() < 0.1 * s_ref[nz].max()
