"""Attention core (forward, dQ, dK, dV) through the C ABI against the oracle's
TAttentionComputer restatement, for both device formulations.  Inputs are fp16 values, so both
sides see the same numbers; the tensor-core kernels round the softmax weights and the score
gradients to fp16 before the second contraction, hence 3e-3 (fp16 rounding 2^-11 per factor)."""
import ctypes as C

import numpy as np
import pytest

from tscale2_b200 import capi
from tscale2_b200.device import DeviceBuffer, check, sync

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


def causal_spans(T, frag, width):
    t = np.arange(T)
    start = np.maximum((t // frag) * frag, t - width).astype(np.int32)
    finish = (t - 1).astype(np.int32)
    none = finish < start
    start[none], finish[none] = 0, -1
    return start, finish


def csr(start, finish):
    has = finish >= start
    return (start[has].astype(np.int32), finish[has].astype(np.int32), np.concatenate([[0], np.cumsum(has)]).astype(np.int32))


def run_device(lib, variant, q, k, v, dout, start, finish, H, slope):
    T = q.shape[0]
    ip = lambda a: a.ctypes.data_as(C.c_void_p)
    Qb, Kb, Vb, DOb = (DeviceBuffer.from_numpy(x) for x in (q, k, v, dout))
    Ob, LSE = DeviceBuffer(q.nbytes), DeviceBuffer(T * H * 4)
    check(lib.ts2_attention_forward(0, None, min(variant, 2), Qb.ptr, Kb.ptr, Vb.ptr, ip(start), ip(finish), T, H, slope, Ob.ptr, LSE.ptr))
    sync()
    o = Ob.download(q.shape, np.float16)
    lse = LSE.download((T, H), np.float32)
    dscale = (dout.astype(np.float32) * o.astype(np.float32)).reshape(T, H, 128).sum(-1).astype(np.float32)
    DS = DeviceBuffer.from_numpy(dscale)
    DQ, DK, DV = (DeviceBuffer(T * H * 128 * 4) for _ in range(3))
    gt = np.float16 if variant == 3 else np.float32  # variant 3: tcgen05 kernels with fp16 gradient outputs
    check(lib.ts2_attention_backward(0, None, variant, Qb.ptr, Kb.ptr, Vb.ptr, DOb.ptr, LSE.ptr, DS.ptr, ip(start), ip(finish), T, H,
                                     slope, DQ.ptr, DK.ptr, DV.ptr))
    sync()
    shape = (T, H * 128)
    return (o.astype(np.float32), lse) + tuple(b.download(shape, gt).astype(np.float32) for b in (DQ, DK, DV))


@pytest.mark.parametrize("variant", [0, 1, 2, 3])
@pytest.mark.parametrize("T,frag,width,H,slope", [(128, 128, 128, 1, 0.0), (300, 100, 48, 2, 0.5), (512, 256, 1000, 2, 0.0),
                                                  (70, 35, 20, 1, 0.25), (640, 640, 64, 1, 0.0)])
def test_attention_matches_oracle(oracle_port, variant, T, frag, width, H, slope):
    lib = capi.load_library()
    rng = np.random.default_rng(T + width + H)
    q, k, v, dout = (rng.standard_normal((T, 128 * H)).astype(np.float16) for _ in range(4))
    k = (k.astype(np.float32) * 1.7).astype(np.float16)  # scores large enough to move the running maximum off zero
    start, finish = causal_spans(T, frag, width)
    ref = oracle_port.attention(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), H, slope, csr(start, finish),
                                dout.astype(np.float32))
    o, lse, dq, dk, dv = run_device(lib, variant, q, k, v, dout, start, finish, H, slope)
    ref_lse = (ref["max_dp"] + np.log2(ref["sum_weight"])).T  # oracle keeps [head][t]
    assert np.abs(lse - ref_lse).max() < 2e-3
    assert rel_l2(o, ref["val"]) < 1.5e-3  # fp16 output
    # the oracle's dScale comes from its own fp32 o; the device path was fed dScale from the fp16 o
    assert rel_l2(dq, ref["dq"]) < 3e-3
    assert rel_l2(dk, ref["dk"]) < 3e-3
    assert rel_l2(dv, ref["dv"]) < 3e-3


def test_arbitrary_single_spans(oracle_port):
    """Spans that are neither causal nor monotone: each node looks at a random interval."""
    lib = capi.load_library()
    rng = np.random.default_rng(3)
    T, H = 200, 1
    q, k, v, dout = (rng.standard_normal((T, 128 * H)).astype(np.float16) for _ in range(4))
    start = rng.integers(0, T, T).astype(np.int32)
    finish = np.minimum(T - 1, start + rng.integers(-3, 60, T)).astype(np.int32)
    none = finish < start
    start[none], finish[none] = 0, -1
    ref = oracle_port.attention(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), H, 0.0, csr(start, finish),
                                dout.astype(np.float32))
    for variant in (0, 1, 2, 3):
        o, lse, dq, dk, dv = run_device(lib, variant, q, k, v, dout, start, finish, H, 0.0)
        assert rel_l2(o, ref["val"]) < 1.5e-3
        assert rel_l2(dq, ref["dq"]) < 3e-3 and rel_l2(dk, ref["dk"]) < 3e-3 and rel_l2(dv, ref["dv"]) < 3e-3


def test_tcgen05_kernels_match_mma_kernels_at_scale():
    """Hundreds of CTAs with up to 18 tiles each, two CTAs per SM in the forward kernel: the size at which a missing
    ordering between warps or MMAs shows (the small cases above run one or two tiles per CTA).  The two device
    formulations share no code, so elementwise agreement within fp16 rounding of the outputs is a strong check."""
    lib = capi.load_library()
    T, H, frag = 16384, 12, 1024
    rng = np.random.default_rng(7)
    q, k, v, dout = (rng.standard_normal((T, H * 128)).astype(np.float16) for _ in range(4))
    start, finish = causal_spans(T, frag, frag)
    ref = run_device(lib, 0, q, k, v, dout, start, finish, H, 0.0)
    for rep in range(4):  # a race does not show on every launch; the last repeat takes the fp16-gradient form
        got = run_device(lib, 3 if rep == 3 else 2, q, k, v, dout, start, finish, H, 0.0)
        for name, a, b in zip(["o", "lse", "dq", "dk", "dv"], got, ref):
            err = np.abs(a - b).max()
            assert err < 2e-2 * max(1.0, np.abs(b).max() / 4), f"{name}: max abs difference {err} (repeat {rep})"


def test_fp16_gradients_saturate_instead_of_overflowing():
    """The engine's form of the backward kernels writes dQ, dK, dV as fp16.  A key that every later node attends to
    (the first token of a sequence) collects gradients of tens of thousands once the weights have moved, more than
    fp16 holds: the store must saturate at +-65504, never write an infinity (which the next kernel's differences
    would turn into NaN and the step into a NaN loss).  Here dout is scaled until dK and dV pass the fp16 range;
    entries that stay in range must still agree with the fp32 form."""
    lib = capi.load_library()
    T, H = 1024, 2
    rng = np.random.default_rng(11)
    q, k, v = (rng.standard_normal((T, 128 * H)).astype(np.float16) for _ in range(3))
    q[:, :] = np.abs(q)  # aligned queries: the sums over the nodes do not cancel
    dout = (np.abs(rng.standard_normal((T, 128 * H))) * 2000).astype(np.float16)
    # every node attends to the first eight keys only: each of them sums the contributions of ~1000 nodes
    t = np.arange(T)
    start = np.zeros(T, np.int32)
    finish = np.minimum(t - 1, 7).astype(np.int32)
    ref = run_device(lib, 2, q, k, v, dout, start, finish, H, 0.0)
    got = run_device(lib, 3, q, k, v, dout, start, finish, H, 0.0)
    overflowed = 0
    for name, a, b in zip(["dq", "dk", "dv"], got[2:], ref[2:]):
        assert np.isfinite(a).all(), f"{name}: {np.count_nonzero(~np.isfinite(a))} non-finite fp16 outputs"
        big = np.abs(b) > 65504
        overflowed += int(big.sum())
        assert (np.abs(a[big]) == 65504).all(), name
        assert (np.sign(a[big]) == np.sign(b[big])).all(), name
        assert rel_l2(a[~big], b[~big]) < 2e-3, name
    assert overflowed > 0, "the case no longer drives any gradient past the fp16 range"
