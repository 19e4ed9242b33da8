"""Primitive by primitive: the restated oracle against the reference's own compiled
functions.  Skipped where the reference-linked build (oracle/_ref) does not exist;
the golden fixtures cover those machines."""
import numpy as np


def _close(a, b, tol=2e-6):
    assert np.linalg.norm(a.astype(np.float64) - b) <= tol * max(np.linalg.norm(b.astype(np.float64)), 1e-30)


def test_linear_primitives(oracle_port, oracle_ref):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((37, 256), dtype=np.float32)
    w = rng.standard_normal((128, 256), dtype=np.float32)
    dy = rng.standard_normal((37, 128), dtype=np.float32)
    _close(oracle_port.mul_forward(x, w), oracle_ref.mul_forward(x, w))
    _close(oracle_port.mul_backward(w, dy), oracle_ref.mul_backward(w, dy))
    _close(oracle_port.sum_rank_one(x, dy), oracle_ref.sum_rank_one(x, dy))


def test_norm_lolu_rope(oracle_port, oracle_ref):
    rng = np.random.default_rng(6)
    s = rng.standard_normal((19, 384), dtype=np.float32)
    s[3, 128:256] = 0  # an all-zero tile normalizes to zero
    g = rng.standard_normal((19, 384), dtype=np.float32)
    for heads in (3, 1):
        _close(oracle_port.normalize_state(s, heads), oracle_ref.normalize_state(s, heads))
        _close(oracle_port.normalize_state_backward(s, g, heads), oracle_ref.normalize_state_backward(s, g, heads))
    gate = rng.standard_normal((19, 384), dtype=np.float32) * 8  # reaches the |2x| > 20 clamps
    _close(oracle_port.lolu(gate, s), oracle_ref.lolu(gate, s))
    for a, b in zip(oracle_port.backprop_lolu(gate, s, g), oracle_ref.backprop_lolu(gate, s, g)):
        _close(a, b)
    for d in (1.0, -1.0):
        _close(oracle_port.rope(s, 128, d), oracle_ref.rope(s, 128, d))


def test_attention(oracle_port, oracle_ref):
    rng = np.random.default_rng(7)
    T, H = 70, 2
    q, k, v, dval = (rng.standard_normal((T, 128 * H), dtype=np.float32) for _ in range(4))
    t = np.arange(T)
    start = np.maximum((t // 35) * 35, t - 20)
    finish = t - 1
    has = finish >= start
    att = (start[has].astype(np.int32), finish[has].astype(np.int32),
           np.concatenate([[0], np.cumsum(has)]).astype(np.int32))
    for slope in (0.0, 0.5):
        a = oracle_port.attention(q, k, v, H, slope, att, dval)
        b = oracle_ref.attention(q, k, v, H, slope, att, dval)
        for key in ("val", "sum_weight", "max_dp", "dq", "dk", "dv"):
            _close(a[key], b[key], 5e-6)
