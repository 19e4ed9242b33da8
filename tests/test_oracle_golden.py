"""The restated CPU oracle against the golden fixtures produced by the
reference-linked build (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest

from golden.make_golden import STRIDE, configs, run

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["c1_e4m3", "c1_half", "c1_alibi_i8", "tiny_moe_e4m3"])
def test_step_matches_golden(oracle_port, name):
    gold = np.load(os.path.join(GOLDEN, name + ".npz"))
    res = run(oracle_port, name)
    assert abs(res["score"] - float(gold["score"])) < 1e-5
    np.testing.assert_allclose(res["target_prob"][::7], gold["target_prob"], rtol=2e-4, atol=1e-9)
    for i, g in enumerate(res["grads"]):
        ref_norm = float(gold[f"grad_norm_{i}"])
        assert ref_norm > 0, "a zero gradient pins nothing"
        assert abs(np.linalg.norm(g.astype(np.float64)) - ref_norm) <= 1e-5 * ref_norm
        s, r = g.reshape(-1)[::STRIDE], gold[f"grad_sample_{i}"]
        assert np.linalg.norm(s - r) <= 1e-5 * np.linalg.norm(r)
    for key in ("states", "state_grads"):
        a = res[key]
        n = np.linalg.norm(a.astype(np.float64).reshape(a.shape[0], -1), axis=1)
        np.testing.assert_allclose(n, gold[key + "_norm"], rtol=1e-5)
        s, r = a.reshape(-1)[::STRIDE], gold[key + "_sample"]
        assert np.linalg.norm(s - r) <= 1e-5 * np.linalg.norm(r)


def test_conversions_match_golden(oracle_port):
    """e4m3 / int8 weight encoders of the reference (sse_utils.h:56-78,161-204) restated in scalar
    code: bit-exact on the fixture bytes."""
    import ml_dtypes
    import oracle
    gold = np.load(os.path.join(GOLDEN, "conversions.npz"))
    src = gold["src"]
    assert np.array_equal(oracle_port.encode(src, oracle.QUANT_E4M3, 1.0), gold["e4m3"])
    assert np.array_equal(oracle_port.encode(src, oracle.QUANT_I8, 0.5), gold["i8_half"])
    table = oracle_port.decode_e4m3_table()
    assert np.array_equal(table, gold["e4m3_table"])
    # the decoder is the standard e4m3 (what the tensor cores read) for every byte the encoder can
    # produce: all but 0x80 (encoder never emits it: underflow clears the sign too) and the NaN codes
    hw = np.arange(256, dtype=np.uint8).view(ml_dtypes.float8_e4m3fn).astype(np.float32)
    ok = np.ones(256, bool)
    ok[[0x80, 0x7F, 0xFF]] = False
    assert np.array_equal(table[ok], hw[ok])
    produced = np.unique(gold["e4m3"])
    assert not np.isin([0x7F, 0xFF], produced).any()
