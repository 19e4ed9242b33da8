"""Pins the oracle's restated optimizer step (ts2o_apply_gradient: row sums of squares, dispersion average, row scale,
momentum, weight update, shrink) against the reference's OWN host-side implementation of the same step,
THostModelMatrix::AddDelta (src/gpt/matrix/host_matrix.cpp:123-157), compiled from the reference's sources
(oracle/opt_ref.cpp; `make -C oracle opt`).  The reference takes the gradient in its delta form (fp16 values times a
power-of-two scale per row); both sides get exactly that gradient.  fp32 on both sides, AVX against scalar summation
order: 2e-6 relative."""
import os

import numpy as np
import pytest

import oracle
from tscale2_b200 import capi, host

pytestmark = pytest.mark.skipif(not os.path.exists(oracle.OPT_REF_PATH),
                                reason="the reference-linked optimizer is built only where the reference sources are")


def close(a, b, tol=2e-6):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.abs(a - b).max() <= tol * max(np.abs(b).max(), 1e-30)


@pytest.mark.parametrize("y,x,per_row,sparsity", [(64, 128, True, 1.0),    # embedding / final layer: one dispersion per row
                                                  (96, 256, False, 1.0),   # a layer matrix: one dispersion for all rows
                                                  (128, 64, False, 0.25),  # sparsity scales the step (sqrt)
                                                  (40, 8, True, 1.0)])
def test_restated_optimizer_equals_the_reference_host_optimizer(oracle_port, y, x, per_row, sparsity):
    rng = np.random.default_rng(y * 1000 + x)
    w = (rng.standard_normal((y, x)) * 0.02).astype(np.float32)
    ag = np.zeros((y, x), np.float32)
    rd = np.zeros(y if per_row else 1, np.float32)
    sw = 0.0
    w_ref, ag_ref, rd_ref, sw_ref = w.copy(), ag.copy(), rd.copy(), sw
    for it in range(4):  # several steps: the dispersion average and the momentum carry over
        grad = (rng.standard_normal((y, x)) * 10.0 ** rng.uniform(-4, 1, (y, 1))).astype(np.float32)
        if it == 2:
            grad[3] = 0  # a row without gradient takes the momentum-only branch of the reference
        step = host.training_step(rate=0.01, l2reg=0.1 if it % 2 else 0.0, iteration=it)
        w_ref, ag_ref, rd_ref, sw_ref, sum2, seen = oracle.reference_add_delta(w_ref, ag_ref, grad, rd_ref, sw_ref, sparsity, step)
        assert np.abs(seen - grad).max() <= 1e-3 * np.abs(grad).max(), "the delta form is fp16: the gradient survives to 1e-3"
        w, ag, rd, sw = oracle_port.apply_gradient(w, ag, seen, rd, sw, sparsity, step)
        assert close(rd, rd_ref) and abs(sw - sw_ref) <= 1e-6 * sw_ref, f"step {it}: dispersion"
        assert close(ag, ag_ref), f"step {it}: momentum"
        assert close(w, w_ref), f"step {it}: weights"
        assert abs(float((w.astype(np.float64) ** 2).sum()) - sum2) <= 1e-5 * sum2, f"step {it}: sum of squares of the new weights"
