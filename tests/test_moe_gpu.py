"""Mixture-of-experts layers: expert selection bit-exact with the oracle's CpuMoe on the same
logits, and the end-to-end step of a small ATT+FFN / ATT+MoE model against the oracle."""
import ctypes as C

import numpy as np
import pytest

import oracle
from tscale2_b200 import capi, host
from tscale2_b200.model import Model

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


@pytest.mark.parametrize("E,k", [(4, 2), (32, 2), (24, 6), (128, 8)])
def test_expert_selection_is_bit_exact(oracle_port, E, k):
    lib = capi.load_library()
    rng = np.random.default_rng(E + k)
    T = 1000
    logits = rng.standard_normal((T, E)).astype(np.float32)
    logits[:50] = np.round(logits[:50])  # plenty of exact ties: the lowest index must win
    ids = np.zeros((T, k), np.int32)
    w = np.zeros((T, k), np.float32)
    rc = lib.ts2_moe_route(0, logits.ctypes.data, T, E, k, ids.ctypes.data, w.ctypes.data)
    assert rc == 0, lib.ts2_last_error(None)
    ref = oracle_port.moe_select(logits, k)  # dense [T][E], zero where not selected
    dense = np.zeros_like(ref)
    for j in range(k):
        dense[np.arange(T), ids[:, j]] = w[:, j]
    assert np.array_equal(dense != 0, ref != 0), "selected expert sets differ"
    np.testing.assert_allclose(dense, ref, rtol=2e-6, atol=0)
    # order of the k choices: descending logit, ties by index
    picked = np.take_along_axis(logits, ids, 1)
    assert (np.diff(picked, axis=1) <= 0).all()


def moe_spec(precision):
    s = host.ModelSpec(dim=128, head_count=1, ffn_tiles=2, vocab=256, attention_widths=[16, 48], expert_dim=128,
                       moe_expert_count=4, moe_selected=2, precision=precision)
    return s.add_blocks(1, attention_type_id=0).add_blocks(1, attention_type_id=1, alibi_slope=0.25, moe=True)


def _moe_run(oracle_port, precision, engine_rounding=False):
    spec = moe_spec(precision)
    mats = host.init_weights(spec, 77, select_std=1.0)
    batch = host.synthetic_batch(spec, 3, 40, 78)
    quant = oracle.QUANT_E4M3 if precision == capi.PREC_FP8 else oracle.QUANT_HALF
    ref = oracle_port.backprop(spec, mats, batch, quant, want_states=True, engine_rounding=engine_rounding)
    return spec, mats, batch, ref


def _moe_engine(spec, mats, batch):
    model = Model(spec, mats, batch.node_count)
    model.set_debug_taps(True)
    model.set_batch(batch)
    model.backprop(host.training_step(), apply=False)
    model.wait()
    return model


def test_moe_step_matches_oracle(oracle_port):
    """The model of the golden fixture tiny_moe_e4m3: one ATT+FFN block, one ATT+MoE block (4 experts, 2 selected), fp16
    operands: every tensor within 5e-3 of the oracle."""
    spec, mats, batch, ref = _moe_run(oracle_port, capi.PREC_F16)
    model = _moe_engine(spec, mats, batch)
    T, L = batch.node_count, len(spec.layers)
    report = [(f"state[{l}]", rel_l2(model.get_state_tap(l, False, T), ref["states"][l])) for l in range(L + 1)]
    report += [(f"state_grad[{l}]", rel_l2(model.get_state_tap(l, True, T), ref["state_grads"][l])) for l in range(L, -1, -1)]
    report += [(n, rel_l2(g, r)) for n, g, r in zip(spec.matrix_names(), model.get_gradients(), ref["grads"])]
    text = "\n".join(f"{n:24s} {e:.3e}" for n, e in report)
    print(text)
    bad = [(n, e) for n, e in report if not e < 5e-3]
    assert not bad, text


def test_moe_fp8_step_is_as_close_to_fp32_as_the_format_allows(oracle_port):
    """e4m3 operands on the same model.  The model is tiny (120 nodes, dim 128): the format's rounding noise averages
    over few terms, and a router logit that the noise moves across a near-tie selects another expert for that node, a
    discrete change.  So the bar is the format's own: the oracle with the engine's e4m3 rounding inserted (router
    logits from the rounded normalized state, as in the engine) against the fp32 oracle gives the distance the format
    causes per tensor, and the engine may be at most 1.5 x that + 1e-2 from the fp32 oracle; the expert choices of
    engine and rounding oracle are compared through the router matrix gradient."""
    spec, mats, batch, ref = _moe_run(oracle_port, capi.PREC_FP8)
    fmt = _moe_run(oracle_port, capi.PREC_FP8, engine_rounding=True)[3]
    model = _moe_engine(spec, mats, batch)
    report, bad = [], []
    for name, g, f, r in zip(spec.matrix_names(), model.get_gradients(), fmt["grads"], ref["grads"]):
        e_engine, e_format = rel_l2(g, r), rel_l2(f, r)
        report.append(f"{name:24s} engine-fp32 {e_engine:.3e}   format-fp32 {e_format:.3e}   engine-format {rel_l2(g, f):.3e}")
        if not e_engine <= 1.5 * e_format + 1e-2:
            bad.append(name)
    text = "\n".join(report)
    print(text)
    assert not bad, f"further from fp32 than the format explains: {bad}\n{text}"


def test_moe_step_applies_and_trains(oracle_port):
    """Apply a few steps on one batch: the training error must fall (optimizer + requantisation of the
    per-expert weight blocks)."""
    spec = moe_spec(capi.PREC_FP8)
    mats = host.init_weights(spec, 5, select_std=1.0)
    batch = host.synthetic_batch(spec, 3, 40, 6)
    model = Model(spec, mats, batch.node_count)
    model.set_batch(batch)
    errs = []
    for i in range(6):
        model.backprop(host.training_step(rate=0.02, iteration=i), apply=True)
        errs.append(model.avg_train_err())
    assert errs[-1] < errs[0] - 0.05, errs


def test_experts_without_rows(oracle_port):
    """32 experts, 2 selected, 24 nodes: most experts receive no row at all (empty segments of the grouped
    contractions, weight gradients that must stay exactly zero), a few receive one or two."""
    s = host.ModelSpec(dim=128, head_count=1, ffn_tiles=2, vocab=256, attention_widths=[16], expert_dim=128,
                       moe_expert_count=32, moe_selected=2, precision=capi.PREC_F16)
    spec = s.add_blocks(1, moe=True)
    mats = host.init_weights(spec, 11, select_std=1.0)
    batch = host.synthetic_batch(spec, 2, 12, 12)
    ref = oracle_port.backprop(spec, mats, batch, oracle.QUANT_HALF, want_states=True)
    model = _moe_engine(spec, mats, batch)
    names = spec.matrix_names()
    grads = model.get_gradients()
    for name, g, r in zip(names, grads, ref["grads"]):
        assert rel_l2(g, r) < 5e-3, name
    X, D, E = 128, 128, 32
    expand = grads[names.index("L1.moe.expand")].reshape(E, X, D)
    used = np.array([expand[e].any() for e in range(E)])
    ref_used = np.array([ref["grads"][names.index("L1.moe.expand")].reshape(E, X, D)[e].any() for e in range(E)])
    assert np.array_equal(used, ref_used) and 0 < used.sum() < E, "the same experts are touched, and some are not"


def test_expert_matrices_step_with_their_sparsity(oracle_port):
    """The applied step of every matrix of a mixture-of-experts model against the restated optimizer on the engine's own
    gradient: the expert matrices move by rate x sqrt(selected / experts) (TModelMatrix::Sparsity), the others by rate."""
    spec = moe_spec(capi.PREC_F16)
    mats = host.init_weights(spec, 5, select_std=1.0)
    batch = host.synthetic_batch(spec, 3, 40, 6)
    model = Model(spec, mats, batch.node_count)
    model.set_batch(batch)
    step = host.training_step(rate=0.01, l2reg=0.05, iteration=2)
    model.backprop(step, apply=False)
    g = model.get_gradients()
    model.discard_gradient()
    model.backprop(step, apply=True)
    new_w, mom = model.get_weights(), model.get_momentum()
    sparsity = spec.matrix_sparsity()
    assert sorted(set(sparsity)) == [0.5, 1.0]
    for i, (name, w0) in enumerate(zip(spec.matrix_names(), mats)):
        n_disp = w0.shape[0] if i < 2 else 1
        w_ref, ag_ref, _, _ = oracle_port.apply_gradient(w0, np.zeros_like(w0), g[i], np.zeros(n_disp, np.float32), 0.0, sparsity[i], step)
        assert rel_l2(new_w[i] - w0, w_ref - w0) < 1e-4, name
        assert rel_l2(mom[i], ag_ref) < 1e-4, name
