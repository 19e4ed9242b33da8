"""Batch preparation on the device (kernels_batch.cu through ts2_set_batch): span tables, reverse ranges, targets, the
inverse label index and the embedding gradient that uses it - against plain numpy restatements of what the reference
derives on the host (TNodesBatch spans, src/gpt/att/att.h:125-211; TLabelInverseIndex::BuildInverseIndex,
src/gpt/compute/gpu_embedding.cuh:38-75), and against the oracle for the gradient itself.  Index work: bit-exact."""
import ctypes as C

import numpy as np
import pytest

import oracle
from tscale2_b200 import capi, host
from tscale2_b200.capi import Ts2Error
from tscale2_b200.model import Model

pytestmark = pytest.mark.gpu

NEG = np.uint32(0x80000000)


def small_spec(vocab=512, widths=(64,), precision=capi.PREC_F16):
    s = host.ModelSpec(dim=256, head_count=2, ffn_tiles=2, vocab=vocab, attention_widths=list(widths), precision=precision)
    return s.add_blocks(1)


def exact_reverse(start, finish):
    T = len(start)
    first, last = np.full(T, T, np.int64), np.full(T, -1, np.int64)
    for t in range(T):
        if finish[t] >= start[t]:
            first[start[t]:finish[t] + 1] = np.minimum(first[start[t]:finish[t] + 1], t)
            last[start[t]:finish[t] + 1] = np.maximum(last[start[t]:finish[t] + 1], t)
    return first, last


def check_reverse(start, finish, rev_first, rev_last, tight):
    T = len(start)
    first, last = exact_reverse(start, finish)
    has = last >= 0
    # a superset: no node outside [rev_first, rev_last] attends to the key
    assert np.all(rev_first[has] <= first[has]) and np.all(rev_last[has] >= last[has])
    none = ~has
    assert np.all((rev_first[none] > rev_last[none]) | (rev_first[none] >= 0))
    assert np.all(rev_first >= 0) and np.all(rev_first <= T) and np.all(rev_last >= -1) and np.all(rev_last < T)
    if tight:  # monotone spans: the first node of the range does attend
        assert np.array_equal(rev_first[has], first[has])
        # the range may run on over span-less nodes only
        spanless = finish < start
        for to in np.flatnonzero(has)[:: max(1, T // 257)]:
            assert np.all(spanless[last[to] + 1:rev_last[to] + 1])


def expand(att, T):
    s, f, p = att
    n = np.diff(p)
    start, finish = np.zeros(T, np.int32), np.full(T, -1, np.int32)
    start[n == 1], finish[n == 1] = s, f
    return start, finish


@pytest.mark.parametrize("n_frag,seq,widths", [(4, 128, (64,)), (3, 100, (16, 1000)), (64, 1024, (1024,)), (1, 5, (2,))])
def test_span_and_target_tables(n_frag, seq, widths):
    spec = small_spec(widths=widths)
    batch = host.synthetic_batch(spec, n_frag, seq, 11)
    T = batch.node_count
    model = Model(spec, host.init_weights(spec, 1), T)
    model.set_batch(batch)
    for a in range(len(widths)):
        tab = model.batch_tables(a)
        start, finish = expand(batch.att[a], T)
        assert np.array_equal(tab["span_start"], start) and np.array_equal(tab["span_finish"], finish)
        check_reverse(start, finish, tab["rev_first"], tab["rev_last"], tight=True)
        target = np.full(T, -1, np.int32)
        target[batch.target_node] = batch.target_id
        assert np.array_equal(tab["target"], target)


def test_reverse_ranges_of_arbitrary_spans():
    lib = capi.load_library()
    rng = np.random.default_rng(5)
    for T in (1, 7, 200, 1024, 1025, 5000):
        start = rng.integers(0, T, T).astype(np.int32)
        finish = np.minimum(T - 1, start + rng.integers(-3, 60, T)).astype(np.int32)
        none = finish < start
        start[none], finish[none] = 0, -1
        rf, rl = np.empty(T, np.int32), np.empty(T, np.int32)
        rc = lib.ts2_op_attention_reverse_ranges(0, None, start.ctypes.data, finish.ctypes.data, T, rf.ctypes.data, rl.ctypes.data)
        assert rc == 0
        check_reverse(start, finish, rf, rl, tight=False)
    # no spans at all
    T = 300
    start, finish = np.zeros(T, np.int32), np.full(T, -1, np.int32)
    rf, rl = np.empty(T, np.int32), np.empty(T, np.int32)
    assert lib.ts2_op_attention_reverse_ranges(0, None, start.ctypes.data, finish.ctypes.data, T, rf.ctypes.data, rl.ctypes.data) == 0
    assert np.all(rf == T) and np.all(rl == -1)


def ragged_batch(spec, T, rng, labels_per_node=(1, 4), used_labels=None, negatives=True):
    """Nodes with a few labels each, some negative, drawn from a small set of labels so that one label has long runs."""
    used = used_labels or spec.label_count
    counts = rng.integers(labels_per_node[0], labels_per_node[1], T)
    counts[0] = max(counts[0], 1)
    label_ptr = np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32)
    n = int(label_ptr[-1])
    # a skewed choice: label 3 takes about half of all entries
    label_arr = np.where(rng.random(n) < 0.5, 3, rng.integers(0, used, n)).astype(np.uint32)
    if negatives:
        label_arr[rng.random(n) < 0.2] |= NEG
    t = np.arange(T)
    start = np.maximum(0, t - 32).astype(np.int32)
    finish = (t - 1).astype(np.int32)
    has = finish >= start
    ptr = np.concatenate([[0], np.cumsum(has)]).astype(np.int32)
    att = [(start[has], finish[has], ptr)]
    target_node = np.flatnonzero(rng.random(T) < 0.7).astype(np.int32)
    target_id = rng.integers(0, spec.vocab, len(target_node)).astype(np.int32)
    return host.Batch.from_arrays(T, label_arr, label_ptr, target_node, target_id, att)


@pytest.mark.parametrize("T,used", [(700, 40), (4096, 5000), (3000, 1)])
def test_inverse_label_index_is_a_stable_sort(T, used):
    spec = small_spec(vocab=70016)  # 17 bits of label: three radix passes
    rng = np.random.default_rng(T)
    batch = ragged_batch(spec, T, rng, labels_per_node=(0, 4), used_labels=used)
    model = Model(spec, host.init_weights(spec, 1), T)
    model.set_batch(batch)
    labels, nodes, negative = model.label_index()
    raw = batch.label_arr
    owner = np.repeat(np.arange(T), np.diff(batch.label_ptr.astype(np.int64)))
    order = np.argsort(raw & ~NEG, kind="stable")
    assert np.array_equal(labels, (raw & ~NEG)[order])
    assert np.array_equal(nodes, owner[order])
    assert np.array_equal(negative, (raw & NEG)[order] != 0)


def test_embedding_gradient_matches_the_oracle_and_repeats_exactly(oracle_port):
    """Several labels per node, negative labels, one label that owns half of the entries (runs that cross many chunks
    of the summation) - against the oracle's embedding delta; and twice the same step gives the same bits, which float
    atomics would not."""
    spec = small_spec(vocab=512)
    rng = np.random.default_rng(21)
    T = 2048
    batch = ragged_batch(spec, T, rng, used_labels=64)
    mats = host.init_weights(spec, 3)
    ref = oracle_port.backprop(spec, mats, batch, oracle.QUANT_HALF, want_states=True)
    model = Model(spec, mats, T)
    model.set_debug_taps(True)
    runs = []
    for _ in range(2):
        model.set_batch(batch)
        model.backprop(host.training_step(), apply=False)
        model.wait()
        runs.append(model.get_gradients()[0].copy())
        model.discard_gradient()
    assert np.array_equal(runs[0], runs[1])
    err = np.linalg.norm(runs[0].astype(np.float64) - ref["grads"][0]) / np.linalg.norm(ref["grads"][0])
    assert err < 5e-3, err
    s0 = model.get_state_tap(0, False, T)
    assert np.linalg.norm(s0 - ref["states"][0]) / np.linalg.norm(ref["states"][0]) < 1e-3
    # the summation itself, from the engine's own state gradient: sum of +-g over the label's nodes
    g = model.get_state_tap(0, True, T).astype(np.float64)
    owner = np.repeat(np.arange(T), np.diff(batch.label_ptr.astype(np.int64)))
    sign = np.where(batch.label_arr & NEG, -1.0, 1.0)
    want = np.zeros((spec.label_count, spec.dim))
    np.add.at(want, (batch.label_arr & ~NEG).astype(np.int64), g[owner] * sign[:, None])
    got = runs[0].astype(np.float64)
    scale = np.abs(want).max()
    k = np.abs(got).max() / scale  # the gradient's global scale factor (a power of two)
    assert np.abs(got - want * k).max() < 1e-4 * scale * k


def test_whole_step_repeats_bit_for_bit():
    """With the embedding gradient summed in a fixed order nothing in the step depends on the schedule."""
    spec = small_spec(vocab=4096, precision=capi.PREC_FP8).add_blocks(1)
    batch = host.synthetic_batch(spec, 4, 256, 5)
    mats = host.init_weights(spec, 9)
    outs = []
    for _ in range(2):
        model = Model(spec, mats, batch.node_count)
        for it in range(3):
            model.set_batch(batch)
            model.backprop(host.training_step(iteration=it), apply=True)
        model.wait()
        outs.append([w.copy() for w in model.get_weights()])
    for a, b in zip(*outs):
        assert np.array_equal(a, b)


def corrupt(batch, what):
    la, lp = batch.label_arr.copy(), batch.label_ptr.copy()
    tn, ti = batch.target_node.copy(), batch.target_id.copy()
    s, f, p = (x.copy() for x in batch.att[0])
    if what == "label":
        la[5] = 10 ** 6
    elif what == "label_ptr":
        lp[7] = lp[-1] + 100
    elif what == "target_id":
        ti[3] = 10 ** 6
    elif what == "target_node":
        tn[3] = -2
    elif what == "dup_target":
        tn[4] = tn[3]
    elif what == "span":
        f[10] = batch.node_count + 5
    elif what == "multi_span":
        p[4:] += 1  # node 3 gets two spans, the arrays grow by one
        s, f = np.insert(s, p[3], 0), np.insert(f, p[3], 0)
    return host.Batch.from_arrays(batch.node_count, la, lp, tn, ti, [(s, f, p)])


@pytest.mark.parametrize("what,code", [("label", capi.TS2_ERR_INVALID_ARG), ("label_ptr", capi.TS2_ERR_INVALID_ARG),
                                       ("target_id", capi.TS2_ERR_INVALID_ARG), ("target_node", capi.TS2_ERR_INVALID_ARG),
                                       ("dup_target", capi.TS2_ERR_UNSUPPORTED), ("span", capi.TS2_ERR_INVALID_ARG),
                                       ("multi_span", capi.TS2_ERR_UNSUPPORTED)])
def test_malformed_batches_are_reported_and_harmless(what, code):
    """The device validates every element: the step on a malformed batch stays inside its buffers, the next wait names
    the element, and the model goes on working."""
    spec = small_spec()
    good = host.synthetic_batch(spec, 2, 64, 1)
    T = good.node_count
    model = Model(spec, host.init_weights(spec, 1), T + 1)
    model.set_batch(corrupt(good, what))
    model.backprop(host.training_step(), apply=False)
    with pytest.raises(Ts2Error) as e:
        model.wait()
    assert e.value.code == code, str(e.value)
    assert "batch:" in str(e.value)
    model.discard_gradient()
    model.set_batch(good)
    model.backprop(host.training_step(), apply=False)
    model.wait()
    assert np.isfinite(model.avg_train_err())


def _tiny_batch(spec, T, n_targets, rng):
    """One fragment of T nodes, one label per node, causal spans of width 32, targets on the first n_targets nodes."""
    label_arr = rng.integers(1, spec.label_count, T).astype(np.uint32)
    label_ptr = np.arange(T + 1, dtype=np.uint32)
    t = np.arange(T)
    start, finish = np.maximum(0, t - 32).astype(np.int32), (t - 1).astype(np.int32)
    has = finish >= start
    ptr = np.concatenate([[0], np.cumsum(has)]).astype(np.int32)
    target_node = np.arange(n_targets, dtype=np.int32)
    target_id = rng.integers(0, spec.vocab, n_targets).astype(np.int32)
    return host.Batch.from_arrays(T, label_arr, label_ptr, target_node, target_id, [(start[has], finish[has], ptr)])


@pytest.mark.parametrize("T,n_targets", [(1, 1), (2, 0), (5, 5), (129, 3), (257, 0)])
def test_smallest_and_targetless_batches_match_the_oracle(oracle_port, T, n_targets):
    """Edge cases of the batch: a single node (no span at all), sizes next to a tile border, no target anywhere (every
    gradient is exactly zero and the training error is 0, not NaN)."""
    spec = small_spec(vocab=512)
    rng = np.random.default_rng(T * 10 + n_targets)
    batch = _tiny_batch(spec, T, n_targets, rng)
    mats = host.init_weights(spec, 4)
    ref = oracle_port.backprop(spec, mats, batch, oracle.QUANT_HALF, want_states=True)
    model = Model(spec, mats, max(T, 4))
    model.set_debug_taps(True)
    model.set_batch(batch)
    model.backprop(host.training_step(), apply=False)
    model.wait()
    L = len(spec.layers)
    assert np.linalg.norm(model.get_state_tap(L, False, T) - ref["states"][L]) <= 2e-3 * np.linalg.norm(ref["states"][L])
    err = model.avg_train_err()
    assert np.isfinite(err)
    for name, g, r in zip(spec.matrix_names(), model.get_gradients(), ref["grads"]):
        assert np.isfinite(g).all(), name
        if n_targets == 0:
            assert not g.any() and not r.any(), name
        else:
            assert np.linalg.norm(g.astype(np.float64) - r) <= 5e-3 * max(np.linalg.norm(r), 1e-30), name
    if n_targets == 0:
        assert err == 0.0
    else:
        assert abs(-err - ref["score"]) < 2e-3
    # and an applied step on such a batch leaves finite weights
    model.backprop(host.training_step(), apply=True)
    model.wait()
    assert all(np.isfinite(w).all() for w in model.get_weights())
