"""TEST INFRASTRUCTURE — ctypes binding of the CPU oracle.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may import
this package.  Two libraries share one interface (oracle/ts2_oracle.h):
libts2_oracle.so (restated primitives, always buildable) and
_ref/libts2_oracle_ref.so (the same driver over the reference's own compiled
CPU functions, built only where the reference sources are present)."""
import ctypes as C
import os
import subprocess

import numpy as np

from tscale2_b200 import capi, host

_HERE = os.path.dirname(os.path.abspath(__file__))
PORT_PATH = os.path.join(_HERE, "libts2_oracle.so")
REF_PATH = os.path.join(_HERE, "_ref", "libts2_oracle_ref.so")
QUANT_I8, QUANT_E4M3, QUANT_HALF, QUANT_NONE = 0, 1, 2, 3


class Outputs(C.Structure):
    _fields_ = [("grads", C.POINTER(C.POINTER(C.c_float))), ("states", C.POINTER(C.c_float)),
                ("state_grads", C.POINTER(C.c_float)), ("target_prob", C.POINTER(C.c_float)),
                ("score", C.c_double), ("seconds", C.c_double)]


def build(reference="/root/reference"):
    """Compile the restatement, and the reference-linked variant where the reference tree exists."""
    subprocess.check_call(["make", "-s", "-C", _HERE])
    if os.path.isdir(os.path.join(reference, "src")):
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", "ckpt", "opt", f"REFERENCE={reference}"])


_fp = C.POINTER(C.c_float)


def _f(a):
    return a.ctypes.data_as(_fp)


class Oracle:
    def __init__(self, kind="port"):
        path = PORT_PATH if kind == "port" else REF_PATH
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = C.CDLL(path)
        self.kind = kind
        L = self.lib
        L.ts2o_backend.restype = C.c_char_p
        L.ts2o_backprop.restype = C.c_int
        L.ts2o_backprop.argtypes = [C.POINTER(capi.ModelDescr), C.POINTER(capi.MatrixView), C.c_int, _fp,
                                    C.POINTER(capi.BatchNodes), C.c_int, C.POINTER(Outputs)]
        L.ts2o_quantize_matrix.argtypes = [_fp, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_void_p, _fp, _fp]
        L.ts2o_apply_gradient.argtypes = [_fp, _fp, _fp, C.c_int64, C.c_int64, _fp, C.c_int64, _fp, C.c_float,
                                          C.POINTER(capi.TrainingStep)]
        L.ts2o_apply_gradient.restype = C.c_int
        for name, n_ptr, ints in [("ts2o_mul_forward", 3, 3), ("ts2o_mul_backward_accum", 3, 3),
                                  ("ts2o_sum_rank_one", 3, 3), ("ts2o_normalize_state", 2, 3),
                                  ("ts2o_normalize_state_backward", 3, 3)]:
            getattr(L, name).argtypes = [_fp] * n_ptr + [C.c_int] * ints
            getattr(L, name).restype = None
        L.ts2o_lolu.argtypes = [_fp, _fp, _fp, C.c_int64]
        L.ts2o_backprop_lolu.argtypes = [_fp] * 5 + [C.c_int64]
        L.ts2o_rope.argtypes = [_fp, C.c_int, C.c_int, C.c_int, C.c_float]
        L.ts2o_attention.argtypes = [_fp, _fp, _fp, C.c_int, C.c_int, C.c_float, C.POINTER(capi.AttentionInfo),
                                     _fp, _fp, _fp, _fp, _fp, _fp, _fp]
        L.ts2o_moe_select.argtypes = [_fp, _fp, C.c_int, C.c_int, C.c_int]
        L.ts2o_moe_select_backward.argtypes = [_fp, _fp, C.c_int, C.c_int]

    def backend(self):
        return self.lib.ts2o_backend().decode()

    # -- whole step -------------------------------------------------------------------------
    def backprop(self, spec: host.ModelSpec, mats, batch: host.Batch, weight_quant, bias=None,
                 want_states=False, engine_rounding=False):
        """engine_rounding: also round the contractions' activation / gradient operands where the B200 engine's fp8
        pipeline (e4m3) or, with int8 weights, its int8 pipeline does (ts2o_set_activation_quant), instead of keeping
        them fp32."""
        self.lib.ts2o_set_activation_quant((2 if weight_quant == QUANT_I8 else 1) if engine_rounding else 0)
        try:
            return self._backprop(spec, mats, batch, weight_quant, bias, want_states)
        finally:
            self.lib.ts2o_set_activation_quant(0)

    def round_e4m3(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros_like(x)
        self.lib.ts2o_round_e4m3.argtypes = [_fp, C.c_int64, _fp]
        self.lib.ts2o_round_e4m3(_f(x), x.size, _f(out))
        return out

    def rowquant_i8(self, x):
        x = np.ascontiguousarray(x, np.float32)
        T, D = x.shape
        q = np.zeros((T, D), np.int8)
        scale = np.zeros(T, np.float32)
        self.lib.ts2o_rowquant_i8.argtypes = [_fp, C.c_int, C.c_int, C.c_void_p, _fp]
        self.lib.ts2o_rowquant_i8(_f(x), T, D, q.ctypes.data_as(C.c_void_p), _f(scale))
        return q, scale

    def _backprop(self, spec, mats, batch, weight_quant, bias, want_states):
        descr, keep = spec.to_c()
        views = host.matrix_views(mats)
        grads = [np.zeros_like(m) for m in mats]
        gptrs = (_fp * len(mats))(*[_f(g) for g in grads])
        T, D, L = batch.node_count, spec.dim, len(spec.layers)
        out = Outputs()
        out.grads = gptrs
        states = state_grads = None
        if want_states:
            states = np.zeros((L + 1, T, D), np.float32)
            state_grads = np.zeros((L + 1, T, D), np.float32)
            out.states, out.state_grads = _f(states), _f(state_grads)
        prob = np.zeros(len(batch.target_node), np.float32)
        out.target_prob = _f(prob)
        b = None if bias is None else _f(np.ascontiguousarray(bias, np.float32))
        rc = self.lib.ts2o_backprop(C.byref(descr), views, len(mats), b, C.byref(batch.c), weight_quant, C.byref(out))
        if rc != 0:
            raise RuntimeError(f"ts2o_backprop failed: {rc}")
        return dict(grads=grads, states=states, state_grads=state_grads, target_prob=prob, score=out.score,
                    seconds=out.seconds)

    # -- matrices ---------------------------------------------------------------------------
    def quantize(self, w, quant, no_scale=False):
        w = np.ascontiguousarray(w, np.float32)
        y, x = w.shape
        deq = np.zeros_like(w)
        sko = C.c_float()
        q = np.zeros((y, x), {QUANT_I8: np.int8, QUANT_E4M3: np.uint8, QUANT_HALF: np.uint16, QUANT_NONE: np.uint8}[quant])
        self.lib.ts2o_quantize_matrix(_f(w), x, y, quant, int(no_scale), q.ctypes.data_as(C.c_void_p), _f(deq),
                                      C.cast(C.byref(sko), _fp))
        return q, deq, sko.value

    def encode(self, src, quant, mult=1.0):
        src = np.ascontiguousarray(src, np.float32)
        dst = np.zeros(src.shape, {QUANT_I8: np.int8, QUANT_E4M3: np.uint8, QUANT_HALF: np.uint16}[quant])
        self.lib.ts2o_encode.argtypes = [_fp, C.c_int64, C.c_int, C.c_float, C.c_void_p]
        self.lib.ts2o_encode(_f(src), src.size, quant, mult, dst.ctypes.data_as(C.c_void_p))
        return dst

    def decode_e4m3_table(self):
        self.lib.ts2o_decode_e4m3.restype = C.c_float
        self.lib.ts2o_decode_e4m3.argtypes = [C.c_uint8]
        return np.array([self.lib.ts2o_decode_e4m3(b) for b in range(256)], np.float32)

    def apply_gradient(self, weights, avg_grad, grad, row_disp, sum_weight, sparsity, step):
        """In-place on copies; returns (weights, avg_grad, row_disp, sum_weight)."""
        w, ag = weights.copy(), avg_grad.copy()
        rd = np.ascontiguousarray(row_disp, np.float32).copy()
        sw = C.c_float(sum_weight)
        y, x = w.shape
        rc = self.lib.ts2o_apply_gradient(_f(w), _f(ag), _f(np.ascontiguousarray(grad, np.float32)), x, y, _f(rd), len(rd),
                                          C.cast(C.byref(sw), _fp), sparsity, C.byref(step))
        assert rc == 0
        return w, ag, rd, sw.value

    # -- primitives -------------------------------------------------------------------------
    def mul_forward(self, x, w):
        T, i = x.shape
        o = w.shape[0]
        y = np.zeros((T, o), np.float32)
        self.lib.ts2o_mul_forward(_f(x), _f(w), _f(y), T, i, o)
        return y

    def mul_backward(self, w, dy):
        T, o = dy.shape
        i = w.shape[1]
        dx = np.zeros((T, i), np.float32)
        self.lib.ts2o_mul_backward_accum(_f(dx), _f(w), _f(dy), T, i, o)
        return dx

    def sum_rank_one(self, x, dy):
        T, i = x.shape
        o = dy.shape[1]
        d = np.zeros((o, i), np.float32)
        self.lib.ts2o_sum_rank_one(_f(x), _f(dy), _f(d), T, i, o)
        return d

    def normalize_state(self, s, head_count):
        out = np.zeros_like(s)
        self.lib.ts2o_normalize_state(_f(s), _f(out), s.shape[0], s.shape[1], head_count)
        return out

    def normalize_state_backward(self, s, dnorm, head_count):
        out = np.zeros_like(s)
        self.lib.ts2o_normalize_state_backward(_f(s), _f(dnorm), _f(out), s.shape[0], s.shape[1], head_count)
        return out

    def lolu(self, gate, vals):
        out = np.zeros_like(vals)
        self.lib.ts2o_lolu(_f(gate), _f(vals), _f(out), vals.size)
        return out

    def backprop_lolu(self, gate, vals, grad):
        a, b = np.zeros_like(vals), np.zeros_like(vals)
        self.lib.ts2o_backprop_lolu(_f(gate), _f(vals), _f(grad), _f(a), _f(b), vals.size)
        return a, b

    def rope(self, p, head_dim=128, direction=1.0):
        out = np.ascontiguousarray(p, np.float32).copy()
        self.lib.ts2o_rope(_f(out), out.shape[0], out.shape[1], head_dim, direction)
        return out

    def attention(self, q, k, v, head_count, alibi_slope, att, d_val=None):
        """att = (start, finish, ptr) int32 arrays.  Returns dict."""
        T = q.shape[0]
        ip = C.POINTER(C.c_int32)
        ai = capi.AttentionInfo(att[0].ctypes.data_as(ip), att[1].ctypes.data_as(ip), att[2].ctypes.data_as(ip))
        val = np.zeros_like(q)
        sw = np.zeros((head_count, T), np.float32)
        mx = np.zeros((head_count, T), np.float32)
        dq = dk = dv = None
        if d_val is not None:
            dq, dk, dv = np.zeros_like(q), np.zeros_like(q), np.zeros_like(q)
        self.lib.ts2o_attention(_f(q), _f(k), _f(v), T, head_count, alibi_slope, C.byref(ai), _f(val), _f(sw), _f(mx),
                                None if d_val is None else _f(d_val), None if dq is None else _f(dq),
                                None if dk is None else _f(dk), None if dv is None else _f(dv))
        return dict(val=val, sum_weight=sw, max_dp=mx, dq=dq, dk=dk, dv=dv)

    def moe_select(self, logits, selected):
        out = np.zeros_like(logits)
        self.lib.ts2o_moe_select(_f(logits), _f(out), logits.shape[0], logits.shape[1], selected)
        return out

    def moe_select_backward(self, weights, dmoe):
        out = np.ascontiguousarray(dmoe, np.float32).copy()
        self.lib.ts2o_moe_select_backward(_f(weights), _f(out), weights.shape[0], weights.shape[1])
        return out


def have_reference_build():
    return os.path.exists(REF_PATH)


OPT_REF_PATH = os.path.join(_HERE, "_ref", "libts2_opt_ref.so")


def reference_add_delta(weights, avg_grad, grad, row_disp, sum_weight, sparsity, step):
    """The reference's own host-side optimizer step, THostModelMatrix::AddDelta (src/gpt/matrix/host_matrix.cpp:123-157),
    compiled from its sources (oracle/opt_ref.cpp).  The gradient goes in as fp32 and is put into the reference's delta
    form (fp16 values times a power-of-two scale per row).  Returns (weights, avg_grad, row_disp, sum_weight, sum2,
    grad_seen): grad_seen is the gradient as the reference then sees it - feed THAT to a restatement under test."""
    lib = C.CDLL(OPT_REF_PATH)
    w = np.ascontiguousarray(weights, np.float32).copy()
    ag = np.ascontiguousarray(avg_grad, np.float32).copy()
    g = np.ascontiguousarray(grad, np.float32)
    rd = np.ascontiguousarray(row_disp, np.float32).copy()
    seen = np.zeros_like(g)
    sw, sum2 = C.c_float(sum_weight), C.c_float()
    y, x = w.shape
    lib.ts2ref_add_delta.argtypes = [_fp, _fp, _fp, C.c_longlong, C.c_longlong, _fp, C.c_longlong, _fp] + [C.c_float] * 7 + [_fp, _fp]
    lib.ts2ref_add_delta.restype = C.c_int
    rc = lib.ts2ref_add_delta(_f(w), _f(ag), _f(g), x, y, _f(rd), len(rd), C.cast(C.byref(sw), _fp), sparsity, step.rate, step.l2reg,
                              step.beta1, step.weight0, step.weight1, step.disp_decay, _f(seen), C.cast(C.byref(sum2), _fp))
    if rc != 0:
        raise ValueError("ts2ref_add_delta: x must be a multiple of 8 and row_disp must divide the rows")
    return w, ag, rd, sw.value, sum2.value, seen
