"""Host-side mirror of the reference's IModel / IModelInstance (src/gpt/compute/model.h:22-56)
over the C ABI.  Method names follow the reference: GetInstance().Init() is set_batch(),
Backprop(), WaitAllCompute(), GetParams(), ComputeScore(), GetAvrgTrainErr()."""
import ctypes as C
from typing import List

import numpy as np

from . import capi, host
from .device import check


class Model:
    """CreateLocalTransformer (src/gpt/compute/model.cu:257-264) for one B200 driven by this process."""

    def __init__(self, spec: host.ModelSpec, mats: List[np.ndarray], max_nodes: int, device: int = 0, bias=None):
        self.lib = capi.load_library()
        self.spec = spec
        self.device = device
        descr, self._keep = spec.to_c()
        views = host.matrix_views(mats)
        h = C.c_void_p()
        b = None if bias is None else np.ascontiguousarray(bias, np.float32).ctypes.data_as(C.POINTER(C.c_float))
        rc = self.lib.ts2_create(C.byref(descr), views, len(mats), b, device, max_nodes, C.byref(h))
        if rc != capi.TS2_OK:
            raise capi.Ts2Error(rc, self.lib.ts2_last_error(None).decode())
        self.h = h
        self.shapes = spec.matrix_shapes()

    def _check(self, rc):
        if rc != capi.TS2_OK:
            raise capi.Ts2Error(rc, self.lib.ts2_last_error(self.h).decode())

    def close(self):
        if getattr(self, "h", None):
            self.lib.ts2_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # IModelInstance::GetNodes + Init
    def set_batch(self, batch: host.Batch):
        self._check(self.lib.ts2_set_batch(self.h, C.byref(batch.c)))
        self._node_count, self._label_count = batch.node_count, len(batch.label_arr)

    # IModel::Backprop
    def backprop(self, step: capi.TrainingStep, apply: bool = True):
        self._check(self.lib.ts2_backprop(self.h, C.byref(step),
                                          capi.GRADIENT_APPLY if apply else capi.GRADIENT_ACCUMULATE))

    # IModel::WaitAllCompute
    def wait(self):
        self._check(self.lib.ts2_wait(self.h))

    # IModelInstance::ComputeScore
    def compute_score(self) -> float:
        v = C.c_float()
        self._check(self.lib.ts2_forward_score(self.h, C.byref(v)))
        return v.value

    # IModel::GetAvrgTrainErr
    def avg_train_err(self) -> float:
        v = C.c_float()
        self._check(self.lib.ts2_avg_train_err(self.h, C.byref(v)))
        return v.value

    def _get(self, what):
        outs = [np.empty(s, np.float32) for s in self.shapes]
        self._check(self.lib.ts2_get_params(self.h, what, host.matrix_views(outs), len(outs)))
        return outs

    def get_weights(self):
        return self._get(capi.PARAM_WEIGHTS)

    def get_momentum(self):
        return self._get(capi.PARAM_MOMENTUM)

    def get_gradients(self):
        """fp32 weight gradients of the last backprop, before the optimizer: the tensors the
        reference hands to HostApplyDelta."""
        return self._get(capi.PARAM_GRADIENT)

    def set_weights(self, mats):
        self._check(self.lib.ts2_set_params(self.h, capi.PARAM_WEIGHTS, host.matrix_views(mats), len(mats)))

    def set_momentum(self, mats):
        self._check(self.lib.ts2_set_params(self.h, capi.PARAM_MOMENTUM, host.matrix_views(mats), len(mats)))

    def set_row_disp(self, index, row_disp, sum_weight):
        rd = np.ascontiguousarray(row_disp, np.float32)
        self._check(self.lib.ts2_set_row_disp(self.h, index, rd.ctypes.data_as(C.POINTER(C.c_float)), rd.size, float(sum_weight)))

    @classmethod
    def from_file(cls, path, max_nodes, device=0, precision=capi.PREC_FP8):
        """IModel::SetParams from a model file in the reference's format (tscale2_b200/checkpoint.py): weights,
        momentum and the dispersion state of every matrix, so that training resumes where the file was written."""
        from . import checkpoint
        mf = checkpoint.load(path)
        mf.spec.precision = precision
        model = cls(mf.spec, [np.ascontiguousarray(m.weights) for m in mf.matrices], max_nodes, device=device, bias=mf.bias)
        model.set_momentum([np.ascontiguousarray(m.momentum) for m in mf.matrices])
        for i, m in enumerate(mf.matrices):
            model.set_row_disp(i, m.row_disp, m.sum_weight)
        return model

    def save(self, path, bias=None, **kw):
        """IModel::GetParams into a model file the reference's tools can load."""
        from . import checkpoint
        checkpoint.save(path, checkpoint.from_model(self, bias=bias, **kw))

    def batch_tables(self, attention_type=0):
        """The per-node tables the device derived from the current batch: dict of int32 arrays span_start,
        span_finish, rev_first, rev_last, target."""
        T = self._node_count
        out = {k: np.empty(T, np.int32) for k in ("span_start", "span_finish", "rev_first", "rev_last", "target")}
        self._check(self.lib.ts2_get_batch_tables(self.h, attention_type, *[out[k].ctypes.data for k in
                                                  ("span_start", "span_finish", "rev_first", "rev_last", "target")]))
        return out

    def label_index(self):
        """(labels, nodes, negative) of the inverse label index of the current batch, sorted by label."""
        cap = max(1, self._label_count)
        labels, nodes = np.empty(cap, np.uint32), np.empty(cap, np.uint32)
        n = C.c_int64()
        self._check(self.lib.ts2_get_label_index(self.h, labels.ctypes.data, nodes.ctypes.data, cap, C.byref(n)))
        labels, nodes = labels[:n.value], nodes[:n.value]
        return labels, nodes & np.uint32(0x7fffffff), (nodes >> np.uint32(31)).astype(bool)

    def get_row_disp(self, index):
        n = self.shapes[index][0] if index < 2 else 1
        rd = np.empty(n, np.float32)
        sw = C.c_float()
        self._check(self.lib.ts2_get_row_disp(self.h, index, rd.ctypes.data_as(C.POINTER(C.c_float)), n, C.byref(sw)))
        return rd, sw.value

    def get_fast_weights(self, index):
        y, x = self.shapes[index]
        dt = np.float16 if (index == 0 or self.spec.precision == capi.PREC_F16) else np.uint8
        out = np.empty((y, x), dt)
        sko = C.c_float()
        self._check(self.lib.ts2_get_fast_weights(self.h, index, out.ctypes.data, out.nbytes, C.byref(sko)))
        return out, sko.value

    def set_debug_taps(self, enable=True):
        self._check(self.lib.ts2_set_debug_taps(self.h, int(enable)))

    def get_state_tap(self, layer, gradient, node_count):
        out = np.empty((node_count, self.spec.dim), np.float32)
        self._check(self.lib.ts2_get_state_tap(self.h, layer, int(gradient), out.ctypes.data_as(C.POINTER(C.c_float)), out.size))
        return out

    def step_health(self, reset=False):
        """(first_bad_step per layer boundary, steps so far): 0 = the state gradient at that boundary was finite in
        every step since the last reset."""
        n = len(self.spec.layers) + 1
        out = np.zeros(n, np.uint32)
        steps = C.c_int64()
        self._check(self.lib.ts2_get_step_health(self.h, int(reset), out.ctypes.data_as(C.POINTER(C.c_uint32)), n, C.byref(steps)))
        return out, steps.value

    def loss_history(self, n):
        out = np.zeros(n, np.float32)
        self._check(self.lib.ts2_get_loss_history(self.h, out.ctypes.data_as(C.POINTER(C.c_float)), n))
        return out

    def discard_gradient(self):
        self._check(self.lib.ts2_discard_gradient(self.h))

    def set_debug_trace(self, enable=True):
        self._check(self.lib.ts2_set_debug_trace(self.h, int(enable)))

    def get_debug_trace(self):
        """[(name, checksum, non-finite count, largest finite magnitude)] of the last step, in stream order."""
        n = C.c_int()
        self._check(self.lib.ts2_get_debug_trace(self.h, None, None, None, 0, C.byref(n)))
        sums = np.zeros(max(n.value, 1), np.uint64)
        bad = np.zeros(max(n.value, 1), np.uint64)
        mx = np.zeros(max(n.value, 1), np.float32)
        self._check(self.lib.ts2_get_debug_trace(self.h, sums.ctypes.data_as(C.POINTER(C.c_uint64)),
                                                 bad.ctypes.data_as(C.POINTER(C.c_uint64)),
                                                 mx.ctypes.data_as(C.POINTER(C.c_float)), n.value, C.byref(n)))
        return [(self.lib.ts2_debug_trace_name(self.h, i).decode(), int(sums[i]), int(bad[i]), float(mx[i]))
                for i in range(n.value)]

    def set_debug_capture(self, record_name, max_bytes):
        self._check(self.lib.ts2_set_debug_capture(self.h, record_name.encode() if record_name else None, max_bytes))

    def debug_read(self, name, layer, shape, dtype):
        out = np.empty(shape, dtype)
        self._check(self.lib.ts2_debug_read(self.h, name.encode(), layer, out.ctypes.data, out.nbytes))
        return out

    def comm_init(self, rank, world, id_bytes):
        buf = (C.c_uint8 * capi.COMM_ID_BYTES).from_buffer_copy(id_bytes)
        self._check(self.lib.ts2_comm_init(self.h, rank, world, buf))

    def set_expert_parallel(self, capacity_factor=0.0):
        """After comm_init, on every rank: the experts of the mixture-of-experts layers are divided over the ranks and
        the (token, choice) rows travel to the experts' owners and back (ts2_set_expert_parallel)."""
        self._check(self.lib.ts2_set_expert_parallel(self.h, capacity_factor))

    def exchange_timing(self, enable=True):
        """(ms, bytes sent to other ranks, exchanges) of the expert-parallel row exchanges since the last call."""
        ms, nbytes, n = C.c_float(), C.c_double(), C.c_int()
        self._check(self.lib.ts2_get_exchange_ms(self.h, int(enable), C.byref(ms), C.byref(nbytes), C.byref(n)))
        return ms.value, nbytes.value, n.value

    def last_step_ms(self):
        v = C.c_float()
        self._check(self.lib.ts2_last_step_ms(self.h, C.byref(v)))
        return v.value

    def timer_begin(self):
        self._check(self.lib.ts2_timer_begin(self.h))

    def timer_end(self) -> float:
        v = C.c_float()
        self._check(self.lib.ts2_timer_end(self.h, C.byref(v)))
        return v.value

    def set_kernel_timing(self, enable=True):
        self._check(self.lib.ts2_set_kernel_timing(self.h, int(enable)))

    def get_kernel_timing(self, reset=False):
        ms, n, fl = C.c_double(), C.c_int64(), C.c_double()
        self._check(self.lib.ts2_get_kernel_timing(self.h, int(reset), C.byref(ms), C.byref(n), C.byref(fl)))
        return ms.value, n.value, fl.value

    def get_kernel_timing_by_class(self):
        """{class: (ms, launches, flops)} of the contraction launches timed since the last reset (read before a
        resetting get_kernel_timing): forward, dx, dw of the layers, the final layer's three, other."""
        out = {}
        for cls, name in enumerate(("other", "forward", "dx", "dw", "final")):
            ms, n, fl = C.c_double(), C.c_int64(), C.c_double()
            self._check(self.lib.ts2_get_kernel_timing_class(self.h, cls, C.byref(ms), C.byref(n), C.byref(fl)))
            out[name] = (ms.value, n.value, fl.value)
        return out

    def get_kernel_bytes(self):
        """Algorithmic bytes of the contraction launches timed since the last reset (read before a resetting
        get_kernel_timing)."""
        v = C.c_double()
        self._check(self.lib.ts2_get_kernel_bytes(self.h, C.byref(v)))
        return v.value

    def launch_count(self, reset=False):
        return self.lib.ts2_launch_count(self.h, int(reset))


def comm_unique_id() -> bytes:
    lib = capi.load_library()
    buf = (C.c_uint8 * capi.COMM_ID_BYTES)()
    check(lib.ts2_comm_unique_id(buf))
    return bytes(buf)
