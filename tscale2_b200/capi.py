"""ctypes view of include/ts2_b200.h: the structs of the C ABI and the loader
of the CUDA library.  No torch types cross this boundary."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libts2b200.so")

TS2_OK = 0
TS2_ERR_INVALID_ARG, TS2_ERR_NO_DEVICE, TS2_ERR_CUDA, TS2_ERR_UNSUPPORTED = -1, -2, -3, -4
TS2_ERR_TOO_LARGE, TS2_ERR_TIMEOUT, TS2_ERR_COMM, TS2_ERR_DEVICE_STATUS = -5, -6, -7, -8
LAYER_ATT, LAYER_ATT_3LIN, LAYER_FFN, LAYER_MOE = 0, 1, 2, 3
MPF_DISABLE_TUNE_EMBED, MPF_DISABLE_TUNE_FINAL_LAYER, MPF_DISABLE_TUNE_LAYERS = 0x8, 0x4000, 0x8000
PREC_FP8, PREC_F16, PREC_INT8 = 0, 1, 2
GRADIENT_ACCUMULATE, GRADIENT_APPLY = 0, 1
LABEL_NEGATIVE, LABEL_MASK = 0x80000000, 0x7FFFFFFF
PARAM_WEIGHTS, PARAM_MOMENTUM, PARAM_GRADIENT = 0, 1, 2
OUT_F32, OUT_F32_ADD, OUT_F16, OUT_BF16 = 0, 1, 2, 3
COMM_ID_BYTES = 128


class LayerParams(C.Structure):
    _fields_ = [("layer_type", C.c_int32), ("alibi_slope", C.c_float), ("attention_type_id", C.c_int32)]


class ModelDescr(C.Structure):
    _fields_ = [
        ("dim", C.c_int32), ("q_dim", C.c_int32), ("tt_dim", C.c_int32), ("head_count", C.c_int32),
        ("ffn_tiles", C.c_int32), ("expert_dim", C.c_int32), ("moe_expert_count", C.c_int32),
        ("moe_selected", C.c_int32), ("label_count", C.c_int32), ("output_token_count", C.c_int32),
        ("attention_type_count", C.c_int32), ("layer_count", C.c_int32),
        ("layers", C.POINTER(LayerParams)), ("flags", C.c_uint64), ("precision", C.c_int32),
        ("reserved", C.c_int32),
    ]


class MatrixView(C.Structure):
    _fields_ = [("data", C.POINTER(C.c_float)), ("x_size", C.c_int64), ("y_size", C.c_int64)]


class AttentionInfo(C.Structure):
    _fields_ = [("span_start", C.POINTER(C.c_int32)), ("span_finish", C.POINTER(C.c_int32)),
                ("span_ptr", C.POINTER(C.c_int32))]


class BatchNodes(C.Structure):
    _fields_ = [
        ("node_count", C.c_int32), ("label_arr", C.POINTER(C.c_uint32)), ("label_ptr", C.POINTER(C.c_uint32)),
        ("target_count", C.c_int32), ("target_node", C.POINTER(C.c_int32)), ("target_id", C.POINTER(C.c_int32)),
        ("attention_type_count", C.c_int32), ("att", C.POINTER(AttentionInfo)),
    ]


class TrainingStep(C.Structure):
    _fields_ = [("rate", C.c_float), ("l2reg", C.c_float), ("beta1", C.c_float), ("weight0", C.c_float),
                ("weight1", C.c_float), ("disp_decay", C.c_float)]


class Ts2Error(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"ts2 error {code}: {msg}")
        self.code = code


_lib = None


def load_library(path=None):
    """Load the CUDA library.  There is no CPU fallback: a missing library is an error."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    path = path or LIB_PATH
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -m tscale2_b200.build` (needs nvcc); "
            "this package has no CPU fallback")
    lib = C.CDLL(path, mode=C.RTLD_GLOBAL)
    _declare(lib)
    _lib = lib
    return lib


def _declare(lib):
    vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_int64, C.c_float
    P = C.POINTER
    sig = {
        "ts2_matrix_count": (i32, [P(ModelDescr)]),
        "ts2_matrix_shape": (i32, [P(ModelDescr), i32, P(i64), P(i64)]),
        "ts2_create": (i32, [P(ModelDescr), P(MatrixView), i32, P(f32), i32, i32, P(vp)]),
        "ts2_destroy": (None, [vp]),
        "ts2_last_error": (C.c_char_p, [vp]),
        "ts2_set_batch": (i32, [vp, P(BatchNodes)]),
        "ts2_backprop": (i32, [vp, P(TrainingStep), i32]),
        "ts2_wait": (i32, [vp]),
        "ts2_forward_score": (i32, [vp, P(f32)]),
        "ts2_avg_train_err": (i32, [vp, P(f32)]),
        "ts2_get_params": (i32, [vp, i32, P(MatrixView), i32]),
        "ts2_set_params": (i32, [vp, i32, P(MatrixView), i32]),
        "ts2_get_batch_tables": (i32, [vp, i32, vp, vp, vp, vp, vp]),
        "ts2_get_label_index": (i32, [vp, vp, vp, i64, P(i64)]),
        "ts2_get_row_disp": (i32, [vp, i32, P(f32), i64, P(f32)]),
        "ts2_set_row_disp": (i32, [vp, i32, P(f32), i64, f32]),
        "ts2_get_fast_weights": (i32, [vp, i32, vp, i64, P(f32)]),
        "ts2_set_debug_taps": (i32, [vp, i32]),
        "ts2_debug_read": (i32, [vp, C.c_char_p, i32, vp, i64]),
        "ts2_get_state_tap": (i32, [vp, i32, i32, P(f32), i64]),
        "ts2_get_step_health": (i32, [vp, i32, P(C.c_uint32), i32, P(i64)]),
        "ts2_get_loss_history": (i32, [vp, P(f32), i32]),
        "ts2_discard_gradient": (i32, [vp]),
        "ts2_set_debug_trace": (i32, [vp, i32]),
        "ts2_get_debug_trace": (i32, [vp, P(C.c_uint64), P(C.c_uint64), P(f32), i32, P(i32)]),
        "ts2_set_debug_capture": (i32, [vp, C.c_char_p, i64]),
        "ts2_debug_trace_name": (C.c_char_p, [vp, i32]),
        "ts2_dp_layout": (i32, [P(ModelDescr), P(i64), i32, P(i64), P(i64), P(C.c_int32), i32]),
        "ts2_comm_unique_id": (i32, [P(C.c_uint8)]),
        "ts2_comm_init": (i32, [vp, i32, i32, P(C.c_uint8)]),
        "ts2_set_expert_parallel": (i32, [vp, f32]),
        "ts2_get_exchange_ms": (i32, [vp, i32, P(f32), P(C.c_double), P(i32)]),
        "ts2_moe_exchange_plan": (i32, [i32, i32, i32, vp, vp, vp, vp, vp, i32, P(i32), P(i32), P(i32)]),
        "ts2_launch_count": (i64, [vp, i32]),
        "ts2_last_step_ms": (i32, [vp, P(f32)]),
        "ts2_timer_begin": (i32, [vp]),
        "ts2_timer_end": (i32, [vp, P(f32)]),
        "ts2_set_kernel_timing": (i32, [vp, i32]),
        "ts2_get_kernel_timing": (i32, [vp, i32, P(C.c_double), P(i64), P(C.c_double)]),
        "ts2_get_kernel_bytes": (i32, [vp, P(C.c_double)]),
        "ts2_get_kernel_timing_class": (i32, [vp, i32, P(C.c_double), P(i64), P(C.c_double)]),
        "ts2_gemm_dw_scaled": (i32, [i32, vp, i32, i32, i64, i64, i64, vp, vp, vp, f32, vp, vp, vp, C.c_size_t]),
        "ts2_device_count": (i32, []),
        "ts2_selftest_wait_limit": (i32, [i32]),
        "ts2_selftest_wait_limit_noalloc": (i32, [i32]),
        "ts2_dev_alloc": (i32, [i32, C.c_size_t, P(vp)]),
        "ts2_dev_free": (i32, [i32, vp]),
        "ts2_dev_upload": (i32, [i32, vp, vp, C.c_size_t]),
        "ts2_dev_download": (i32, [i32, vp, vp, C.c_size_t]),
        "ts2_dev_memset": (i32, [i32, vp, i32, C.c_size_t]),
        "ts2_dev_sync": (i32, [i32]),
        "ts2_gemm_tn": (i32, [i32, vp, i32, i32, i64, i64, i64, vp, i64, vp, i64, vp, i64, f32, vp, vp]),
        "ts2_gemm_dx": (i32, [i32, vp, i32, i32, i64, i64, i64, vp, vp, vp, f32, vp, vp]),
        "ts2_gemm_dw_workspace_bytes": (C.c_size_t, [i64, i64, i64]),
        "ts2_gemm_dw_noalloc": (i32, [i32, vp, i32, i32, i64, i64, i64, vp, vp, vp, f32]),
        "ts2_gemm_tn_grouped": (i32, [i32, vp, i32, i32, i64, i64, i64, vp, vp, vp, f32, i32, vp]),
        "ts2_gemm_dw_grouped": (i32, [i32, vp, i32, i32, i64, i64, i64, vp, vp, vp, f32, i32, vp]),
        "ts2_moe_route": (i32, [i32, vp, i32, i32, i32, vp, vp]),
        "ts2_op_tilenorm_backward": (i32, [i32, vp, vp, vp, vp, i32, i32, vp, i32, vp]),
        "ts2_op_cast_grad": (i32, [i32, vp, i32, vp, i64, vp, vp, vp]),
        "ts2_op_ffn_act_backward": (i32, [i32, vp, i32, vp, vp, vp, i32, i32, vp]),
        "ts2_op_att_gate_backward": (i32, [i32, vp, i32, vp, vp, vp, i32, i32, vp, vp, vp]),
        "ts2_op_rowquant_i8": (i32, [i32, vp, vp, i32, i32, vp, vp]),
        "ts2_op_attention_reverse_ranges": (i32, [i32, vp, vp, vp, i32, vp, vp]),
        "ts2_attention_forward": (i32, [i32, vp, i32, vp, vp, vp, vp, vp, i32, i32, f32, vp, vp]),
        "ts2_attention_backward": (i32, [i32, vp, i32, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, f32, vp, vp, vp]),
        "ts2_gemm_dw": (i32, [i32, vp, i32, i32, i64, i64, i64, vp, vp, vp, f32, vp, C.c_size_t]),
    }
    missing = []
    for name, (res, args) in sig.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            missing.append(name)
            continue
        fn.restype = res
        fn.argtypes = args
    lib._ts2_signatures = sig
    lib._ts2_missing = missing  # tests assert this is empty
