"""Operator-level micro-benchmarks through the C ABI (no torch): the contraction kernels at the
shapes of BASELINE config 2 (backward GEMM microbench) or any other shape, and the attention core.

    python -m tscale2_b200.microbench --op dx --prec fp8 --M 16384 --N 4096 --K 4096
    python -m tscale2_b200.microbench --op dw --prec int8 --M 4096 --N 4096 --K 16384   # dW[M][N], K tokens
    python -m tscale2_b200.microbench --op config2
    python -m tscale2_b200.microbench --op att --T 16384 --heads 12 --variant 3      # attention forward + backward
    python -m tscale2_b200.microbench --op step --blocks 1 --T 65536 --iters 2       # training steps of a short model

Times with CUDA events around each launch on the launching stream (ts2_set_kernel_timing); operands are
random bytes of the operand format (no NaN codes), larger than L2 for the config-2 shapes.  One JSON line
per measurement."""
import argparse
import ctypes as C
import json

import numpy as np

from . import capi
from .device import DeviceBuffer, check, sync

PREC = {"fp8": (capi.PREC_FP8, 1), "f16": (capi.PREC_F16, 2), "int8": (capi.PREC_INT8, 1)}


def _operand(rng, n_elems, es):
    if es == 1:
        return rng.integers(0, 256, n_elems, dtype=np.uint8) & np.uint8(0xBF)  # clears bit 6: |e4m3| < 2, no NaN; any int8
    return rng.standard_normal(n_elems).astype(np.float16)


def time_gemm(lib, op, prec_name, M, N, K, iters, warmup=3):
    prec, es = PREC[prec_name]
    rng = np.random.default_rng(1)
    A = DeviceBuffer.from_numpy(_operand(rng, M * K, es))
    B = DeviceBuffer.from_numpy(_operand(rng, N * K, es))
    if op == "dw":
        Cb = DeviceBuffer(M * N * 4)
        ws_bytes = lib.ts2_gemm_dw_workspace_bytes(K, N, M)
        WS = DeviceBuffer(max(ws_bytes, 16))

        def run():
            check(lib.ts2_gemm_dw(0, None, prec, capi.OUT_F32, K, N, M, A.ptr, B.ptr, Cb.ptr, 1.0, WS.ptr, ws_bytes))
    else:
        Cb = DeviceBuffer(M * N * 2)

        def run():
            check(lib.ts2_gemm_tn(0, None, prec, capi.OUT_BF16, M, N, K, A.ptr, K, B.ptr, K, Cb.ptr, N, 1.0, None, None))
    for _ in range(warmup):
        run()
    sync()
    check(lib.ts2_set_kernel_timing(None, 1))
    lib.ts2_get_kernel_timing(None, 1, None, None, None)
    for _ in range(iters):
        run()
    sync()
    ms, n, fl = C.c_double(), C.c_int64(), C.c_double()
    check(lib.ts2_get_kernel_timing(None, 1, C.byref(ms), C.byref(n), C.byref(fl)))
    check(lib.ts2_set_kernel_timing(None, 0))
    per = ms.value / max(n.value, 1)
    return {"op": op, "prec": prec_name, "M": M, "N": N, "K": K, "ms": per, "tflops": 2.0 * M * N * K / per / 1e9,
            "launches": n.value, "layout": "dW[M][N] = dY[K][M]^T . X[K][N] (token-major operands)" if op == "dw"
            else "C[M][N] = A[M][K] . B[N][K]^T"}


def time_attention(lib, T, heads, variant, iters, warmup=2, doc=1024):
    """Forward and backward attention core over documents of `doc` tokens with a causal window of the same length.
    The times include the entry points' host work (span upload, reverse ranges): the kernels' own times are what a
    profiler run of this command shows."""
    import time
    rng = np.random.default_rng(1)
    Q = heads * 128
    q, k, v, do = (DeviceBuffer.from_numpy(rng.standard_normal((T, Q)).astype(np.float16)) for _ in range(4))
    o, lse, dsc = DeviceBuffer(T * Q * 2), DeviceBuffer(T * heads * 4), DeviceBuffer.from_numpy(np.zeros((T, heads), np.float32))
    gb = 2 if variant == 3 else 4
    dq, dk, dv = (DeviceBuffer(T * Q * gb) for _ in range(3))
    t = np.arange(T)
    start = np.maximum((t // doc) * doc, t - doc).astype(np.int32)
    finish = (t - 1).astype(np.int32)
    none = finish < start
    start[none], finish[none] = 0, -1
    ip = lambda a: a.ctypes.data_as(C.c_void_p)

    def fwd():
        check(lib.ts2_attention_forward(0, None, min(variant, 2), q.ptr, k.ptr, v.ptr, ip(start), ip(finish), T, heads, 0.0, o.ptr, lse.ptr))

    def bwd():
        check(lib.ts2_attention_backward(0, None, variant, q.ptr, k.ptr, v.ptr, do.ptr, lse.ptr, dsc.ptr, ip(start), ip(finish), T, heads,
                                         0.0, dq.ptr, dk.ptr, dv.ptr))
    out = {"op": "att", "T": T, "heads": heads, "variant": variant, "doc": doc}
    for name, f in (("forward", fwd), ("backward", bwd)):
        for _ in range(warmup):
            f()
        sync()
        t0 = time.perf_counter()
        for _ in range(iters):
            f()
        sync()
        out[name + "_ms_incl_host"] = (time.perf_counter() - t0) * 1e3 / iters
    return out


def time_steps(blocks, T, seq, iters, prec_name, dim=768, heads=12, ffn_tiles=24, vocab=50304):
    """Applied training steps of a model with the headline benchmark's layer shapes but only `blocks` blocks: every
    kernel of the step runs at full width on a few GB of device memory, which is what a profiler capture wants."""
    from . import host
    from .model import Model
    spec = host.ModelSpec(dim=dim, head_count=heads, ffn_tiles=ffn_tiles, vocab=vocab, attention_widths=[seq],
                          precision=PREC[prec_name][0]).add_blocks(blocks)
    model = Model(spec, host.init_weights(spec, 1000), T)
    model.set_batch(host.synthetic_batch(spec, T // seq, seq, 1000))
    step = host.training_step(rate=0.01, iteration=10)
    model.backprop(step, apply=True)
    model.wait()
    model.timer_begin()
    for _ in range(iters):
        model.backprop(step, apply=True)
    ms = model.timer_end()
    return {"op": "step", "blocks": blocks, "T": T, "seq": seq, "prec": prec_name, "ms_per_step": ms / iters,
            "loss": model.avg_train_err(), "launches": model.launch_count()}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="config2", choices=["dx", "tn", "dw", "config2", "att", "step"])
    ap.add_argument("--blocks", type=int, default=1)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--T", type=int, default=16384)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--variant", type=int, default=3, choices=[0, 1, 2, 3])
    ap.add_argument("--prec", default="fp8", choices=sorted(PREC))
    ap.add_argument("--M", type=int, default=16384)
    ap.add_argument("--N", type=int, default=4096)
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    lib = capi.load_library()
    if args.op == "step":
        print(json.dumps(time_steps(args.blocks, args.T, args.seq, args.iters, args.prec if args.prec != "int8" else "fp8")))
    elif args.op == "att":
        print(json.dumps(time_attention(lib, args.T, args.heads, args.variant, args.iters, args.warmup)))
    elif args.op == "config2":
        # BASELINE config 2: T = 16384 tokens, 4096 x 4096 weights: dX = dY.W^T (M=T, N=in, K=out), dW = X^T.dY (K = T)
        for prec in ("fp8", "int8", "f16"):
            print(json.dumps(time_gemm(lib, "dx", prec, 16384, 4096, 4096, args.iters, args.warmup)), flush=True)
            print(json.dumps(time_gemm(lib, "dw", prec, 4096, 4096, 16384, args.iters, args.warmup)), flush=True)
    else:
        print(json.dumps(time_gemm(lib, "tn" if args.op == "dx" else args.op, args.prec, args.M, args.N, args.K, args.iters, args.warmup)))


if __name__ == "__main__":
    main()
