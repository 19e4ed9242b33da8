#!/usr/bin/env python
"""Headline benchmark: training tokens/s (forward + backward + gradient apply) of the dense
12-block GPT of BASELINE.json (dim 768, 12 heads of the reference's fixed head width 128,
FFN 3072, vocab 50304, 64 sequences x 1024 tokens per GPU, e4m3 contractions) on N B200s,
data parallel.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference        # the reference's CPU path on the host cores

Prints one JSON line (rank 0).  Inputs are seeded uniform random tokens, weights N(0, 0.02).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from tscale2_b200 import capi, host  # noqa: E402

WORKLOADS = {
    # BASELINE.json configs[2]
    "c3_dense12_d768": dict(dim=768, heads=12, ffn_tiles=24, vocab=50304, blocks=12, seq=1024, seqs=64),
    # BASELINE.json configs[0], for quick checks
    "c1_dense2_d256": dict(dim=256, heads=4, ffn_tiles=8, vocab=4096, blocks=2, seq=128, seqs=4),
    # BASELINE.json configs[3]: 12 attention + mixture-of-experts blocks, 32 experts of width 1024, 2 selected; on more
    # than one GPU the experts are divided over the ranks (--expert-parallel 0: every rank computes all experts)
    "c4_moe12_d1024": dict(dim=1024, heads=16, ffn_tiles=8, vocab=50304, blocks=12, seq=1024, seqs=32, experts=32, selected=2,
                           expert_dim=1024),
    # BASELINE.json configs[4]: 24 blocks, dim 2048, 16 heads, FFN 8192, 8 sequences of 4096 tokens per GPU
    "c5_dense24_d2048": dict(dim=2048, heads=16, ffn_tiles=64, vocab=50304, blocks=24, seq=4096, seqs=8),
}




def make_spec(w, precision):
    moe = "experts" in w
    spec = host.ModelSpec(dim=w["dim"], head_count=w["heads"], ffn_tiles=w["ffn_tiles"], vocab=w["vocab"],
                          attention_widths=[w["seq"]], precision=precision, expert_dim=w.get("expert_dim", 128),
                          moe_expert_count=w.get("experts", 0), moe_selected=w.get("selected", 2))
    return spec.add_blocks(w["blocks"], moe=moe)


def flops_per_token(w):
    """Algorithmic contraction work, no recompute and no padding: 6 flops per parameter of every
    linear layer (2 forward, 4 backward) plus the attention core (forward 4*w*128*H per token at
    mean causal width w = seq/2, backward 2.5x)."""
    d, q, f = w["dim"], 128 * w["heads"], 128 * w["ffn_tiles"]
    if "experts" in w:  # per token: the selected experts' three matrices and the router
        ffn = 3 * d * w["expert_dim"] * w["selected"] + d * w["experts"]
    else:
        ffn = 3 * d * f
    p = w["blocks"] * (5 * d * q + ffn) + w["vocab"] * d
    att = w["blocks"] * 3.5 * 4 * (w["seq"] / 2) * q
    return 6.0 * p + att, 4.0 * p


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.samples, self.proc = device, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.device), f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], 0, set()
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx = max(mx, float(s[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def run_cpu_reference(w, steps, warmup):
    """The reference's CPU path (oracle/_ref: its own compiled cpu_util.cpp, layer_att_reference.h,
    rope.cpp, att.cpp under the restated layer drivers; the restated port where that build is absent)
    on a bounded sample of the workload: the same model, one fragment of `n_tok` tokens per step."""
    import oracle
    kind = "reference" if oracle.have_reference_build() else "port"
    if kind == "port" and not os.path.exists(oracle.PORT_PATH):
        oracle.build()
    if kind == "reference":
        os.environ["OMP_NUM_THREADS"] = "1"
    orc = oracle.Oracle("ref" if kind == "reference" else "port")
    cores = 1 if kind == "reference" else (os.cpu_count() or 1)
    spec = make_spec(w, capi.PREC_FP8)
    mats = host.init_weights(spec, 1000)
    fpt, _ = flops_per_token(w)
    n_tok = int(max(4, min(w["seq"], round(12e9 / fpt))))  # ~10-20 s of scalar fp32 per step
    times = []
    for i in range(warmup + steps):
        batch = host.Batch(np.random.default_rng(2000 + i).integers(0, spec.vocab, (1, n_tok + 1)), spec.attention_widths)
        r = orc.backprop(spec, mats, batch, oracle.QUANT_E4M3)
        if i >= warmup:
            times.append(r["seconds"])
    sec = float(np.mean(times))
    return dict(value=n_tok / sec, unit="tokens/s", cores=cores, kind=kind,
                sample=f"{w_name(w)} model, 1 fragment of {n_tok} tokens per step, {len(times)} step(s), "
                       f"{sec:.2f} s/step, single-threaded scalar fp32" if kind == "reference" else
                       f"{w_name(w)} model, 1 fragment of {n_tok} tokens per step, OpenMP over rows"), n_tok, sec


def measure_cublaslt_fp8(seconds=1.5):
    """Dense e4m3 x e4m3 -> bf16 rate of the vendor library on this GPU (torch._scaled_mm, 8192^3): best of 10 launches
    (burst) and back to back for `seconds` (sustained, power-capped).  MEASURED_PEAKS.json has no fp8 figure; this one is
    reported beside the 2 x bf16 working peak, it is not the denominator of roofline.frac."""
    import torch
    try:
        n = 8192
        a = torch.randn(n, n, device="cuda").to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device="cuda").to(torch.float8_e4m3fn).t()
        one = torch.ones((), device="cuda")
        f = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        for _ in range(3):
            f()
        torch.cuda.synchronize()
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            f()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        reps = max(10, int(seconds * 1e3 / best))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            f()
        e1.record()
        torch.cuda.synchronize()
        flops = 2.0 * n ** 3
        return {"burst": flops / best / 1e9, "sustained": flops * reps / e0.elapsed_time(e1) / 1e9, "how": "torch._scaled_mm e4m3 8192^3 -> bf16"}
    except Exception as e:  # an absent or changed private API must not cost the bench line
        return {"unavailable": str(e)[:200]}


def run_c2_gemm(args):
    """BASELINE.json configs[1], the backward-GEMM microbench: X int8 [16384 x 4096] with per-row scales ~U(0.01, 0.1),
    W int8 [4096 x 4096] with per-column scales, dY e4m3 [16384 x 4096] ~ N(0,1); dX = dY . W^T and dW = X^T . dY, fp32
    accumulate, bf16 output, one GPU.  A mixed fp8 x int8 MMA does not exist, so two variants are timed:
      fp8 : X and W converted to e4m3, dY e4m3;
      int8: X and W as they are, dY quantized to int8 (per row for dX, per column for dW).
    Scales that lie along the contraction (W's column scales for dX, X's row scales for dW) cannot be applied in an
    epilogue; they are folded into dY when it is (re)quantized, once, outside the timed region; the scales across the
    output (the int8 row / column scales of dY) are applied in the epilogue.  Every launch is timed with CUDA events on
    its stream; operands + output of a launch are 208 - 224 MB (> L2).  A few output rows are checked against float64."""
    import ctypes as C
    import ml_dtypes
    from tscale2_b200.device import DeviceBuffer, check, sync
    lib = capi.load_library()
    T, n_in, n_out = 16384, 4096, 4096
    rng = np.random.default_rng(1)
    Xq = rng.integers(-127, 128, (T, n_in), dtype=np.int8)
    sx = rng.uniform(0.01, 0.1, T).astype(np.float32)
    Wq = np.random.default_rng(2).integers(-127, 128, (n_in, n_out), dtype=np.int8)
    sw = np.random.default_rng(2).uniform(0.01, 0.1, n_out).astype(np.float32)
    dY = np.random.default_rng(3).standard_normal((T, n_out)).astype(np.float32)
    e4 = ml_dtypes.float8_e4m3fn
    dY_e4 = dY.astype(e4)
    dYf = dY_e4.astype(np.float32)
    dY_x = dYf * sw[None, :]   # operand of dX: W's column scales folded in
    dY_w = dYf * sx[:, None]   # operand of dW: X's row scales folded in
    variants = {}
    # fp8
    variants["fp8"] = dict(prec=capi.PREC_FP8, dx_a=dY_x.astype(e4), dx_b=Wq.astype(np.float32).astype(e4), dx_row=None,
                           dw_a=Xq.astype(np.float32).astype(e4), dw_b=dY_w.astype(e4), dw_col=None)
    # int8: per-row quantization of dY for dX, per-column for dW
    r = np.abs(dY_x).max(1) / 127
    c = np.abs(dY_w).max(0) / 127
    variants["int8"] = dict(prec=capi.PREC_INT8, dx_a=np.rint(dY_x / r[:, None]).astype(np.int8), dx_b=Wq, dx_row=r.astype(np.float32),
                            dw_a=Xq, dw_b=np.rint(dY_w / c[None, :]).astype(np.int8), dw_col=c.astype(np.float32))
    peaks, peak_src = measured_peaks()
    out = {}
    sample = np.arange(0, T, T // 8)[:8]          # rows of dX checked against float64
    sample_w = np.arange(0, n_in, n_in // 8)[:8]  # rows of dW
    for name, v in variants.items():
        A, B = DeviceBuffer.from_numpy(v["dx_a"]), DeviceBuffer.from_numpy(v["dx_b"])
        DX = DeviceBuffer(T * n_in * 2)
        ROW = DeviceBuffer.from_numpy(v["dx_row"]) if v["dx_row"] is not None else None
        A2, B2 = DeviceBuffer.from_numpy(v["dw_a"]), DeviceBuffer.from_numpy(v["dw_b"])
        DW = DeviceBuffer(n_in * n_out * 2)
        COL = DeviceBuffer.from_numpy(v["dw_col"]) if v["dw_col"] is not None else None

        def dx():
            check(lib.ts2_gemm_tn(0, None, v["prec"], capi.OUT_BF16, T, n_in, n_out, A.ptr, n_out, B.ptr, n_out, DX.ptr, n_in, 1.0,
                                  ROW.ptr if ROW else None, None))

        def dw():  # dW[in][out] = X^T . dY: the entry point's "dY" operand is X, its "X" operand is dY
            check(lib.ts2_gemm_dw_scaled(0, None, v["prec"], capi.OUT_BF16, T, n_out, n_in, A2.ptr, B2.ptr, DW.ptr, 1.0, None,
                                         COL.ptr if COL else None, None, 0))
        res = {}
        for op, f in (("dx", dx), ("dw", dw)):
            for _ in range(max(args.warmup, 3)):
                f()
            sync()
            check(lib.ts2_set_kernel_timing(None, 1))
            lib.ts2_get_kernel_timing(None, 1, None, None, None)
            for _ in range(args.steps):
                f()
            sync()
            ms, n, fl = C.c_double(), C.c_int64(), C.c_double()
            check(lib.ts2_get_kernel_timing(None, 1, C.byref(ms), C.byref(n), C.byref(fl)))
            check(lib.ts2_set_kernel_timing(None, 0))
            res[op] = {"ms": ms.value / n.value, "tflops": fl.value / ms.value / 1e9, "launches": n.value}
        # correctness of what was timed, on a sample of rows, against float64 of the same quantized operands
        got = DX.download((T, n_in), ml_dtypes.bfloat16).astype(np.float64)[sample]
        a64 = v["dx_a"].astype(np.float64)[sample] * (v["dx_row"][sample, None] if v["dx_row"] is not None else 1.0)
        want = a64 @ v["dx_b"].astype(np.float64).T
        res["dx"]["rel_l2_vs_float64"] = float(np.linalg.norm(got - want) / np.linalg.norm(want))
        got = DW.download((n_in, n_out), ml_dtypes.bfloat16).astype(np.float64)[sample_w]
        want = v["dw_a"].astype(np.float64)[:, sample_w].T @ (v["dw_b"].astype(np.float64) * (v["dw_col"][None, :] if v["dw_col"] is not None else 1.0))
        res["dw"]["rel_l2_vs_float64"] = float(np.linalg.norm(got - want) / np.linalg.norm(want))
        assert res["dx"]["rel_l2_vs_float64"] < 5e-3 and res["dw"]["rel_l2_vs_float64"] < 5e-3, res  # bf16 output rounding
        out[name] = res
    flops = 2.0 * T * n_in * n_out
    f8 = out["fp8"]
    both_ms = f8["dx"]["ms"] + f8["dw"]["ms"]
    achieved = 2 * flops / both_ms / 1e9
    peak = 2.0 * peaks["bf16_tflops"]
    vendor = measure_cublaslt_fp8()
    line = {"metric": "bwd GEMM TFLOP/s (dX + dW)", "value": achieved, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": both_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "e4m3", "data": "synthetic",
            "config": {"workload": "c2_gemm", "tokens": T, "in": n_in, "out": n_out, "variant": "fp8 (headline); int8 under variants",
                       "l2": "operands and output of one launch are 208-224 MB, larger than L2"},
            "variants": out,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": None,
                         "kernel": "gemm_kernel (tcgen05), isolated launches", "fp8_cublaslt_tflops": vendor,
                         "peak_source": f"2 x bf16_tflops (burst: isolated launches) of MEASURED_PEAKS.json ({peak_src}); nominal dense fp8 is 4500"},
            "gpu_launches": int(2 * 2 * args.steps)}
    print(json.dumps(line))


def check_steps(model, n, arm):
    """A step that produced a non-finite loss or gradient did not do the work it is timed for: no number."""
    losses = model.loss_history(min(n, 256))
    first_bad, steps = model.step_health(reset=True)
    if not np.isfinite(losses).all() or first_bad.any():
        i = int(np.flatnonzero(~np.isfinite(losses))[0]) if not np.isfinite(losses).all() else None
        raise SystemExit(f"bench: {arm}: non-finite step: first bad loss at timed step {None if i is None else i + 1} of {n}; "
                         f"first step (since model creation, now at {steps}) with a non-finite state gradient per layer boundary: "
                         f"{first_bad.tolist()}; refusing to report a throughput")


def w_name(w):
    for k, v in WORKLOADS.items():
        if v is w:
            return k
    return "custom"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3_dense12_d768", choices=sorted(WORKLOADS) + ["c2_gemm"])
    ap.add_argument("--precision", default="fp8", choices=["fp8", "f16", "int8"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--expert-parallel", type=int, default=1, choices=[0, 1],
                    help="mixture-of-experts workloads on more than one GPU: divide the experts over the ranks")
    args = ap.parse_args()
    if args.workload == "c2_gemm":
        if args.impl == "reference" or args.gpus != 1:
            print(json.dumps({"impl": args.impl, "unavailable": "c2_gemm is a one-GPU kernel microbench of this library"}))
            return
        run_c2_gemm(args)
        return
    w = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    tokens_per_gpu = w["seq"] * w["seqs"]
    config = {"workload": args.workload, "blocks": w["blocks"], "dim": w["dim"], "heads": w["heads"], "head_dim": 128,
              "ffn": 128 * w["ffn_tiles"], "vocab": w["vocab"], "seq_len": w["seq"], "sequences_per_gpu": w["seqs"],
              "global_tokens_per_step": tokens_per_gpu * args.gpus, "parallelism": f"dp{args.gpus}",
              "l2": "inputs larger than L2 (activations of one step are several GB)"}
    if "experts" in w:
        config.update({"experts": w["experts"], "experts_selected": w["selected"], "expert_ffn": w["expert_dim"]})

    if args.impl == "reference":
        if rank != 0:
            return
        ran_steps, ran_warmup = max(1, min(args.steps, 3)), min(args.warmup, 1)
        cb, n_tok, sec = run_cpu_reference(w, ran_steps, ran_warmup)
        config = dict(config, sample_tokens_per_step=n_tok, sample="one fragment of the workload's model per step, see cpu_baseline.sample")
        # steps / warmup are the ones this arm ran (each is ~10-20 s of scalar CPU work), not the ones asked for
        line = {"impl": "reference", "metric": "train tokens/s (fwd+bwd)", "value": cb["value"], "unit": "tokens/s",
                "n_gpus": args.gpus, "steps": ran_steps, "warmup": ran_warmup, "steps_requested": args.steps,
                "warmup_requested": args.warmup, "ms_per_step": sec * 1e3,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": config, "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    import torch
    import torch.distributed as dist
    from tscale2_b200.model import Model, comm_unique_id

    if args.gpus != world:
        print(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run", file=sys.stderr)
        sys.exit(2)
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    precision = {"fp8": capi.PREC_FP8, "f16": capi.PREC_F16, "int8": capi.PREC_INT8}[args.precision]
    spec = make_spec(w, precision)
    # same weights on every rank; router weights N(0, 1) for the mixture-of-experts workload (BASELINE.json configs[3])
    mats = host.init_weights(spec, 1000, select_std=1.0 if "experts" in w else None)
    model = Model(spec, mats, tokens_per_gpu, device=local_rank)
    del mats
    if world > 1:
        ids = [comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        model.comm_init(rank, world, ids[0])
        if "experts" in w and args.expert_parallel and w["experts"] % world == 0:
            # capacity = the worst case (every row of every rank on one rank): the synthetic router (weights N(0, 1), no
            # balancing term) sends up to ~3x a rank's share to the most popular experts
            model.set_expert_parallel(float(world))
            config["parallelism"] = f"dp{world} x ep{world} (experts divided over the ranks, rows exchanged with ncclSend / ncclRecv)"

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    total_steps = args.warmup + args.steps
    batches = [host.synthetic_batch(spec, w["seqs"], w["seq"], 1000 + rank + 97 * i) for i in range(min(total_steps, 4))]
    train_step = host.training_step(rate=0.01, iteration=10)

    # ---- device-timed arm: inputs resident, K steps bracketed by events on the engine's stream ----
    model.set_batch(batches[0])
    for _ in range(args.warmup):
        model.backprop(train_step, apply=True)
    model.wait()
    barrier()
    model.set_kernel_timing(True)
    model.get_kernel_timing(reset=True)
    model.launch_count(reset=True)
    ep_on = "ep" in config["parallelism"]
    if ep_on:
        model.exchange_timing(True)
    sampler = ClockSampler(local_rank)
    sampler.start()
    model.timer_begin()
    for _ in range(args.steps):
        model.backprop(train_step, apply=True)
    ms = model.timer_end()
    launches = model.launch_count()
    barrier()
    exchange = None
    if ep_on:  # device time of the row exchanges (events on the compute stream), this rank
        x_ms, x_bytes, x_n = model.exchange_timing(False)
        exchange = {"ms_per_step": x_ms / args.steps, "gb_sent_per_step": x_bytes / args.steps / 1e9,
                    "gbs_per_direction": x_bytes / 1e9 / max(x_ms / 1e3, 1e-9), "exchanges_per_step": x_n / args.steps}
    clocks = sampler.stop()
    # every step of the timed region is checked afterwards (no device read inside it): the per-step training error
    # from the engine's loss ring, and the per-layer-boundary flags the norm-backward kernel raises on a NaN / infinity
    check_steps(model, args.steps, "device-timed arm")
    gemm_bytes = model.get_kernel_bytes()
    gemm_classes = model.get_kernel_timing_by_class()
    gemm_ms, gemm_n, gemm_flops = model.get_kernel_timing(reset=True)
    model.set_kernel_timing(False)

    # ---- end-to-end arm: every step uploads its batch from pinned host memory and reads the loss back ----
    for i in range(min(args.warmup, 2)):
        model.set_batch(batches[i % len(batches)])
        model.backprop(train_step, apply=True)
        model.avg_train_err()
    barrier()
    loss = 0.0
    e2e_losses = []
    model.timer_begin()  # events on the engine's stream: copies, kernels and the idle gaps between steps
    for i in range(args.steps):
        model.set_batch(batches[i % len(batches)])
        model.backprop(train_step, apply=True)
        loss = model.avg_train_err()  # device -> host read, waits for the step
        e2e_losses.append(loss)
    e2e_ms = model.timer_end()
    barrier()
    if not np.isfinite(e2e_losses).all():
        bad = int(np.flatnonzero(~np.isfinite(e2e_losses))[0])
        raise SystemExit(f"bench: end-to-end arm: training loss is {e2e_losses[bad]} at timed step {bad + 1}; "
                         "refusing to report a throughput")
    check_steps(model, args.steps, "end-to-end arm")
    t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max, e2e_ms_max = float(t[0]), float(t[1])
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    b0 = batches[0]
    # what ts2_set_batch copies: labels (CSR), one target per node, 4 per-node span arrays per attention type
    h2d_bytes = int(b0.label_arr.nbytes + b0.label_ptr.nbytes + 4 * b0.node_count + 16 * b0.node_count * len(b0.att))
    global_tokens = tokens_per_gpu * world
    value = global_tokens * args.steps / (ms_max / 1e3)
    e2e_value = global_tokens * args.steps / (e2e_ms_max / 1e3)
    peaks, peak_src = measured_peaks()
    fpt, bwd_fpt = flops_per_token(w)
    # dominant kernel: the tcgen05 contraction (all forward, dX and dW launches of the step)
    achieved = gemm_flops / (gemm_ms / 1e3) / 1e12 if gemm_ms > 0 else None
    if args.precision in ("fp8", "int8"):
        peak = 2.0 * peaks["bf16_tflops_sustained"]
        peak_note = f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peak_src}); no fp8 / int8 peak is measured there"
    else:
        peak = peaks["bf16_tflops_sustained"]
        peak_note = f"bf16_tflops_sustained of MEASURED_PEAKS.json ({peak_src})"
    # DRAM traffic per launch needs ncu, so it is not measured in this run.  For the headline workload it comes from a
    # small-case capture (profiles/gemm_dram_traffic_one_block_step.md): one block of the same model at the same number
    # of nodes launches exactly the contractions of one layer pair and of the final layer; 12 x the layer launches + the
    # final layer's moved 0.980 x the algorithmic bytes the library counted for the same launches (operands once, outputs
    # once; the last lines written are still in L2 when a kernel ends).  Other workloads: null.
    traffic = None
    if args.workload == "c3_dense12_d768" and args.precision == "fp8" and gemm_n:
        traffic = 0.980 * gemm_bytes / gemm_n
    by_class = {}
    for name, (c_ms, c_n, c_fl) in gemm_classes.items():
        if c_n:
            by_class[name] = {"tflops": c_fl / c_ms / 1e9, "ms_per_step": c_ms / args.steps, "launches_per_step": c_n / args.steps}
    # the target of the north star is stated on the backward contractions of the layers alone (dX + dW, operand format)
    bw_ms = gemm_classes["dx"][0] + gemm_classes["dw"][0]
    bw_fl = gemm_classes["dx"][2] + gemm_classes["dw"][2]
    backward = {"tflops": bw_fl / bw_ms / 1e9, "frac": bw_fl / bw_ms / 1e9 / peak, "ms_per_step": bw_ms / args.steps} if bw_ms > 0 else None
    vendor_fp8 = measure_cublaslt_fp8() if (args.precision == "fp8" and world == 1) else None
    if vendor_fp8 and backward and "sustained" in vendor_fp8:
        backward["frac_of_cublaslt_fp8_sustained"] = backward["tflops"] / vendor_fp8["sustained"]
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": (achieved / peak) if achieved else None, "traffic": traffic,
                "traffic_source": ("small-case ncu capture scaled by the units processed: 0.980 x algorithmic bytes "
                                   "(profiles/gemm_dram_traffic_one_block_step.md)") if traffic else None,
                "algorithmic_bytes_per_launch": gemm_bytes / gemm_n if gemm_n else None,
                "hbm_gbs_algorithmic": gemm_bytes / (gemm_ms / 1e3) / 1e9 if gemm_ms > 0 else None,
                "hbm_peak_gbs": peaks.get("hbm_gbs"), "kernel": "gemm_kernel (tcgen05)",
                "launches_per_step": gemm_n / args.steps, "share_of_step": gemm_ms / ms_max, "peak_source": peak_note,
                "step_flops_per_token": fpt, "step_tflops": value / world * fpt / 1e12,
                "by_class": by_class, "backward_gemm": backward, "fp8_cublaslt_tflops": vendor_fp8}
    line = {"metric": "train tokens/s (fwd+bwd)", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_max / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": {"fp8": "e4m3", "f16": "f16", "int8": "int8 (dW contractions fp16)"}[args.precision], "data": "synthetic", "config": config,
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms_max / args.steps, "last_loss": loss,
                    "losses_checked": len(e2e_losses)},
            "gpu_launches": int(launches), "roofline": roofline}
    if exchange:
        line["expert_exchange"] = exchange
    if world == 1 and not args.no_cpu_baseline:
        cb, _, _ = run_cpu_reference(w, 1, 0)
        line["cpu_baseline"] = cb
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
