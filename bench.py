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
    # BASELINE.json configs[3]: 12 attention + mixture-of-experts blocks, 32 experts of width 1024, 2 selected;
    # every rank holds all experts (no expert-parallel exchange)
    "c4_moe12_d1024": dict(dim=1024, heads=16, ffn_tiles=8, vocab=50304, blocks=12, seq=1024, seqs=32, experts=32, selected=2,
                           expert_dim=1024),
    # BASELINE.json configs[4]: 24 blocks, dim 2048, 16 heads, FFN 8192, 8 sequences of 4096 tokens per GPU
    "c5_dense24_d2048": dict(dim=2048, heads=16, ffn_tiles=64, vocab=50304, blocks=24, seq=4096, seqs=8),
}


# average DRAM bytes per contraction launch from one ncu capture of a whole step (see profiles/)
NCU_GEMM_TRAFFIC_BYTES_PER_LAUNCH = {("c3_dense12_d768", "fp8"): 533793211}


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
    ap.add_argument("--workload", default="c3_dense12_d768", choices=sorted(WORKLOADS))
    ap.add_argument("--precision", default="fp8", choices=["fp8", "f16"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
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
    precision = capi.PREC_FP8 if args.precision == "fp8" else capi.PREC_F16
    spec = make_spec(w, precision)
    # same weights on every rank; router weights N(0, 1) for the mixture-of-experts workload (BASELINE.json configs[3])
    mats = host.init_weights(spec, 1000, select_std=1.0 if "experts" in w else None)
    model = Model(spec, mats, tokens_per_gpu, device=local_rank)
    del mats
    if world > 1:
        ids = [comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        model.comm_init(rank, world, ids[0])

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
    sampler = ClockSampler(local_rank)
    sampler.start()
    model.timer_begin()
    for _ in range(args.steps):
        model.backprop(train_step, apply=True)
    ms = model.timer_end()
    launches = model.launch_count()
    barrier()
    clocks = sampler.stop()
    # every step of the timed region is checked afterwards (no device read inside it): the per-step training error
    # from the engine's loss ring, and the per-layer-boundary flags the norm-backward kernel raises on a NaN / infinity
    check_steps(model, args.steps, "device-timed arm")
    gemm_bytes = model.get_kernel_bytes()
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
    if args.precision == "fp8":
        peak = 2.0 * peaks["bf16_tflops_sustained"]
        peak_note = f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peak_src}); no fp8 peak is measured there"
    else:
        peak = peaks["bf16_tflops_sustained"]
        peak_note = f"bf16_tflops_sustained of MEASURED_PEAKS.json ({peak_src})"
    # DRAM traffic per launch: dram__bytes_read.sum + dram__bytes_write.sum of the 183 contraction launches of one step
    # of this workload, averaged (ncu capture summarised in profiles/gemm_dram_traffic_c3_dense12_d768_step.md);
    # the algorithmic bytes next to it are counted by the library at launch time over the timed region
    traffic = NCU_GEMM_TRAFFIC_BYTES_PER_LAUNCH.get((args.workload, args.precision))
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": (achieved / peak) if achieved else None, "traffic": traffic,
                "algorithmic_bytes_per_launch": gemm_bytes / gemm_n if gemm_n else None,
                "hbm_gbs_algorithmic": gemm_bytes / (gemm_ms / 1e3) / 1e9 if gemm_ms > 0 else None,
                "hbm_peak_gbs": peaks.get("hbm_gbs"), "kernel": "gemm_kernel (tcgen05)",
                "launches_per_step": gemm_n / args.steps, "share_of_step": gemm_ms / ms_max, "peak_source": peak_note,
                "step_flops_per_token": fpt, "step_tflops": value / world * fpt / 1e12}
    line = {"metric": "train tokens/s (fwd+bwd)", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_max / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "e4m3" if args.precision == "fp8" else "f16", "data": "synthetic", "config": config,
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms_max / args.steps, "last_loss": loss,
                    "losses_checked": len(e2e_losses)},
            "gpu_launches": int(launches), "roofline": roofline}
    if world == 1 and not args.no_cpu_baseline:
        cb, _, _ = run_cpu_reference(w, 1, 0)
        line["cpu_baseline"] = cb
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
