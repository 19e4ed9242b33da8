"""Run by test_dp_gpu.py under torchrun, one process per GPU.  Expert parallel on top of data parallel
(ts2_set_expert_parallel): every rank routes its own tokens, the (token, choice) rows travel to the experts' owners and
the results back.  Checked:
  * after one applied step the update of every matrix (new weights - old weights, relative L2) equals that of ONE
    process that accumulates the ranks' batches and applies once.  fp16 operands: the forward pass is identical bit for
    bit (the experts' results return as fp32 in this pipeline), the expert contractions of the backward pass sum the
    same products in another order: 1e-4.  e4m3 operands: results return as fp16, whose 1e-4 flips e4m3 roundings and
    now and then the expert choice of a borderline token downstream, and the ranks agree on one power-of-two gradient
    scale per layer where the single process picks one per batch; the first step's update is normalised by the
    gradient's own magnitude, so it shows every flip: 0.25 (the distance between two e4m3 runs that differ in rounding
    only; measured 0.07 - 0.11);
  * the ranks stay bit-identical over further steps, and the loss stays finite;
  * a capacity too small for the rows a rank would receive is refused on every rank with TS2_ERR_TOO_LARGE.
Switches for a run by hand (any number of GPUs that divides the expert count): TS2_TEST_EP=0 leaves expert parallel off
(the plain data-parallel step of the same model), TS2_TEST_QUICK=1 runs the fp16 pipeline only and skips the capacity
case, TS2_TEST_EXPERTS=n changes the expert count (the capacity case needs at least 4 experts on rank 0)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tscale2_b200 import capi, host  # noqa: E402
from tscale2_b200.model import Model, comm_unique_id  # noqa: E402


def moe_spec(precision):
    s = host.ModelSpec(dim=256, head_count=2, ffn_tiles=4, vocab=1024, attention_widths=[64], expert_dim=256,
                       moe_expert_count=int(os.environ.get("TS2_TEST_EXPERTS", "8")), moe_selected=2, precision=precision)
    return s.add_blocks(1).add_blocks(2, moe=True)


def connect(model, rank, world):
    ids = [comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    model.comm_init(rank, world, ids[0])


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    problems = []
    quick = os.environ.get("TS2_TEST_QUICK") == "1"  # fp16 operands only, no capacity case
    for precision, tol in ((capi.PREC_F16, 1e-4), (capi.PREC_FP8, 0.25))[:1 if quick else 2]:
        spec = moe_spec(precision)
        mats = host.init_weights(spec, 5, select_std=1.0)
        batches = [host.synthetic_batch(spec, 6, 200, 300 + r) for r in range(world)]
        model = Model(spec, mats, batches[0].node_count, device=local)
        connect(model, rank, world)
        if os.environ.get("TS2_TEST_EP", "1") == "1":
            model.set_expert_parallel()
        model.set_batch(batches[rank])
        step0 = host.training_step(rate=0.01, iteration=0)
        model.backprop(step0, apply=True)
        w_ep = model.get_weights()
        print(f"rank {rank} precision {precision}: loss {model.avg_train_err():.6f}", flush=True)
        if rank == 0:
            single = Model(spec, mats, batches[0].node_count, device=local)
            for r in range(world):
                single.set_batch(batches[r])
                single.backprop(step0, apply=(r == world - 1))
                print(f"single, batch {r}: loss {single.avg_train_err():.6f}", flush=True)
            worst = 0.0
            for name, a, b, w0 in zip(spec.matrix_names(), w_ep, single.get_weights(), mats):
                upd = np.linalg.norm(b.astype(np.float64) - w0)
                d = np.linalg.norm(a.astype(np.float64) - b) / upd
                worst = max(worst, d)
                if not d <= tol:
                    problems.append(f"precision {precision}, {name}: the update of the expert-parallel step differs from that of "
                                    f"the accumulated single-process step by {d:.3e} (relative L2)")
            print(f"precision {precision}: largest relative L2 difference of an update {worst:.3e}", flush=True)
            single.close()
        model.backprop(host.training_step(rate=0.01, iteration=1), apply=False)
        for i in range(3):
            model.set_batch(batches[(rank + i) % world])
            model.backprop(host.training_step(rate=0.01, iteration=2 + i), apply=True)
        model.wait()
        sums = [float(np.abs(x.astype(np.float64)).sum()) for x in model.get_weights()]
        sums += [float(np.abs(x.astype(np.float64)).sum()) for x in model.get_momentum()]
        sums = torch.tensor(sums, dtype=torch.float64)
        gathered = [torch.zeros_like(sums) for _ in range(world)]
        dist.all_gather(gathered, sums)
        if not all(bool((g == gathered[0]).all()) for g in gathered):
            problems.append(f"precision {precision}: weights or momentum differ between ranks")
        if not np.isfinite(model.avg_train_err()):
            problems.append(f"precision {precision}: loss is not finite")
        model.close()
    if quick:
        dist.barrier()
        dist.destroy_process_group()
        if problems:
            raise SystemExit(f"rank {rank}: " + "; ".join(problems))
        return
    # capacity: with factor 1 and a router that sends every token to experts 0 and 1 (both on rank 0), rank 0 would
    # receive twice its own rows
    spec = moe_spec(capi.PREC_F16)
    mats = host.init_weights(spec, 5, select_std=0.0)
    for name, m in zip(spec.matrix_names(), mats):
        if name.endswith("moe.select"):
            m[:] = 0
            m[0, :] = 1.0
            m[1, :] = 0.5
    batch = host.synthetic_batch(spec, 6, 200, 300 + rank)
    model = Model(spec, mats, batch.node_count, device=local)
    connect(model, rank, world)
    model.set_expert_parallel(1.0)
    model.set_batch(batch)
    try:
        model.backprop(host.training_step(), apply=False)
        model.wait()
        problems.append("a step beyond the capacity of the received layout was not refused")
    except capi.Ts2Error as e:
        if e.code != capi.TS2_ERR_TOO_LARGE:
            problems.append(f"capacity: error {e.code} instead of TS2_ERR_TOO_LARGE")
    model.close()
    dist.barrier()
    dist.destroy_process_group()
    if problems:
        raise SystemExit(f"rank {rank}: " + "; ".join(problems))


if __name__ == "__main__":
    main()
