"""Run by test_dp_gpu.py under torchrun, one process per GPU.  Data parallel = reduce-scatter of the gradient buckets
during the backward pass, optimizer and requantiser on each rank's parts, all-gather of the quantized weights:
  * after one applied step the weights equal those of ONE process that accumulates the ranks' batches and applies once
    (the sum of two gradients is exact in either order, and every sum inside a rank has a fixed order: bit for bit);
  * after more steps, one of them accumulated and not applied, every rank still holds bit-identical weights, momentum
    and quantized weights, and the loss is finite."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tscale2_b200 import capi, host  # noqa: E402
from tscale2_b200.model import Model, comm_unique_id  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    spec = host.ModelSpec(dim=256, head_count=2, ffn_tiles=8, vocab=4096, attention_widths=[256],
                          precision=capi.PREC_FP8).add_blocks(3)
    mats = host.init_weights(spec, 3)
    batches = [host.synthetic_batch(spec, 8, 256, 100 + r) for r in range(world)]
    model = Model(spec, mats, batches[0].node_count, device=local)
    ids = [comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    model.comm_init(rank, world, ids[0])
    model.set_batch(batches[rank])
    step0 = host.training_step(rate=0.01, iteration=0)
    model.backprop(step0, apply=True)
    w_dp = model.get_weights()  # collective: brings the other ranks' parts of the fp32 master weights in
    problems = []
    if rank == 0:
        single = Model(spec, mats, batches[0].node_count, device=local)
        for r in range(world):
            single.set_batch(batches[r])
            single.backprop(step0, apply=(r == world - 1))
        for name, a, b in zip(spec.matrix_names(), w_dp, single.get_weights()):
            d = float(np.abs(a.astype(np.float64) - b).max())
            if d > 0.0:
                problems.append(f"{name}: data-parallel step differs from the accumulated single-process step by {d}")
        single.close()
    # one accumulated (not applied) step, then applied ones: the exchange must cover the accumulated gradient too
    model.backprop(host.training_step(rate=0.01, iteration=1), apply=False)
    for i in range(3):
        model.backprop(host.training_step(rate=0.01, iteration=2 + i), apply=True)
    model.wait()
    sums = [float(np.abs(x.astype(np.float64)).sum()) for x in model.get_weights()]
    sums += [float(np.abs(x.astype(np.float64)).sum()) for x in model.get_momentum()]
    sums += [float(model.get_fast_weights(i)[0].astype(np.float64).sum()) for i in (0, 1, 2, 6, 7, 9)]
    sums = torch.tensor(sums, dtype=torch.float64)
    gathered = [torch.zeros_like(sums) for _ in range(world)]
    dist.all_gather(gathered, sums)
    err = model.avg_train_err()
    if not all(bool((g == gathered[0]).all()) for g in gathered):
        problems.append("weights, momentum or quantized weights differ between ranks")
    if not np.isfinite(err):
        problems.append(f"loss {err} is not finite")
    dist.destroy_process_group()
    if problems:
        raise SystemExit(f"rank {rank}: " + "; ".join(problems))


if __name__ == "__main__":
    main()
