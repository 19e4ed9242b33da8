"""Run by test_dp_gpu.py under torchrun, one process per GPU: three applied steps on different batches per rank;
with the gradient summed over the ranks every rank must end with bit-identical weights."""
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
    batch = host.synthetic_batch(spec, 8, 256, 100 + rank)
    model = Model(spec, mats, batch.node_count, device=local)
    ids = [comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    model.comm_init(rank, world, ids[0])
    model.set_batch(batch)
    # one accumulated (not applied) step first: the sum over ranks must cover it too
    model.backprop(host.training_step(rate=0.01, iteration=0), apply=False)
    for i in range(3):
        model.backprop(host.training_step(rate=0.01, iteration=i), apply=True)
    model.wait()
    sums = torch.tensor([float(np.abs(x.astype(np.float64)).sum()) for x in model.get_weights()], dtype=torch.float64)
    gathered = [torch.zeros_like(sums) for _ in range(world)]
    dist.all_gather(gathered, sums)
    err = model.avg_train_err()
    ok = all(bool((g == gathered[0]).all()) for g in gathered) and np.isfinite(err)
    dist.destroy_process_group()
    if not ok:
        raise SystemExit(f"rank {rank}: weights differ between ranks or loss {err} is not finite")


if __name__ == "__main__":
    main()
