"""Data-parallel contract of the engine on CPU ranks (gloo, world size 2): every rank
back-propagates its own batch, the flat fp32 gradient (matrices concatenated in C-ABI order) is
SUMMED across ranks, and every rank applies the same optimizer step to the same weights — which
must equal one process that sums the two gradients itself.  The GPU engine does the same with
ncclAllReduce on its flat gradient buffer (csrc/model.cu apply())."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tscale2_b200 import host


def _spec():
    return host.ModelSpec(dim=128, head_count=1, ffn_tiles=1, vocab=64, attention_widths=[16]).add_blocks(1)


def _rank_batch(spec, rank):
    # same rule as bench.py: the batch seed depends on the rank, the weights do not
    return host.synthetic_batch(spec, 2, 16, 1000 + rank)


def _flat(mats):
    return np.concatenate([m.reshape(-1) for m in mats])


def _worker(rank, world, port, out_dir):
    import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["OMP_NUM_THREADS"] = "1"
    dist.init_process_group("gloo", rank=rank, world_size=world)
    orc = oracle.Oracle("port")
    spec = _spec()
    mats = host.init_weights(spec, 1000)
    res = orc.backprop(spec, mats, _rank_batch(spec, rank), oracle.QUANT_HALF)
    flat = torch.from_numpy(_flat(res["grads"]).copy())
    dist.all_reduce(flat, op=dist.ReduceOp.SUM)
    step = host.training_step(rate=0.01, iteration=2)
    new = []
    off = 0
    for i, w in enumerate(mats):
        g = flat[off:off + w.size].numpy().reshape(w.shape)
        off += w.size
        n_disp = w.shape[0] if i < 2 else 1
        new.append(orc.apply_gradient(w, np.zeros_like(w), g, np.zeros(n_disp, np.float32), 0.0, 1.0, step)[0])
    np.save(os.path.join(out_dir, f"rank{rank}.npy"), _flat(new))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_equal_one_process_with_summed_gradient(tmp_path, oracle_port):
    import oracle
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.start_processes(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True, start_method="spawn")
    spec = _spec()
    mats = host.init_weights(spec, 1000)
    grads = [oracle_port.backprop(spec, mats, _rank_batch(spec, r), oracle.QUANT_HALF)["grads"] for r in range(2)]
    assert not np.array_equal(_flat(grads[0]), _flat(grads[1])), "ranks must see different batches"
    step = host.training_step(rate=0.01, iteration=2)
    ref = []
    for i, w in enumerate(mats):
        n_disp = w.shape[0] if i < 2 else 1
        ref.append(oracle_port.apply_gradient(w, np.zeros_like(w), grads[0][i] + grads[1][i], np.zeros(n_disp, np.float32), 0.0, 1.0,
                                              step)[0])
    ref = _flat(ref)
    r0, r1 = np.load(tmp_path / "rank0.npy"), np.load(tmp_path / "rank1.npy")
    assert np.array_equal(r0, r1), "replicated optimizer: both ranks hold identical weights after the step"
    assert np.allclose(r0, ref, rtol=0, atol=1e-7)
