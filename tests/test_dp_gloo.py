"""Data-parallel contract of the engine on CPU ranks (gloo, world size 2), driven by the engine's own layout of the
exchange (ts2_dp_layout, computed by the CUDA library without a device): every rank back-propagates its own batch
(CPU oracle), lays its gradient out in the engine's flat padded buffer, the buckets are reduce-scattered onto the
parts the layout assigns to each rank, each rank keeps only its parts, and an all-gather of the parts must reproduce
the gradient that one process gets by summing the two gradients itself; the optimizer step on it then matches too.
What runs on the GPU in place of the gloo calls is ncclReduceScatter / ncclAllGather on the same offsets
(csrc/model.cu reduce_matrices(), apply()); the two-GPU test of that is tests/test_dp_gpu.py."""
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


def _to_flat(mats, layout):
    mo, bo, be, _ = layout
    flat = np.zeros(int(bo[-1] + be[-1]), np.float32)
    for m, off in zip(mats, mo):
        flat[off:off + m.size] = m.reshape(-1)
    return flat


def _from_flat(flat, shapes, layout):
    return [flat[off:off + y * x].reshape(y, x).copy() for (y, x), off in zip(shapes, layout[0])]


def test_layout_tiles_every_bucket_for_every_world_size():
    spec = host.ModelSpec(dim=256, head_count=2, ffn_tiles=4, vocab=515 * 32, attention_widths=[64]).add_blocks(2)
    mo, bo, be, bf = host.dp_layout(spec)
    shapes = spec.matrix_shapes()
    assert list(bf) == [0, 1, 2, 7, 10, 15] and len(bo) == 2 + len(spec.layers)
    assert bo[0] == 0 and all(bo[i] + be[i] == bo[i + 1] for i in range(len(bo) - 1)), "buckets are contiguous"
    for i, ((y, x), off) in enumerate(zip(shapes, mo)):
        b = max(k for k in range(len(bf)) if bf[k] <= i)
        assert bo[b] <= off and off + y * x <= bo[b] + be[b], "a matrix lies inside its bucket"
        if i + 1 < len(mo) and (i + 1) not in bf:
            assert mo[i + 1] == off + y * x, "matrices of a bucket are packed"
    for world in (1, 2, 4, 8):
        assert all(e % (4 * world) == 0 for e in be), "every rank's part is a whole number of 16-byte vectors"


def _worker(rank, world, port, out_dir):
    import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["OMP_NUM_THREADS"] = "1"
    dist.init_process_group("gloo", rank=rank, world_size=world)
    orc = oracle.Oracle("port")
    spec = _spec()
    layout = host.dp_layout(spec)
    _, bo, be, _ = layout
    mats = host.init_weights(spec, 1000)
    res = orc.backprop(spec, mats, _rank_batch(spec, rank), oracle.QUANT_HALF)
    flat = torch.from_numpy(_to_flat(res["grads"], layout))
    owned = torch.zeros_like(flat)  # what this rank holds after the exchange: only its parts
    for off, n in zip(bo, be):
        part = int(n) // world
        out = torch.empty(part)
        dist.reduce_scatter(out, [flat[off + r * part:off + (r + 1) * part].clone() for r in range(world)], op=dist.ReduceOp.SUM)
        owned[off + rank * part:off + (rank + 1) * part] = out
    # all-gather of the parts (the engine gathers the requantized weights this way; here: the summed gradient itself)
    full = torch.zeros_like(flat)
    for off, n in zip(bo, be):
        part = int(n) // world
        pieces = [torch.empty(part) for _ in range(world)]
        dist.all_gather(pieces, owned[off + rank * part:off + (rank + 1) * part].clone())
        full[off:off + int(n)] = torch.cat(pieces)
    np.save(os.path.join(out_dir, f"grad{rank}.npy"), full.numpy())
    np.save(os.path.join(out_dir, f"owned{rank}.npy"), owned.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_equal_one_process_with_summed_gradient(tmp_path, oracle_port):
    import oracle
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.start_processes(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True, start_method="spawn")
    spec = _spec()
    layout = host.dp_layout(spec)
    shapes = spec.matrix_shapes()
    mats = host.init_weights(spec, 1000)
    grads = [oracle_port.backprop(spec, mats, _rank_batch(spec, r), oracle.QUANT_HALF)["grads"] for r in range(2)]
    assert not np.array_equal(_to_flat(grads[0], layout), _to_flat(grads[1], layout)), "ranks must see different batches"
    want = _to_flat([a + b for a, b in zip(grads[0], grads[1])], layout)
    g0, g1 = np.load(tmp_path / "grad0.npy"), np.load(tmp_path / "grad1.npy")
    assert np.array_equal(g0, g1), "after the all-gather both ranks hold the same buffer"
    assert np.array_equal(g0, want), "reduce-scatter onto the layout's parts + all-gather = the summed gradient"
    o0, o1 = np.load(tmp_path / "owned0.npy"), np.load(tmp_path / "owned1.npy")
    assert not np.any((o0 != 0) & (o1 != 0)), "no element is owned by both ranks"
    assert np.array_equal(o0 + o1, want), "every element is owned by one of them"
    # the optimizer step on the exchanged gradient equals the step on the locally summed one
    step = host.training_step(rate=0.01, iteration=2)
    for i, (w, g) in enumerate(zip(mats, _from_flat(g0, shapes, layout))):
        n_disp = w.shape[0] if i < 2 else 1
        a = oracle_port.apply_gradient(w, np.zeros_like(w), g, np.zeros(n_disp, np.float32), 0.0, 1.0, step)[0]
        b = oracle_port.apply_gradient(w, np.zeros_like(w), grads[0][i] + grads[1][i], np.zeros(n_disp, np.float32), 0.0, 1.0, step)[0]
        assert np.array_equal(a, b)
