"""Expert-parallel exchange of the mixture-of-experts layers on CPU: the plan the CUDA library computes on the host
(ts2_moe_exchange_plan - the same function ts2_backprop calls once per layer) checked for any world size, and carried
out by two gloo ranks with send / recv in the engine's order (what runs on the GPU in place of the gloo calls is
ncclSend / ncclRecv on the same blocks, csrc/model.cu ep_exchange(); the two-GPU test is tests/test_dp_gpu.py)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tscale2_b200 import host


def pad(n):
    return (n + 127) // 128 * 128


def own_rows(rank, counts):
    """This rank's (token, choice) rows sorted by expert, segments padded to 128: row value = (rank, expert, index)."""
    E = counts.shape[1]
    seg = np.concatenate([[0], np.cumsum([pad(c) for c in counts[rank]])])
    rows = np.full((seg[-1], 3), -1, np.int64)
    for e in range(E):
        n = counts[rank, e]
        rows[seg[e]:seg[e] + n] = np.stack([np.full(n, rank), np.full(n, e), np.arange(n)], 1)
    return rows, seg


@pytest.mark.parametrize("world,E,seed", [(2, 4, 0), (2, 32, 1), (4, 32, 2), (8, 32, 3), (8, 8, 4), (1, 4, 5)])
def test_plan_places_every_row_with_its_owner(world, E, seed):
    rng = np.random.default_rng(seed)
    counts = rng.integers(0, 700, (world, E)).astype(np.int32)
    counts[rng.random((world, E)) < 0.2] = 0  # experts nobody chose on some rank
    plans = [host.moe_exchange_plan(world, r, counts) for r in range(world)]
    per = E // world
    received = []
    for r, p in enumerate(plans):
        rows, seg = own_rows(r, counts)
        assert np.array_equal(p["own_seg"], seg)
        # the received layout: local experts only, padded to 128, sources in rank order
        x = np.full((p["x_seg"][-1], 3), -1, np.int64)
        assert p["x_seg"][-1] % 128 == 0 and p["x_seg"][-1] <= p["max_x_rows"]
        for e in range(E):
            total = counts[:, e].sum() if e // per == r else 0
            assert p["x_valid"][e] == total and p["x_seg"][e + 1] - p["x_seg"][e] == pad(total)
        received.append(x)
    assert plans[0]["max_x_rows"] == max(p["x_seg"][-1] for p in plans)
    # carry the plan out: every block a rank sends is a block its peer expects, in the same order
    for a in range(world):
        rows_a, _ = own_rows(a, counts)
        for b in range(world):
            sends = [m for m in plans[a]["out"] if m[0] == b]
            recvs = [m for m in plans[b]["recv"] if m[0] == a]
            assert len(sends) == len(recvs)
            for s, v in zip(sends, recvs):
                assert s[3] == v[3] and s[2] == v[2], "both sides agree on the size and the place of a block"
                if a == b:
                    assert v[1] == s[1]
                received[b][v[2]:v[2] + v[3]] = rows_a[s[1]:s[1] + s[3]]
    for r, p in enumerate(plans):
        x = received[r]
        for e in range(E):
            seg = x[p["x_seg"][e]:p["x_seg"][e + 1]]
            n = p["x_valid"][e]
            assert np.all(seg[n:] == -1), "padding stays untouched"
            want = np.concatenate([np.stack([np.full(c, s), np.full(c, e), np.arange(c)], 1) for s, c in enumerate(counts[:, e])]) \
                if n else np.zeros((0, 3), np.int64)
            assert np.array_equal(seg[:n], want), "an expert's rows: all ranks' rows for it, in rank order, each in its own order"


def _exchange(plan, rank, to_owner, own, x):
    """The engine's order: blocks to send in expert order, then blocks to receive; gloo needs the two sides interleaved
    without deadlock, so the sends are posted first (isend) like NCCL's grouped calls."""
    reqs = []
    for peer, own_row, x_row, rows in plan["recv"]:
        if peer == rank:
            if to_owner:
                x[x_row:x_row + rows] = own[own_row:own_row + rows]
            else:
                own[own_row:own_row + rows] = x[x_row:x_row + rows]
    for peer, own_row, x_row, rows in plan["out"]:
        if peer != rank:
            blk = own[own_row:own_row + rows]
            reqs.append(dist.isend(blk.clone(), peer) if to_owner else dist.irecv(blk, peer))
    for peer, own_row, x_row, rows in plan["recv"]:
        if peer != rank:
            blk = x[x_row:x_row + rows]
            reqs.append(dist.irecv(blk, peer) if to_owner else dist.isend(blk.clone(), peer))
    for q in reqs:
        q.wait()


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    E, D = 8, 16
    rng = np.random.default_rng(100 + rank)
    mine = torch.from_numpy(rng.integers(0, 300, E).astype(np.int32))
    gathered = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)  # the per-expert row counts of all ranks (ncclAllGather on the GPU)
    counts = torch.stack(gathered).numpy()
    plan = host.moe_exchange_plan(world, rank, counts)
    rows, seg = own_rows(rank, counts)
    own = torch.zeros(seg[-1], D)
    valid = rows[:, 0] >= 0
    own[valid] = torch.from_numpy(rng.standard_normal((int(valid.sum()), D)).astype(np.float32))
    x = torch.full((int(plan["x_seg"][-1]), D), float("nan"))
    _exchange(plan, rank, True, own, x)
    # the owner's work on the rows of its experts: here y = 2 x + expert index
    y = torch.full_like(x, float("nan"))
    for e in range(E):
        a, n = int(plan["x_seg"][e]), int(plan["x_valid"][e])
        y[a:a + n] = 2 * x[a:a + n] + e
    back = torch.zeros_like(own)
    _exchange(plan, rank, False, back, y)
    want = torch.zeros_like(own)
    for e in range(E):
        a, n = int(seg[e]), int(counts[rank, e])
        want[a:a + n] = 2 * own[a:a + n] + e
    ok = bool(torch.equal(back, want)) and not bool(torch.isnan(back).any())
    np.save(os.path.join(out_dir, f"ok{rank}.npy"), np.array([ok, int(valid.sum())]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_send_rows_to_the_owners_and_get_results_back(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.start_processes(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True, start_method="spawn")
    for r in range(2):
        ok, n = np.load(tmp_path / f"ok{r}.npy")
        assert ok and n > 0
