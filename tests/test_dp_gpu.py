"""Data-parallel step on two GPUs through NCCL (reduce-scatter per bucket queued during the backward pass, optimizer
on each rank's parts, all-gather of the quantized weights): equal to one process with the summed gradient, and the
ranks stay bit-identical (tests/dp_two_ranks.py); expert parallel on top of it (tests/ep_two_ranks.py).  Needs two
GPUs; skipped otherwise."""
import os
import subprocess
import sys

import pytest

from tscale2_b200 import capi

pytestmark = pytest.mark.gpu


def test_two_ranks_stay_identical():
    lib = capi.load_library()
    if lib.ts2_device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29517", os.path.join(here, "dp_two_ranks.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


def test_expert_parallel_equals_one_process():
    lib = capi.load_library()
    if lib.ts2_device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29519", os.path.join(here, "ep_two_ranks.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
