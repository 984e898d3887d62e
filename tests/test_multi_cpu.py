"""CPU tests of the multi-GPU path: the striping of lists over ranks, and the whole exchange protocol run as
two gloo ranks with the CPU checker standing in for the CUDA engine."""
import os
import subprocess
import sys

import numpy as np
import pytest

from paraselect_b200.multi import owned_mask_rows, stripe_layout

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_stripes_partition_every_list(world):
    rng = np.random.default_rng(world)
    sizes = np.concatenate([rng.integers(0, 50, 40), [0, 1, 5000, 7, 40000, 100001]])
    offsets = np.zeros(sizes.size + 1, np.int64)
    offsets[1:] = np.cumsum(sizes)
    seen = np.zeros(offsets[-1], np.int32)
    for r in range(world):
        gb, loff = stripe_layout(offsets, r, world)
        length = loff[1:] - loff[:-1]
        assert np.all(gb >= offsets[:-1]) and np.all(gb + length <= offsets[1:])
        big = sizes >= world * 4096
        assert np.all(length[big] >= sizes[big] // world) and np.all(length[big] <= sizes[big] // world + 1)
        assert np.all((length[~big] == 0) | (length[~big] == sizes[~big]))
        mask = owned_mask_rows(gb, loff, 0, int(offsets[-1]))
        assert mask.sum() == loff[-1]
        seen += mask
    assert np.all(seen == 1)  # every row belongs to exactly one rank


def test_two_gloo_ranks_reproduce_the_single_rank_search():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29577", os.path.join(ROOT, "tests", "multi_cpu_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "MULTI_OK" in r.stdout
