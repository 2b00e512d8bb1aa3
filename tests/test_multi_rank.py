"""Multi-rank host logic on CPU: two gloo ranks shard a batch, each evaluates its chunk
(here with the CPU oracle standing in for the device), and the optional gather
reassembles the outputs in batch order.  No collective touches the data path."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, fixture


def _worker(rank, world, port, total, result_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from conftest import load_oracle, load_package
    pkg, oracle = load_package(), load_oracle()
    dist.init_process_group("gloo", rank=rank, world_size=world)
    param, bin_ = fixture("convolution")
    x = np.random.default_rng(42).standard_normal((total, 1, 4, 4)).astype(np.float32)  # same on every rank
    begin, end = pkg.shard_range(total, world, rank)
    model = oracle.Model(param, bin_)
    local = np.stack([model.run([x[i]])[0] for i in range(begin, end)]) if end > begin else np.zeros((0, 2, 4, 4), np.float32)
    gathered = pkg.gather_outputs(torch.from_numpy(local), total)
    if rank == 0:
        full = np.stack([model.run([xi])[0] for xi in x])
        np.save(result_path, np.array([np.array_equal(gathered.numpy(), full), gathered.shape[0] == total]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("total", [7, 8, 1])
def test_two_ranks_shard_and_gather(tmp_path, total):
    port = 29500 + (os.getpid() + total) % 2000
    out = str(tmp_path / "ok.npy")
    mp.spawn(_worker, args=(2, port, total, out), nprocs=2, join=True)
    ok = np.load(out)
    assert ok.all()
