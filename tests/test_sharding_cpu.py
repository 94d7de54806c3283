"""Multi-rank sharding logic on CPU: two gloo ranks each take their row shard of a W4G128
weight, run the matmul (here: the CPU oracle standing in for the device), all-gather, and
must reproduce the unsharded result bit for bit."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle_lib as ol
from __graft_entry__ import load_package

pkg = load_package()
N, K, M = 128, 256, 3


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    blocks = pkg.synth.bg128_weight(5, 1, N, K)
    x = pkg.synth.activations(6, 1, M, K)
    mine, rows, lo = pkg.shard.shard_blocks(blocks, N, K, rank, world)
    y_local = torch.from_numpy(ol.matmul_w4(np.ascontiguousarray(mine), rows, K, x))
    parts = [torch.zeros_like(y_local) for _ in range(world)]
    dist.all_gather(parts, y_local)
    y = torch.cat(parts, dim=1).numpy()
    if rank == 0:
        np.save(os.path.join(out_dir, "y.npy"), y)
    dist.destroy_process_group()


def test_row_sharded_matmul_world2(tmp_path):
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    y = np.load(tmp_path / "y.npy")
    blocks = pkg.synth.bg128_weight(5, 1, N, K)
    x = pkg.synth.activations(6, 1, M, K)
    assert y.tobytes() == ol.matmul_w4(blocks, N, K, x).tobytes()


def test_shard_ranges():
    assert pkg.shard.row_range(9728, 3, 8) == (3648, 4864)
    with pytest.raises(ValueError):
        pkg.shard.row_range(9728 + 8, 0, 8)
    blocks = pkg.synth.bg128_weight(5, 2, 64, 256)
    parts = [pkg.shard.shard_blocks(blocks, 64, 256, r, 4)[0] for r in range(4)]
    assert np.concatenate(parts).tobytes() == blocks.tobytes()
    assert pkg.shard.expert_range(128, 7, 8) == (112, 128)
    with pytest.raises(ValueError):
        pkg.shard.expert_range(128, 0, 3)
