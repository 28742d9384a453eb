"""Two CPU ranks over gloo: the multi-GPU plumbing (sharding by global board index, statistics
all-reduce, max-over-ranks timing) without a GPU."""
from __future__ import annotations

import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    from connect6_b200 import shard
    from connect6_b200.boards import generate_planes
    r, w, _ = shard.init_from_env(backend="gloo")
    assert (r, w) == (rank, world)
    lo, hi = shard.shard_range(1000, r, w)
    planes = generate_planes(lo, hi - lo)
    stats = torch.zeros(9, dtype=torch.int64)
    stats[0] = hi - lo
    stats[1] = int(planes[:, 0].sum())
    stats[8] = rank + 1
    shard.reduce_rollout_stats(stats)
    slow = shard.max_over_ranks(10.0 * (rank + 1))
    shard.barrier()
    np.save(os.path.join(out_dir, f"rank{rank}.npy"), np.concatenate([stats.numpy(), [int(slow)]]))
    dist.destroy_process_group()


def test_two_rank_shard_and_reduce(tmp_path):
    from connect6_b200.boards import generate_planes
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    whole = generate_planes(0, 1000)
    for rank in range(world):
        got = np.load(tmp_path / f"rank{rank}.npy")
        assert got[0] == 1000                       # every board counted exactly once
        assert got[1] == int(whole[:, 0].sum())     # same boards as the unsharded generator
        assert got[8] == 3 and got[9] == 20         # sum and max over ranks


def test_single_process_is_a_no_op():
    from connect6_b200 import shard
    s = torch.arange(9, dtype=torch.int64)
    assert torch.equal(shard.reduce_rollout_stats(s.clone()), s)
    assert shard.max_over_ranks(3.5) == 3.5
    shard.barrier()
