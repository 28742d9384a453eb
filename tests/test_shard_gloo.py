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
    # the ring-buffered asynchronous reducer gives the same sums, step after step
    red = shard.RolloutStatsReducer("cpu", depth=2)
    for t in range(5):
        buf = red.buffer()
        buf.zero_()
        buf[0] = (rank + 1) * (t + 1)
        red.submit()
    assert int(red.drain()[0]) == 3 * 5
    # default random stream of the drop-in samplers: same key on every rank after the same
    # torch.manual_seed, but a different first board index
    from connect6_b200 import selfplay
    torch.manual_seed(1234)
    seed, base = selfplay.default_stream()
    np.save(os.path.join(out_dir, f"stream{rank}.npy"), np.array([seed, base], dtype=np.uint64))
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
    s0, s1 = np.load(tmp_path / "stream0.npy"), np.load(tmp_path / "stream1.npy")
    assert s0[0] == s1[0] == 1234                   # the key follows torch.manual_seed on every rank
    assert s0[1] == 0 and s1[1] == 1 << 40          # ranks never share a (key, offset, board) triple


def test_default_sampler_stream_on_one_process():
    from connect6_b200 import selfplay
    torch.manual_seed(99)
    assert selfplay.default_stream() == (99, 0)
    selfplay.set_seed(5, board_index0=77)
    assert selfplay.default_stream() == (5, 77)
    selfplay.set_seed(None)
    torch.manual_seed(100)
    assert selfplay.default_stream() == (100, 0)


def test_single_process_is_a_no_op():
    from connect6_b200 import shard
    s = torch.arange(9, dtype=torch.int64)
    assert torch.equal(shard.reduce_rollout_stats(s.clone()), s)
    assert shard.max_over_ranks(3.5) == 3.5
    shard.barrier()
